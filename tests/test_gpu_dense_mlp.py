"""Dense W4A16 SwiGLU MLP (the model's first, non-MoE layers) on the grouped kernels: the
intermediate dim is cut into 2048-column slices that run as experts every token visits with
weight 1.  Checked against the oracle's int4 GEMM (the reference's gemm_w4a16 arithmetic,
cuda/int4_gemm.cu:15-48 / src/tensor.cpp:53-63) chained as gate, up, silu*up, down."""
import numpy as np
import pytest

import oracle
from glmserve_b200.quant import quantize_w4_np, round_bf16_np
from helpers import assert_layer_close, bf16_tensor

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _dense_case(H, I, n, seed):
    rng = np.random.default_rng(seed)
    mk = lambda r, c: quantize_w4_np((rng.standard_normal((r, c)) * 0.02).astype(np.float32), 128)
    gq, gs = mk(I, H)
    uq, us = mk(I, H)
    dq, ds = mk(H, I)
    gs, us, ds = (s.astype(np.float16).astype(np.float32) for s in (gs, us, ds))
    x = round_bf16_np(rng.standard_normal((n, H)).astype(np.float32))
    return x, (gq, gs, uq, us, dq, ds)


def _oracle_dense(x, w):
    gq, gs, uq, us, dq, ds = w
    g = oracle.gemm_w4a16(x, gq, gs, 128)
    u = oracle.gemm_w4a16(x, uq, us, 128)
    h = (g / (np.float32(1) + np.exp(-g, dtype=np.float32))).astype(np.float32) * u
    return oracle.gemm_w4a16(h.astype(np.float32), dq, ds, 128)


@pytest.mark.parametrize("H,I,n,path_name", [(1024, 4096, 5, "PATH_DECODE"), (1024, 4096, 70, "PATH_DECODE"),
                                             (1024, 4096, 300, "PATH_PREFILL"), (1024, 2048, 9, "PATH_DECODE"),
                                             (6144, 12288, 8, "PATH_DECODE")])
def test_dense_mlp_matches_oracle(H, I, n, path_name):
    from glmserve_b200 import ops
    dev = torch.device("cuda:0")
    x, w = _dense_case(H, I, n, seed=H + I + n)
    t = [torch.from_numpy(a).to(dev) for a in w]
    mlp = ops.DenseMLP(t[0], t[1].half(), t[2], t[3].half(), t[4], t[5].half())
    out = mlp.forward(bf16_tensor(x, dev), path=getattr(ops, path_name))
    assert mlp.layer.status() == 0
    assert_layer_close(out.cpu().numpy(), _oracle_dense(x, w), f"dense mlp H={H} I={I} n={n}")
    again = mlp.forward(bf16_tensor(x, dev), path=getattr(ops, path_name))
    assert torch.equal(out, again)


def test_fixed_routing_reports_its_routing():
    from glmserve_b200 import ops
    dev = torch.device("cuda:0")
    x, w = _dense_case(1024, 4096, 3, seed=5)
    t = [torch.from_numpy(a).to(dev) for a in w]
    mlp = ops.DenseMLP(t[0], t[1].half(), t[2], t[3].half(), t[4], t[5].half())
    n = 3
    xb = bf16_tensor(x, dev)
    out = torch.empty((n, 1024), dtype=torch.float32, device=dev)
    ids = torch.empty((n, 2), dtype=torch.int32, device=dev)
    wts = torch.empty((n, 2), dtype=torch.float32, device=dev)
    ws = mlp.layer._workspace(n)
    import ctypes as C
    from glmserve_b200._lib import lib, check
    check(lib().gsb_moe_layer_forward(mlp.layer._h, C.c_void_p(xb.data_ptr()), n, C.c_void_p(out.data_ptr()),
                                      C.c_void_p(ws.data_ptr()), C.c_size_t(ws.numel()), ops.PATH_DECODE, None,
                                      C.c_void_p(ids.data_ptr()), C.c_void_p(wts.data_ptr()), None), "forward")
    assert ids.cpu().tolist() == [[0, 1]] * n and wts.cpu().tolist() == [[1.0, 1.0]] * n

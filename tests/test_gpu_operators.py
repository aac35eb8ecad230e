"""Parity of the operator-surface entry points (the reference's cuda/kernels.cuh names)
against the CPU oracle, through the C ABI."""
import os

import numpy as np
import pytest

import oracle
from glmserve_b200.quant import dequantize_w4_np, prepack_np, quantize_w4_np, round_bf16_np
from glmserve_b200.synth import CONFIGS, make_layer_np, make_x_np
from helpers import assert_layer_close, load_tiny

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def _t(a, dev, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    return t.to(dtype) if dtype is not None else t


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_router_golden_ids_bit_exact(golden_dir, dev, tag):
    from glmserve_b200 import ops
    z = np.load(os.path.join(golden_dir, "router_cases.npz"))
    ids, w = ops.moe_router(_t(z[f"{tag}_logits"], dev), _t(z[f"{tag}_bias"], dev), int(z[f"{tag}_topk"]))
    assert np.array_equal(ids.cpu().numpy(), z[f"{tag}_ids"])
    np.testing.assert_allclose(w.cpu().numpy(), z[f"{tag}_w"], rtol=0, atol=1e-4)


@pytest.mark.parametrize("n,E,k,bias,norm", [(2048, 256, 8, True, True), (257, 160, 6, False, False),
                                             (64, 16, 4, True, True), (3, 1000, 32, True, True),
                                             (1, 8, 8, False, True)])
def test_router_vs_oracle_bit_exact(dev, n, E, k, bias, norm):
    from glmserve_b200 import ops
    rng = np.random.default_rng(n + E)
    logits = (rng.standard_normal((n, E)) * 1.6).astype(np.float32)
    b = (0.01 * rng.standard_normal(E)).astype(np.float32) if bias else None
    ids_o, w_o, ties = oracle.router(logits, b, k, norm, 2.5)
    assert ties == 0
    ids, w = ops.moe_router(_t(logits, dev), None if b is None else _t(b, dev), k, norm, 2.5)
    assert np.array_equal(ids.cpu().numpy(), ids_o)
    np.testing.assert_allclose(w.cpu().numpy(), w_o, rtol=0, atol=2e-7 * 2.5)


def test_router_ties_and_empty(dev):
    from glmserve_b200 import ops
    ids, w = ops.moe_router(torch.zeros((2, 40), device=dev), None, 5)
    assert ids.cpu().tolist() == [[0, 1, 2, 3, 4]] * 2
    np.testing.assert_allclose(w.cpu().numpy(), 0.5, atol=1e-6)
    ids, w = ops.moe_router(torch.zeros((0, 40), device=dev), None, 5)
    assert ids.shape == (0, 5)


@pytest.mark.parametrize("n,E,k", [(64, 256, 8), (1, 256, 8), (37, 16, 4), (8192, 256, 8), (1000, 7, 3), (5, 1024, 2)])
def test_dispatch_bit_exact(dev, n, E, k):
    from glmserve_b200 import ops
    rng = np.random.default_rng(n * 7 + E)
    if n >= 1000:   # skewed loads, some experts empty
        p = rng.dirichlet(np.full(E, 0.3))
        ids = np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(n)]).astype(np.int32)
    else:
        ids = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    offs_o, tok_o, row_o = oracle.dispatch(ids, E)
    offs, tok, row = ops.moe_dispatch(_t(ids, dev), E)
    assert np.array_equal(offs.cpu().numpy(), offs_o)
    assert np.array_equal(tok.cpu().numpy(), tok_o)
    assert np.array_equal(row.cpu().numpy(), row_o)


@pytest.mark.parametrize("n,E,k", [(8192, 256, 8), (1100, 256, 8), (3000, 7, 3), (4097, 1024, 2), (20000, 33, 5)])
def test_dispatch_many_blocks_bit_exact(dev, n, E, k):
    """Above 8192 slots the dispatch with scratch runs one block per 4096 slots; the permutation
    is the stable sort's all the same (ragged last block, empty experts, skewed loads)."""
    from glmserve_b200 import ops
    rng = np.random.default_rng(n + 13 * E)
    p = rng.dirichlet(np.full(E, 0.3))
    ids = np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(n)]).astype(np.int32)
    offs_o, tok_o, row_o = oracle.dispatch(ids, E)
    offs, tok, row = ops.moe_dispatch_ws(_t(ids, dev), E)
    assert np.array_equal(offs.cpu().numpy(), offs_o)
    assert np.array_equal(tok.cpu().numpy(), tok_o)
    assert np.array_equal(row.cpu().numpy(), row_o)


def test_dispatch_empty(dev):
    from glmserve_b200 import ops
    offs, tok, row = ops.moe_dispatch(torch.zeros((0, 4), dtype=torch.int32, device=dev), 8)
    assert offs.cpu().tolist() == [0] * 9


def test_expert_ffn_w4a16_operator_tiny(golden_dir, dev):
    from glmserve_b200 import ops
    L = load_tiny(golden_dir)
    r = oracle.moe_layer_w4(L["x"], L)
    Lns = dict(L, sg_q=None, sg_sc=None, su_q=None, su_sc=None, sd_q=None, sd_sc=None)
    want = oracle.moe_experts_w4(L["x"], r["ids"], r["w"], Lns)
    got = ops.moe_expert_ffn_w4a16(_t(L["x"], dev), _t(r["ids"], dev), _t(r["w"], dev),
                                   _t(L["gate_q"], dev), _t(L["gate_sc"], dev), _t(L["up_q"], dev),
                                   _t(L["up_sc"], dev), _t(L["down_q"], dev), _t(L["down_sc"], dev), L["group"])
    assert_layer_close(got.cpu().numpy(), want, "moe_expert_ffn_w4a16")


def test_expert_ffn_w4a16_reference_tiny_checkpoint_shape(dev):
    """H=64, I=48, E=8, top-2, group 16: the shape of the reference's own W4 gate
    (tools/make_tiny_checkpoint.py:21-69, tests/test_w4_quantized.py)."""
    from glmserve_b200 import ops
    cfg = dict(H=64, E=8, topk=2, I=48, Is=48, group=16)
    L = make_layer_np(cfg, seed=5, shared=False)
    x = make_x_np(8, 64, seed=6)
    r = oracle.moe_layer_w4(x, L)
    got = ops.moe_expert_ffn_w4a16(_t(x, dev), _t(r["ids"], dev), _t(r["w"], dev), _t(L["gate_q"], dev),
                                   _t(L["gate_sc"], dev), _t(L["up_q"], dev), _t(L["up_sc"], dev),
                                   _t(L["down_q"], dev), _t(L["down_sc"], dev), 16)
    assert_layer_close(got.cpu().numpy(), r["out"], "tiny-checkpoint shape")


def test_expert_ffn_fp32_operator(dev):
    from glmserve_b200 import ops
    rng = np.random.default_rng(11)
    E, I, H, n, k = 4, 96, 160, 9, 2
    gw = (rng.standard_normal((E, I, H)) * 0.05).astype(np.float32)
    uw = (rng.standard_normal((E, I, H)) * 0.05).astype(np.float32)
    dw = (rng.standard_normal((E, H, I)) * 0.05).astype(np.float32)
    x = rng.standard_normal((n, H)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(n)]).astype(np.int32)
    w = rng.random((n, k)).astype(np.float32)
    want = np.zeros((n, H), np.float32)
    for t in range(n):
        for j in range(k):
            e = ids[t, j]
            g = oracle.linear(gw[e], x[t:t + 1])[0]
            u = oracle.linear(uw[e], x[t:t + 1])[0]
            h = (g / (1 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
            want[t] += w[t, j] * oracle.linear(dw[e], h[None])[0]
    got = ops.moe_expert_ffn(_t(x, dev), _t(ids, dev), _t(w, dev), _t(gw, dev), _t(uw, dev), _t(dw, dev))
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("n,inn,out,g,bias", [(5, 256, 40, 32, True), (1, 6144, 64, 128, False), (70, 128, 24, 16, False)])
def test_gemm_w4a16_operator(dev, n, inn, out, g, bias):
    from glmserve_b200 import ops
    rng = np.random.default_rng(inn + out)
    q, s = quantize_w4_np((rng.standard_normal((out, inn)) * 0.02).astype(np.float32), g)
    x = round_bf16_np(rng.standard_normal((n, inn)).astype(np.float32))
    b = rng.standard_normal(out).astype(np.float32) if bias else None
    want = oracle.gemm_w4a16(x, q, s, g, bias=b)
    got = ops.gemm_w4a16(_t(x, dev), _t(q, dev), _t(s, dev), g, None if b is None else _t(b, dev))
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-4, atol=1e-4)


def test_rmsnorm_silu_add_quantize(golden_dir, dev):
    from glmserve_b200 import ops
    z = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    got = ops.rmsnorm(_t(z["x"], dev), _t(z["w"], dev), float(z["eps"])).cpu().numpy()
    np.testing.assert_allclose(got, z["out_ref"], rtol=2e-7, atol=0)
    rng = np.random.default_rng(2)
    g = rng.standard_normal(1000).astype(np.float32) * 3
    u = rng.standard_normal(1000).astype(np.float32)
    want = (g / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32) * u
    np.testing.assert_allclose(ops.silu_mul(_t(g, dev), _t(u, dev)).cpu().numpy(), want, rtol=1e-6, atol=1e-7)
    y = _t(g, dev)
    ops.add_inplace(y, _t(u, dev))
    assert np.array_equal(y.cpu().numpy(), g + u)
    x = rng.standard_normal((3, 64)).astype(np.float32)
    xq, xs = ops.quantize_act_q8(_t(x, dev))
    amax = np.abs(x.reshape(3, 2, 32)).max(-1)
    np.testing.assert_allclose(xs.cpu().numpy(), amax / 127.0, rtol=1e-6)
    np.testing.assert_allclose(xq.cpu().numpy().reshape(3, 2, 32) * xs.cpu().numpy()[..., None],
                               x.reshape(3, 2, 32), atol=float(amax.max()) / 127.0 * 0.51)


def test_qgemm_family_reports_unsupported(dev):
    import ctypes as C
    from glmserve_b200._lib import lib
    assert lib().gsb_qtype_has_i8(12) == 0
    assert lib().gsb_gemm_q(12, None, None, None, None, C.c_int64(1), C.c_int64(256), C.c_int64(8),
                            C.c_int64(144), None) == 2


def test_invalid_arguments_are_rejected_before_launch(dev):
    import ctypes as C
    from glmserve_b200._lib import lib
    L = lib()
    assert L.gsb_moe_router(None, None, 4, 16, 2, 1, C.c_float(1.0), None, None, None) == 1
    assert L.gsb_moe_router(None, None, -1, 16, 2, 1, C.c_float(1.0), None, None, None) == 1
    x = torch.zeros((4, 16), device=dev)
    ids = torch.zeros((4, 2), dtype=torch.int32, device=dev)
    assert L.gsb_moe_router(C.c_void_p(x.data_ptr()), None, 4, 2048, 2, 1, C.c_float(1.0),
                            C.c_void_p(ids.data_ptr()), C.c_void_p(x.data_ptr()), None) == 2
    assert L.gsb_prepack_bytes(1, 33, 512) == 0


@pytest.mark.parametrize("pair", [True, False])
def test_prepack_matches_numpy_twin(dev, pair):
    from glmserve_b200 import ops
    rng = np.random.default_rng(3)
    E, rows, cols = 3, 64, 1024
    qa, sa = quantize_w4_np((rng.standard_normal((E, rows, cols)) * 0.02).astype(np.float32), 128)
    if pair:
        qb, sb = quantize_w4_np((rng.standard_normal((E, rows, cols)) * 0.02).astype(np.float32), 128)
        want = prepack_np(qa, sa, qb, sb)
        got = ops.prepack_gate_up(_t(qa, dev), _t(sa, dev, torch.float16), _t(qb, dev), _t(sb, dev, torch.float16))
        got32 = ops.prepack_gate_up(_t(qa, dev), _t(sa, dev), _t(qb, dev), _t(sb, dev))
    else:
        want = prepack_np(qa, sa)
        got = ops.prepack_down(_t(qa, dev), _t(sa, dev, torch.float16))
        got32 = ops.prepack_down(_t(qa, dev), _t(sa, dev))
    assert np.array_equal(got.cpu().numpy(), want)
    assert np.array_equal(got32.cpu().numpy(), want)


def _glm_dim_experts(E=8, topk=2, seed=31):
    cfg = dict(H=6144, E=E, topk=topk, I=2048, Is=2048, group=128)
    return make_layer_np(cfg, seed=seed, shared=False)


def test_expert_ffn_w4a16_operator_at_glm_dimensions(dev):
    """moe_expert_ffn_w4a16 with the reference's own signature (raw layout, fp32 activations and scales) at
    hidden 6144 / intermediate 2048, where the reference's kernel cannot launch (it asks for more than the
    48 KiB of shared memory a kernel gets without opting in, cuda/moe_expert.cu:232-243): first the
    direct-layout kernel, then - with the operator cache on - the tile-stream kernels behind the same call,
    for a decode-sized and a prefill-sized batch; the cached call repeats bit for bit."""
    from glmserve_b200 import ops
    L = _glm_dim_experts()
    args = [_t(L[k], dev) for k in ("gate_q", "gate_sc", "up_q", "up_sc", "down_q", "down_sc")]
    for n in (8, 600):
        x = make_x_np(n, L["H"], seed=n)
        rng = np.random.default_rng(n)
        ids = np.stack([rng.permutation(L["E"])[:L["topk"]] for _ in range(n)]).astype(np.int32)
        w = rng.random((n, L["topk"])).astype(np.float32)
        want = oracle.moe_experts_w4(x, ids, w, L)
        xt, it, wt = _t(x, dev), _t(ids, dev), _t(w, dev)
        if n == 8:
            assert ops.operator_cache_bytes() == 0
            direct = ops.moe_expert_ffn_w4a16(xt, it, wt, *args, L["group"])
            assert_layer_close(direct.cpu().numpy(), want, "direct-layout kernel at GLM dimensions")
        ops.operator_cache_enable(1 << 30)
        try:
            fast = ops.moe_expert_ffn_w4a16(xt, it, wt, *args, L["group"])
            assert ops.operator_cache_bytes() > 0
            assert_layer_close(fast.cpu().numpy(), want, f"cached tile-stream kernels, n={n}")
            again = ops.moe_expert_ffn_w4a16(xt, it, wt, *args, L["group"])
            assert torch.equal(fast, again)
        finally:
            ops.operator_cache_enable(0)
        assert ops.operator_cache_bytes() == 0


@pytest.mark.parametrize("n,inn,out,bias", [(8, 6144, 2048, False), (64, 2048, 6144, True), (5, 512, 256, True),
                                            (33, 1536, 128, False), (1, 1024, 6144, False)])
def test_gemm_w4a16_operator_cached_fast_path(dev, n, inn, out, bias):
    """gemm_w4a16 with the reference's signature through the operator cache: the matrix is packed like one
    expert's down projection and the rows run on the split-K kernel (2048-column stages, several units per
    stage for 512 / 1024 columns, the shared-memory variant otherwise)."""
    from glmserve_b200 import ops
    rng = np.random.default_rng(inn + out)
    q, s = quantize_w4_np((rng.standard_normal((out, inn)) * 0.02).astype(np.float32), 128)
    x = rng.standard_normal((n, inn)).astype(np.float32)
    b = rng.standard_normal(out).astype(np.float32) if bias else None
    want = oracle.gemm_w4a16(x, q, s, 128, b)
    ops.operator_cache_enable(1 << 28)
    try:
        got = ops.gemm_w4a16(_t(x, dev), _t(q, dev), _t(s, dev), 128, _t(b, dev) if bias else None)
        assert ops.operator_cache_bytes() > 0
        got2 = ops.gemm_w4a16(_t(x, dev), _t(q, dev), _t(s, dev), 128, _t(b, dev) if bias else None)
    finally:
        ops.operator_cache_enable(0)
    g = got.cpu().numpy()
    rel = float(np.linalg.norm(g - want) / np.linalg.norm(want))
    assert np.isfinite(g).all() and rel <= 1e-3, f"rel-L2 {rel:.2e}"   # activations rounded to fp16

"""W4 checkpoint written by the reference's converter -> glmserve_b200.checkpoint -> the native
layer, against the reference's own CPU output (GLM52Model::moe_mlp, stored in the fixture by
tests/golden/make_w4_checkpoint_fixture.py).  Group 16 and 48-wide experts: the direct-layout
kernels.  The layer keeps fp16 scales and a bf16 router weight; the reference keeps both in fp32,
which is inside the tolerance (and flips no routing decision on this input)."""
import os

import numpy as np
import pytest

from glmserve_b200.checkpoint import Checkpoint
from helpers import assert_layer_close, bf16_tensor

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_w4_ckpt")


def _to_torch(L, dev):
    out = {}
    for k, v in L.items():
        if isinstance(v, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(v)).to(dev)
            out[k] = t.half() if k.endswith("_sc") else t
        else:
            out[k] = v
    return out


def test_converted_checkpoint_layer_matches_reference_output():
    from glmserve_b200 import ops
    dev = torch.device("cuda:0")
    ck = Checkpoint(FIX)
    L = ck.load_moe_layer(2)
    e = np.load(os.path.join(FIX, "expected.npz"))
    layer = ops.MoELayer(_to_torch(L, dev))
    assert not layer.prepacked
    out = layer.forward(bf16_tensor(e["x"], dev), path=ops.PATH_DIRECT)
    assert_layer_close(out.cpu().numpy(), e["out_ref"], "tiny W4 checkpoint, layer 2")


def test_converted_checkpoint_dense_layer_operator():
    """Layer 0's dense MLP through the gemm_w4a16 operator chain (group 16)."""
    import oracle
    from glmserve_b200 import ops
    dev = torch.device("cuda:0")
    ck = Checkpoint(FIX)
    gq, gs, uq, us, dq, ds = (np.asarray(a) for a in ck.load_dense_mlp(0))
    rng = np.random.default_rng(7)
    x = rng.standard_normal((5, gq.shape[1] * 2)).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    g = ops.gemm_w4a16(t(x), t(gq), t(gs), 16)
    u = ops.gemm_w4a16(t(x), t(uq), t(us), 16)
    h = ops.silu_mul(g, u)
    y = ops.gemm_w4a16(h, t(dq), t(ds), 16)
    go, uo = oracle.gemm_w4a16(x, gq, gs, 16), oracle.gemm_w4a16(x, uq, us, 16)
    ho = (go / (np.float32(1) + np.exp(-go, dtype=np.float32))).astype(np.float32) * uo
    yo = oracle.gemm_w4a16(ho.astype(np.float32), dq, ds, 16)
    np.testing.assert_allclose(y.cpu().numpy(), yo, rtol=0, atol=2e-4)

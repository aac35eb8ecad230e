"""The CPU oracle against the golden vectors the reference produced (CPU only)."""
import os

import numpy as np
import pytest

import oracle
from glmserve_b200.quant import dequantize_w4_np, quantize_w4_np, round_bf16_np
from glmserve_b200.synth import CONFIGS, make_layer_np, make_x_np


def _load_layer(golden_dir):
    z = np.load(os.path.join(golden_dir, "tiny_layer.npz"))
    L = {k: z[k] for k in z.files}
    for k in ("H", "E", "topk", "I", "Is", "group"):
        L[k] = int(L[k])
    L["norm_topk"] = bool(L["norm_topk"])
    L["routed_scale"] = float(L["routed_scale"])
    return L


def test_layer_bit_equal_to_reference_moe_mlp(golden_dir):
    L = _load_layer(golden_dir)
    r = oracle.moe_layer_w4(L["x"], L)
    assert r["ties"] == 0
    assert np.array_equal(r["logits"], L["logits_ref"])       # linear_forward, bit for bit
    assert np.array_equal(r["out"], L["out_ref"])             # moe_mlp, bit for bit
    assert np.array_equal(r["ids"], L["ids_numpy"])           # numpy twin's selection
    np.testing.assert_allclose(r["w"], L["w_numpy"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(r["out"], L["out_numpy"], rtol=0, atol=1e-5)


def test_layer_is_thread_count_invariant(golden_dir):
    L = _load_layer(golden_dir)
    a = oracle.moe_layer_w4(L["x"], L, nthreads=1)["out"]
    b = oracle.moe_layer_w4(L["x"], L, nthreads=4)["out"]
    assert np.array_equal(a, b)


def test_fixture_inputs_regenerate_from_seed(golden_dir):
    L = _load_layer(golden_dir)
    G = make_layer_np(CONFIGS["tiny"], seed=1234)
    for k in ("gate_q", "gate_sc", "down_q", "sd_q", "router_w", "e_bias"):
        assert np.array_equal(G[k], L[k]), k
    assert np.array_equal(make_x_np(64, 256, seed=99), L["x"])


@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_router_cases(golden_dir, tag):
    z = np.load(os.path.join(golden_dir, "router_cases.npz"))
    ids, w, ties = oracle.router(z[f"{tag}_logits"], z[f"{tag}_bias"], int(z[f"{tag}_topk"]))
    assert ties == 0
    assert np.array_equal(ids, z[f"{tag}_ids"])
    np.testing.assert_allclose(w, z[f"{tag}_w"], rtol=0, atol=1e-4)  # tests/test_moe_router.cpp:64-72


def test_router_tie_goes_to_lower_id():
    logits = np.zeros((1, 8), np.float32)
    ids, w, ties = oracle.router(logits, None, 3, norm_topk=True, routed_scale=2.5)
    assert ids.tolist() == [[0, 1, 2]] and ties == 1
    np.testing.assert_allclose(w, 2.5 / 3, atol=1e-6)


def test_rmsnorm_golden(golden_dir):
    z = np.load(os.path.join(golden_dir, "rmsnorm.npz"))
    assert np.array_equal(oracle.rmsnorm_rows(z["x"], z["w"], float(z["eps"])), z["out_ref"])


def test_dispatch_is_stable_counting_sort():
    rng = np.random.default_rng(0)
    ids = np.stack([rng.permutation(16)[:4] for _ in range(37)]).astype(np.int32)
    offs, tok, row = oracle.dispatch(ids, 16)
    flat = ids.reshape(-1)
    order = np.argsort(flat, kind="stable")
    assert np.array_equal(tok, order // 4) and np.array_equal(row, order % 4)
    assert np.array_equal(offs, np.concatenate([[0], np.cumsum(np.bincount(flat, minlength=16))]))


def test_dispatch_empty():
    offs, tok, row = oracle.dispatch(np.zeros((0, 4), np.int32), 8)
    assert offs.tolist() == [0] * 9 and tok.size == 0


def test_dequant_rule_and_quantiser_roundtrip():
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((6, 64)) * 0.02).astype(np.float32)
    w[2, :32] = 0.0                                            # all-zero group -> scale 1.0
    q, s = quantize_w4_np(w, 32)
    assert s[2, 0] == 1.0 and np.all((q[2, :16] & 0xF) == 8)
    d = oracle.dequant_int4(q, s, w.size, 32).reshape(w.shape)
    assert np.array_equal(d, dequantize_w4_np(q, s, 32))
    assert np.max(np.abs(d - w)) <= np.max(s) * 0.5 * 1.01 + 1e-6
    lo, hi = q & 0xF, q >> 4                                   # even column in the low nibble
    assert np.array_equal(lo[0].astype(int) - 8, np.clip(np.rint(w[0, 0::2] / np.repeat(
        np.max(np.abs(w[0].reshape(2, 32)), axis=1) / np.float32(7), 16)), -8, 7).astype(int))
    assert hi.dtype == np.uint8


def test_gemm_w4a16_equals_linear_on_dequantised():
    rng = np.random.default_rng(6)
    w = (rng.standard_normal((20, 96)) * 0.02).astype(np.float32)
    q, s = quantize_w4_np(w, 32)
    x = round_bf16_np(rng.standard_normal((3, 96)).astype(np.float32))
    bias = rng.standard_normal(20).astype(np.float32)
    y = oracle.gemm_w4a16(x, q, s, 32, bias=bias)
    assert np.array_equal(y, oracle.linear(dequantize_w4_np(q, s, 32), x, bias))


def test_experts_entry_matches_layer(golden_dir):
    L = _load_layer(golden_dir)
    r = oracle.moe_layer_w4(L["x"], L)
    Lns = dict(L, sg_q=None, sg_sc=None, su_q=None, su_sc=None, sd_q=None, sd_sc=None)
    routed = oracle.moe_experts_w4(L["x"], r["ids"], r["w"], Lns)
    full_noshared = oracle.moe_layer_w4(L["x"], Lns)["out"]
    assert np.array_equal(routed, full_noshared)


@pytest.mark.skipif(not oracle.ref_available(), reason="reference library not built here")
def test_mid_config_bit_equal_to_reference():
    L = make_layer_np(CONFIGS["mid"], seed=7)
    x = make_x_np(24, L["H"], seed=8)
    out_ref, _ = oracle.ref_moe_mlp_w4(x, L)
    assert np.array_equal(oracle.moe_layer_w4(x, L)["out"], out_ref)
    assert np.array_equal(oracle.ref_dequant_int4(L["sd_q"], L["sd_sc"], L["sd_q"].size * 2, L["group"]),
                          oracle.dequant_int4(L["sd_q"], L["sd_sc"], L["sd_q"].size * 2, L["group"]))

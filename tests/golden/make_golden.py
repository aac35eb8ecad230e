"""Regenerates the golden fixtures in this folder from the reference itself.

Run in a container that holds the reference tree (environment variable REF_ROOT points at it):
    python tests/golden/make_golden.py
It builds oracle/_ref/libglmref.so (the reference's own CPU float32 MoE, compiled from the
reference sources in place) and imports the reference's numpy twin
(tools/make_tiny_checkpoint.py) to produce:

  tiny_layer.npz   benchmark configuration 1 (H=256, E=16, top-4, I=128, g=32, 64 tokens):
                   every input tensor plus `out_ref` (GLM52Model::moe_mlp), `logits_ref`
                   (linear_forward), `out_numpy` / `ids_numpy` / `w_numpy` (the numpy twin).
  router_cases.npz the shape of the reference's router unit test (n=7, E=32, top-4, scale
                   2.5, normalised, bias 0.05*N(0,1)) plus an E=256/top-8 case; expected
                   ids and weights from the numpy twin's rule (stable argsort of -choose).
  rmsnorm.npz      rows through the reference's rmsnorm_rows.
The GPU box never runs this script; it only reads the .npz files.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF_ROOT = os.environ.get("REF_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
if not os.path.isdir(os.path.join(REF_ROOT, "tools")):
    sys.exit("set REF_ROOT to the reference checkout (its tools/ folder is imported to generate the vectors)")

import oracle  # noqa: E402
from glmserve_b200.quant import dequantize_w4_np  # noqa: E402
from glmserve_b200.synth import CONFIGS, make_layer_np, make_x_np  # noqa: E402


def load_numpy_twin():
    spec = importlib.util.spec_from_file_location(
        "make_tiny_checkpoint", os.path.join(REF_ROOT, "tools", "make_tiny_checkpoint.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def numpy_twin_layer(twin, L, x):
    """Feeds the layer to the reference's numpy moe() through its weight-dict naming."""
    cfg = dict(num_experts_per_tok=L["topk"], routed_scaling_factor=L["routed_scale"],
               norm_topk_prob=L["norm_topk"])
    p = "l."
    W = {p + "mlp.gate.weight": L["router_w"], p + "mlp.gate.e_score_correction_bias": L["e_bias"]}
    g = L["group"]
    for e in range(L["E"]):
        ep = p + f"mlp.experts.{e}."
        W[ep + "gate_proj.weight"] = dequantize_w4_np(L["gate_q"][e], L["gate_sc"][e], g)
        W[ep + "up_proj.weight"] = dequantize_w4_np(L["up_q"][e], L["up_sc"][e], g)
        W[ep + "down_proj.weight"] = dequantize_w4_np(L["down_q"][e], L["down_sc"][e], g)
    sp = p + "mlp.shared_experts."
    W[sp + "gate_proj.weight"] = dequantize_w4_np(L["sg_q"], L["sg_sc"], g)
    W[sp + "up_proj.weight"] = dequantize_w4_np(L["su_q"], L["su_sc"], g)
    W[sp + "down_proj.weight"] = dequantize_w4_np(L["sd_q"], L["sd_sc"], g)
    return twin.moe(cfg, W, p, x)


def twin_router(twin, logits, bias, topk, scale, norm=True):
    ids, ws = [], []
    for t in range(logits.shape[0]):
        score = twin.sigmoid(logits[t])
        choose = score + bias
        idx = np.argsort(-choose, kind="stable")[:topk]
        w = score[idx].astype(np.float32)
        if norm and w.sum() > 0:
            w = w / w.sum()
        ids.append(idx.astype(np.int32))
        ws.append((w * scale).astype(np.float32))
    return np.stack(ids), np.stack(ws)


def main():
    oracle.build(with_ref=True)
    assert oracle.ref_available(), "reference tree not found; cannot regenerate fixtures"
    twin = load_numpy_twin()

    L = make_layer_np(CONFIGS["tiny"], seed=1234)
    x = make_x_np(64, L["H"], seed=99)
    out_ref, _ = oracle.ref_moe_mlp_w4(x, L)
    logits_ref = oracle.ref_linear_forward(L["router_w"], x)
    out_numpy = numpy_twin_layer(twin, L, x).astype(np.float32)
    ids_np, w_np = twin_router(twin, twin.linear(x, L["router_w"]), L["e_bias"], L["topk"],
                               L["routed_scale"])
    np.savez_compressed(os.path.join(HERE, "tiny_layer.npz"), x=x, out_ref=out_ref,
                        logits_ref=logits_ref, out_numpy=out_numpy, ids_numpy=ids_np, w_numpy=w_np,
                        **{k: v for k, v in L.items() if v is not None})

    rng = np.random.default_rng(3)
    cases = {}
    for tag, n, E, k in (("a", 7, 32, 4), ("b", 33, 256, 8), ("c", 5, 160, 8)):
        logits = rng.standard_normal((n, E)).astype(np.float32)
        bias = (0.05 * rng.standard_normal(E)).astype(np.float32)
        ids, w = twin_router(twin, logits, bias, k, 2.5)
        cases.update({f"{tag}_logits": logits, f"{tag}_bias": bias, f"{tag}_ids": ids, f"{tag}_w": w,
                      f"{tag}_topk": np.int32(k)})
    np.savez_compressed(os.path.join(HERE, "router_cases.npz"), **cases)

    xr = rng.standard_normal((5, 384)).astype(np.float32) * 3.0
    wr = (1.0 + 0.02 * rng.standard_normal(384)).astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "rmsnorm.npz"), x=xr, w=wr, eps=np.float32(1e-5),
                        out_ref=oracle.ref_rmsnorm_rows(xr, wr, 1e-5))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()

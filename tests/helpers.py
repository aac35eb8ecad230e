"""Shared helpers for the GPU parity tests."""
import numpy as np

# Tolerances of the layer output against the fp32 CPU reference (bf16 activations in).
MAX_ABS_TOL = 2e-2
REL_L2_TOL = 1e-3


def rel_l2(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


def assert_layer_close(out, ref, what=""):
    out = np.asarray(out, np.float32)
    ref = np.asarray(ref, np.float32)
    assert np.isfinite(out).all(), f"{what}: non-finite output"
    ma = float(np.max(np.abs(out - ref))) if out.size else 0.0
    rl = rel_l2(out, ref) if out.size else 0.0
    assert ma <= MAX_ABS_TOL and rl <= REL_L2_TOL, f"{what}: max-abs {ma:.3e}, rel-L2 {rl:.3e}"
    return ma, rl


def load_tiny(golden_dir):
    import os
    z = np.load(os.path.join(golden_dir, "tiny_layer.npz"))
    L = {k: z[k] for k in z.files}
    for k in ("H", "E", "topk", "I", "Is", "group"):
        L[k] = int(L[k])
    L["norm_topk"] = bool(L["norm_topk"])
    L["routed_scale"] = float(L["routed_scale"])
    return L


def bf16_tensor(x_np, device):
    import torch
    return torch.from_numpy(np.ascontiguousarray(x_np, np.float32)).to(device).to(torch.bfloat16)

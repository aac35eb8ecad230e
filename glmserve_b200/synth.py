"""Seeded synthetic MoE layers in the reference's resident-weight layout.

Layout (src/model_gpu.cpp:948-1000 of the reference): ``gate_q, up_q : u8 [E, I, H/2]``,
``gate_sc, up_sc : [E, I, H/g]``, ``down_q : u8 [E, H, I/2]``, ``down_sc : [E, H, I/g]``,
shared expert ``sg_q, su_q : u8 [Is, H/2]``, ``sd_q : u8 [H, Is/2]`` with their scales,
``router_w : [E, H]`` (bf16-representable), ``e_bias : f32 [E]``.  Scales hold
fp16-representable values.  Weights ~N(0, 0.02), bias ~N(0, 0.01), activations ~N(0, 1)
rounded to bf16 - the value distributions the benchmark configurations name.
"""
from __future__ import annotations

import numpy as np

from .quant import quantize_w4_np, quantize_w4_torch, round_bf16_np

CONFIGS = {
    # name: H, E, topk, I, Is, group
    "tiny": dict(H=256, E=16, topk=4, I=128, Is=128, group=32),
    "mid": dict(H=1024, E=32, topk=8, I=512, Is=512, group=128),
    "wide": dict(H=4096, E=8, topk=2, I=2048, Is=2048, group=128),
    "glm": dict(H=6144, E=256, topk=8, I=2048, Is=2048, group=128),
}


def zipf_bias(E: int, rng: np.random.Generator, amplitude: float, s: float = 1.1) -> np.ndarray:
    """A Zipf(s)-ranked additive router bias used to skew per-expert loads: the expert with
    rank r (a seeded permutation of the experts) gets ``amplitude * ln(E * p_r)`` with
    ``p_r = r**-s / sum(r**-s)``.  With amplitude 0.04 on the GLM-scale layer (E=256, top-8,
    8192 tokens) the loads span about 0.01x to 8x the mean."""
    ranks = rng.permutation(E).astype(np.float64) + 1.0
    p = ranks ** (-s)
    p /= p.sum()
    return (amplitude * np.log(E * p)).astype(np.float32)


def make_layer_np(cfg: dict, seed: int, shared: bool = True, zipf_amplitude: float = 0.0) -> dict:
    """numpy layer dict for small shapes (tests, golden vectors)."""
    H, E, topk, I, Is, g = (cfg[k] for k in ("H", "E", "topk", "I", "Is", "group"))
    rng = np.random.default_rng(seed)
    L = dict(H=H, E=E, topk=topk, I=I, Is=Is, group=g, norm_topk=True, routed_scale=2.5)
    L["router_w"] = round_bf16_np((rng.standard_normal((E, H)) * 0.02).astype(np.float32))
    L["e_bias"] = (rng.standard_normal(E) * 0.01).astype(np.float32)
    if zipf_amplitude:
        L["e_bias"] = (L["e_bias"] + zipf_bias(E, rng, zipf_amplitude)).astype(np.float32)
    for name, shape in (("gate", (E, I, H)), ("up", (E, I, H)), ("down", (E, H, I))):
        w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
        L[name + "_q"], L[name + "_sc"] = quantize_w4_np(w, g)
    if shared:
        for name, shape in (("sg", (Is, H)), ("su", (Is, H)), ("sd", (H, Is))):
            w = (rng.standard_normal(shape) * 0.02).astype(np.float32)
            L[name + "_q"], L[name + "_sc"] = quantize_w4_np(w, g)
    else:
        for name in ("sg", "su", "sd"):
            L[name + "_q"] = L[name + "_sc"] = None
    return L


def make_x_np(n: int, H: int, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return round_bf16_np(rng.standard_normal((n, H)).astype(np.float32))


def make_layer_torch(cfg: dict, seed: int, device, shared: bool = True,
                     zipf_amplitude: float = 0.0) -> dict:
    """Layer dict of torch tensors generated and quantised on ``device`` (GLM scale takes
    seconds on a GPU).  Scales are float16; router_w is bfloat16; e_bias float32."""
    import torch

    H, E, topk, I, Is, g = (cfg[k] for k in ("H", "E", "topk", "I", "Is", "group"))
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    L = dict(H=H, E=E, topk=topk, I=I, Is=Is, group=g, norm_topk=True, routed_scale=2.5)
    L["router_w"] = (torch.randn((E, H), generator=gen, device=device) * 0.02).to(torch.bfloat16)
    bias = torch.randn((E,), generator=gen, device=device) * 0.01
    if zipf_amplitude:
        rng = np.random.default_rng(seed)
        bias = bias + torch.from_numpy(zipf_bias(E, rng, zipf_amplitude)).to(device)
    L["e_bias"] = bias.float().contiguous()
    for name, rows, cols in (("gate", I, H), ("up", I, H), ("down", H, I)):
        q = torch.empty((E, rows, cols // 2), dtype=torch.uint8, device=device)
        sc = torch.empty((E, rows, cols // g), dtype=torch.float16, device=device)
        step = max(1, min(E, (1 << 28) // (rows * cols)))
        for e0 in range(0, E, step):
            e1 = min(E, e0 + step)
            w = torch.randn((e1 - e0, rows, cols), generator=gen, device=device) * 0.02
            q[e0:e1], sc[e0:e1] = quantize_w4_torch(w, g)
        L[name + "_q"], L[name + "_sc"] = q, sc
    if shared:
        for name, rows, cols in (("sg", Is, H), ("su", Is, H), ("sd", H, Is)):
            w = torch.randn((rows, cols), generator=gen, device=device) * 0.02
            L[name + "_q"], L[name + "_sc"] = quantize_w4_torch(w, g)
    else:
        for name in ("sg", "su", "sd"):
            L[name + "_q"] = L[name + "_sc"] = None
    return L


def make_x_torch(n: int, H: int, seed: int, device):
    import torch

    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    return torch.randn((n, H), generator=gen, device=device).to(torch.bfloat16)


def layer_to_np(L: dict) -> dict:
    """torch layer dict -> numpy dict in the oracle's input types (float32 scales etc.)."""
    import torch

    out = {}
    for k, v in L.items():
        if isinstance(v, torch.Tensor):
            out[k] = v.detach().cpu().numpy() if v.dtype == torch.uint8 else v.detach().float().cpu().numpy()
        else:
            out[k] = v
    return out


def layer_to_torch(L: dict, device) -> dict:
    """numpy layer dict -> torch tensors on ``device`` in the kernels' input types."""
    import torch

    out = {}
    for k, v in L.items():
        if isinstance(v, np.ndarray):
            t = torch.from_numpy(np.ascontiguousarray(v)).to(device)
            if k.endswith("_sc"):
                t = t.to(torch.float16)
            elif k == "router_w":
                t = t.to(torch.bfloat16)
            out[k] = t.contiguous()
        else:
            out[k] = v
    return out

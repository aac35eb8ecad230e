"""W4 quantiser and number-format helpers (numpy and torch forms of the same rule).

The rule is the reference converter's (tools/convert_hf_to_glmserve.py:233-246): per row
and per group of ``group`` input columns, ``s = max|w| / 7`` (1.0 when the group is all
zero), ``q = clip(rint(w / s), -8, 7) + 8``; two values per byte with the even column in
the low nibble.  Scales are then rounded to fp16 and kept as float32 values, which is the
scale format the B200 kernels store.
"""
from __future__ import annotations

import numpy as np


def round_bf16_np(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bf16, returned as float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return (((u + r) >> 16) << 16).astype(np.uint32).view(np.float32)


def f32_to_bf16_bits_np(a: np.ndarray) -> np.ndarray:
    """float32 (already bf16-representable or not) -> uint16 bf16 bit patterns (RNE)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def quantize_w4_np(w: np.ndarray, group: int):
    """w float32 [..., out, in] -> (packed uint8 [..., out, in/2], scales float32 [..., out, in/group])."""
    w = np.ascontiguousarray(w, np.float32)
    *lead, out, inn = w.shape
    assert inn % 2 == 0 and inn % group == 0
    g = w.reshape(*lead, out, inn // group, group)
    s = (np.max(np.abs(g), axis=-1) / np.float32(7.0)).astype(np.float32)
    s = np.where(s > 0.0, s, np.float32(1.0)).astype(np.float32)
    q = np.rint(g / s[..., None])
    q = (np.clip(q, -8, 7).astype(np.int16) + 8).astype(np.uint8).reshape(*lead, out, inn)
    packed = (q[..., 0::2] | (q[..., 1::2] << 4)).astype(np.uint8)
    s16 = s.astype(np.float16).astype(np.float32)
    return packed, s16


def dequantize_w4_np(packed: np.ndarray, scales: np.ndarray, group: int) -> np.ndarray:
    """Inverse map used by host-side checks: float32 [..., out, in]."""
    lo = (packed & 0x0F).astype(np.int16) - 8
    hi = (packed >> 4).astype(np.int16) - 8
    q = np.stack([lo, hi], axis=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)
    return q.astype(np.float32) * np.repeat(scales.astype(np.float32), group, axis=-1)


def quantize_w4_torch(w, group: int):
    """torch form of quantize_w4_np (any device); returns (uint8 packed, float16 scales)."""
    import torch

    *lead, out, inn = w.shape
    g = w.float().reshape(*lead, out, inn // group, group)
    s = g.abs().amax(dim=-1) / 7.0
    s = torch.where(s > 0, s, torch.ones_like(s))
    q = torch.round(g / s[..., None]).clamp_(-8, 7).to(torch.int16) + 8
    q = q.to(torch.uint8).reshape(*lead, out, inn)
    packed = q[..., 0::2] | (q[..., 1::2] << 4)
    return packed.contiguous(), s.to(torch.float16).contiguous()

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


# ---- tile stream (host reference of the device repack, csrc/prepack.cu) ------------------
CHUNK_COLS, CHUNK_WEIGHT_BYTES, CHUNK_BYTES = 512, 8192, 8448
_NIBBLE_PERM = (0, 2, 4, 6, 1, 3, 5, 7)  # output nibble p holds column perm[p] of its word


def prepack_np(a_q, a_sc, b_q=None, b_sc=None) -> np.ndarray:
    """numpy twin of gsb_prepack_gate_up (b given) / gsb_prepack_down (b None).

    a_q/b_q: uint8 [E, rows, cols/2]; a_sc/b_sc: [E, rows, cols/128] (fp16-representable).
    Returns the uint8 tile stream [E * units * chunks * 8448].  Unit = 32 rows (gate/up:
    16 rows of a then the same 16 rows of b); chunk = 512 columns: eight 1 KiB blocks
    (kstep*2 + half unit) then fp16 scales [kstep][half unit][16].
    """
    E, rows, rb = a_q.shape
    cols = rb * 2
    pair = b_q is not None
    units = rows // 16 if pair else rows // 32
    chunks = cols // CHUNK_COLS
    out = np.zeros((E, units, chunks, CHUNK_BYTES), np.uint8)

    def nat_words(q):  # [E, rows, cols/8] uint32, nibble i = column i of the word
        return np.ascontiguousarray(q).view(np.uint32).reshape(E, rows, cols // 8)

    def perm_words(wd):
        o = np.zeros_like(wd)
        for p, src in enumerate(_NIBBLE_PERM):
            o |= ((wd >> np.uint32(4 * src)) & np.uint32(0xF)) << np.uint32(4 * p)
        return o

    wa = perm_words(nat_words(a_q))
    wb = perm_words(nat_words(b_q)) if pair else None
    wout = out[..., :CHUNK_WEIGHT_BYTES].view(np.uint32).reshape(E, units, chunks, 8, 2, 32, 4)
    sout = out[..., CHUNK_WEIGHT_BYTES:].view(np.float16).reshape(E, units, chunks, 4, 2, 16)
    for m in range(2):
        if pair:
            src_w, src_s = (wa, a_sc) if m == 0 else (wb, b_sc)
            rsel = lambda u: slice(16 * u, 16 * u + 16)  # noqa: E731
        else:
            src_w, src_s = wa, a_sc
            rsel = lambda u, m=m: slice(32 * u + 16 * m, 32 * u + 16 * m + 16)  # noqa: E731
        for u in range(units):
            wr = src_w[:, rsel(u), :].reshape(E, 2, 8, chunks, 4, 4, 4)   # [E, h, g, c, s, t, j]
            # block layout [h][lane = 4g + t][j]
            blk = wr.transpose(0, 3, 4, 1, 2, 5, 6).reshape(E, chunks, 4, 2, 32, 4)  # [E,c,s,h,lane,j]
            for s in range(4):
                wout[:, u, :, s * 2 + m] = blk[:, :, s]
            sc = np.asarray(src_s)[:, rsel(u), :].astype(np.float16).reshape(E, 16, chunks, 4)
            sout[:, u, :, :, m, :] = sc.transpose(0, 2, 3, 1)
    return out.reshape(-1)


def frag_pos(f):
    """Position of feature f inside a fragment-ordered activation row (csrc/decode_w4.cu)."""
    kb, kk = f >> 7, f & 127
    t, j, el = kk >> 5, (kk >> 3) & 3, kk & 7
    return (kb << 7) + (((j << 2) + t) << 3) + el

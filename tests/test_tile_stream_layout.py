"""Host-side check of the tile-stream layout: the numpy packer, read back with the index
arithmetic the decode kernel's consumer warps use, must reproduce the dequantised matrix."""
import numpy as np

from glmserve_b200.quant import (CHUNK_BYTES, CHUNK_WEIGHT_BYTES, dequantize_w4_np, frag_pos,
                                 prepack_np, quantize_w4_np)


def _consumer_view(stream, E, units, K):
    """Re-reads a tile stream the way decode_gemm_kernel's consumers do: warp (ck, ks, m),
    lane (g, t), word j -> unit rows g / g+8 of half m, columns kb*128 + 32t + 8j + 0..7,
    nibble pairs from the 0x000f000f / 0x00f000f0 masks.  Returns q-8 as [E, units, 32, K]
    and the scales [E, units, 32, K/128]."""
    chunks = K // 512
    s8 = stream.reshape(E, units, chunks, CHUNK_BYTES)
    W = np.zeros((E, units, 32, K), np.float32)
    S = np.zeros((E, units, 32, K // 128), np.float32)
    for c in range(chunks):
        chunk = s8[:, :, c]
        sc = chunk[..., CHUNK_WEIGHT_BYTES:].view(np.float16).reshape(E, units, 4, 2, 16)
        for ks in range(4):
            for m in range(2):
                blk = chunk[..., (ks * 2 + m) * 1024:(ks * 2 + m + 1) * 1024].view(np.uint32).reshape(E, units, 2, 32, 4)
                kb = c * 4 + ks
                for lane in range(32):
                    g, t = lane >> 2, lane & 3
                    for h in range(2):
                        row = m * 16 + g + 8 * h
                        S[:, :, row, kb] = sc[:, :, ks, m, g + 8 * h]
                        for j in range(4):
                            w = blk[:, :, h, lane, j]
                            lo0 = (w & 0x000F000F)
                            hi0 = (w & 0x00F000F0) >> 4
                            w8 = w >> 8
                            lo1 = (w8 & 0x000F000F)
                            hi1 = (w8 & 0x00F000F0) >> 4
                            col = kb * 128 + 32 * t + 8 * j
                            for idx, v in enumerate((lo0, hi0, lo1, hi1)):
                                W[:, :, row, col + 2 * idx] = (v & 0xFFFF).astype(np.float32) - 8
                                W[:, :, row, col + 2 * idx + 1] = (v >> 16).astype(np.float32) - 8
    return W, S


def test_down_layout_roundtrip():
    rng = np.random.default_rng(0)
    E, rows, cols = 2, 64, 1024
    w = (rng.standard_normal((E, rows, cols)) * 0.02).astype(np.float32)
    q, s = quantize_w4_np(w, 128)
    stream = prepack_np(q, s)
    assert stream.size == E * (rows // 32) * (cols // 512) * CHUNK_BYTES
    W, S = _consumer_view(stream, E, rows // 32, cols)
    deq = (W * np.repeat(S, 128, axis=-1)).reshape(E, rows, cols)
    assert np.array_equal(deq, dequantize_w4_np(q, s, 128))


def test_gate_up_layout_interleaves_16_and_16():
    rng = np.random.default_rng(1)
    E, I, H = 1, 48, 512
    qg, sg = quantize_w4_np((rng.standard_normal((E, I, H)) * 0.02).astype(np.float32), 128)
    qu, su = quantize_w4_np((rng.standard_normal((E, I, H)) * 0.02).astype(np.float32), 128)
    stream = prepack_np(qg, sg, qu, su)
    W, S = _consumer_view(stream, E, I // 16, H)
    deq = W * np.repeat(S, 128, axis=-1)          # [E, units, 32, H]
    assert np.array_equal(deq[:, :, :16].reshape(E, I, H), dequantize_w4_np(qg, sg, 128))
    assert np.array_equal(deq[:, :, 16:].reshape(E, I, H), dequantize_w4_np(qu, su, 128))


def test_frag_pos_is_a_permutation_within_128():
    p = np.array([frag_pos(f) for f in range(512)])
    assert sorted(p.tolist()) == list(range(512))
    assert all(p[f] // 128 == f // 128 for f in range(512))
    # the four lanes of a quad (t = 0..3) read adjacent 16-byte pieces for a given word j
    assert [frag_pos(32 * t) for t in range(4)] == [0, 8, 16, 24]

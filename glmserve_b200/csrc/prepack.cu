// One-time repack of the reference's resident int4 layout into the tile stream described
// in launchers.cuh.  One block per 8448-byte chunk.
#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

__global__ void __launch_bounds__(256)
prepack_kernel(const uint8_t* __restrict__ a_q, const void* __restrict__ a_sc,
               const uint8_t* __restrict__ b_q, const void* __restrict__ b_sc, int scales_f32,
               int rows, int cols, int units, int chunks, uint8_t* __restrict__ out) {
    const int64_t cid = blockIdx.x;                 // ((e * units) + u) * chunks + c
    const int c = (int)(cid % chunks);
    const int u = (int)((cid / chunks) % units);
    const int64_t e = cid / ((int64_t)chunks * units);
    uint8_t* dst = out + cid * kChunkBytes;
    const int64_t row_bytes = cols / 2;
    const int ngroups = cols / 128;
    // weight words
    for (int wi = threadIdx.x; wi < kChunkWeightBytes / 4; wi += blockDim.x) {
        const int blk = wi >> 8;                    // 256 words per 1 KiB block
        const int s = blk >> 1, m = blk & 1;
        const int in_blk = wi & 255;
        const int h = in_blk >> 7;                  // half: row g or row g + 8
        const int lane = (in_blk >> 2) & 31;
        const int j = in_blk & 3;
        const int g = lane >> 2, t = lane & 3;
        const int r_local = g + 8 * h;              // 0..15 within the half unit
        const uint8_t* src_q;
        int64_t row;
        if (b_q) { src_q = m ? b_q : a_q; row = (int64_t)u * 16 + r_local; }
        else     { src_q = a_q;           row = (int64_t)u * 32 + m * 16 + r_local; }
        const int64_t col = (int64_t)c * kChunkCols + s * 128 + t * 32 + j * 8;
        const uint32_t nat = *reinterpret_cast<const uint32_t*>(
            src_q + (e * rows + row) * row_bytes + col / 2);
        // natural nibble i holds column i; output nibble p holds column perm[p]
        uint32_t o = 0;
        const int perm[8] = {0, 2, 4, 6, 1, 3, 5, 7};
#pragma unroll
        for (int p = 0; p < 8; ++p) o |= ((nat >> (4 * perm[p])) & 0xFu) << (4 * p);
        reinterpret_cast<uint32_t*>(dst)[wi] = o;
    }
    // scales [s][m][16] fp16
    for (int si = threadIdx.x; si < 128; si += blockDim.x) {
        const int s = si >> 5, m = (si >> 4) & 1, r_local = si & 15;
        const void* src_s;
        int64_t row;
        if (b_q) { src_s = m ? b_sc : a_sc; row = (int64_t)u * 16 + r_local; }
        else     { src_s = a_sc;            row = (int64_t)u * 32 + m * 16 + r_local; }
        const int64_t idx = (e * rows + row) * ngroups + (int64_t)c * 4 + s;
        __half v = scales_f32 ? __float2half_rn(reinterpret_cast<const float*>(src_s)[idx])
                              : reinterpret_cast<const __half*>(src_s)[idx];
        reinterpret_cast<__half*>(dst + kChunkWeightBytes)[si] = v;
    }
}

int launch_prepack(const uint8_t* a_q, const void* a_sc, const uint8_t* b_q, const void* b_sc,
                   int scales_f32, int experts, int rows, int cols, void* out, cudaStream_t s) {
    const int units = b_q ? rows / 16 : rows / 32;
    const int chunks = cols / kChunkCols;
    const int64_t total = (int64_t)experts * units * chunks;
    if (total <= 0 || total > 0x7fffffffLL) return GSB_ERR_UNSUPPORTED;
    prepack_kernel<<<(unsigned)total, 256, 0, s>>>(a_q, a_sc, b_q, b_sc, scales_f32, rows, cols,
                                                   units, chunks, reinterpret_cast<uint8_t*>(out));
    return launch_status();
}

}  // namespace gsb

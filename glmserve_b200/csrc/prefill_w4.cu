// Prefill-shaped W4A16 grouped GEMM on the 5th-generation tensor cores (tcgen05 / TMEM).
//
// D[weight row, token] = sum_k W[row, k] * X[token, k] for one tile = (expert segment of up
// to 256 token rows) x (128 weight rows = four 32-row units of the tile stream).
//   A operand (M = 128 weight rows): int4 chunks arrive by 1-D bulk copies; eight dequant
//     warps unpack them to fp16 (q - 8) * scale and store them into shared memory in the
//     K-major 128-byte-swizzled layout the tensor core reads.
//   B operand (N = 16..256 token rows): fp16 activations, gathered into expert order
//     beforehand, loaded by TMA (2-D tiled, 128-byte swizzle, no multicast).
//   D: fp32 in tensor memory, two buffers of 256 columns so the epilogue of one tile overlaps
//     the main loop of the next.
// One thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x N x 16); tcgen05.commit
// releases shared-memory stages and publishes finished accumulators through mbarriers.
// Epilogue warps read the accumulator with tcgen05.ld: the gate/up kernel pairs gate and up
// rows (lanes l and l^16 of a warp) to fuse SwiGLU and stores fp16 h; the down kernel stores
// the slot's fp16 output row.  Persistent CTAs walk a tile list built on the device.
// All waits are bounded (see mbar_wait); a timeout is recorded in the status word.
#include <cuda.h>

#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

namespace {

constexpr int kPfThreads = 512;        // 16 warps
// A (dequantised weights, 16 KiB) and B (activations, 32 KiB) stages are template parameters
// AS / BS of the kernel; one stage = one 64-column k-block.
constexpr int kBN = 256;               // token rows per tile (TMA box rows)
constexpr int kABytes = 128 * 128;     // 128 weight rows x 64 fp16
constexpr int kBBytes = kBN * 128;     // 256 token rows x 64 fp16
constexpr int kQBytes = 4 * kChunkBytes;  // four units x one 512-column chunk
constexpr long long kPfWaitLimit = 2000000000LL;
constexpr int kTileHeader = 4;

struct PrefillKArgs {
    const uint8_t* packed;
    const uint8_t* shared_packed;
    const int* tiles;        // [0] = ntiles; then int4 {expert, first slot, tokens, row block}
    int K, Ks;               // input dims (routed / shared)
    int units, units_s;      // 32-row units per expert
    int E;
    __half* hbuf; int ldh;   // gate/up output, natural feature order
    __half* ybuf; int H;     // down output [slots, H]
    __half* const* ydst;     // optional per-row output pointers (expert parallel: rows live on the
                             // token's home GPU and are stored there over NVLink); overrides ybuf
    int* status;
};

__device__ __forceinline__ void pf_timeout(const PrefillKArgs& a, volatile int* abort_flag, int where) {
    *abort_flag = 1;
    if (atomicCAS(a.status + kStatusCode, 0, GSB_ERR_TIMEOUT) == 0) {
        a.status[kStatusWhere] = 100 + where;
        a.status[kStatusAux] = (int)blockIdx.x;
    }
}

// ---- tcgen05 wrappers --------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 bytes apart, groups of
// eight rows 1024 bytes apart (stride byte offset); descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;      // stride byte offset
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// Instruction descriptor, kind::f16: fp32 accumulate, fp16 A and B, both K-major, M=128.
__device__ __forceinline__ uint32_t make_idesc(uint32_t n) {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// eight int4 (tile-stream order) -> four fp16x2 of (q - 8) * s, each product rounded once
__device__ __forceinline__ uint4 dequant8(uint32_t w, __half2 s2) {
    const __half2 k1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
    const __half2 k16th = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));
    const __half2 km72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));
    uint32_t lo0 = (w & 0x000f000fu) | 0x64006400u;
    uint32_t hi0 = (w & 0x00f000f0u) | 0x64006400u;
    const uint32_t w8 = w >> 8;
    uint32_t lo1 = (w8 & 0x000f000fu) | 0x64006400u;
    uint32_t hi1 = (w8 & 0x00f000f0u) | 0x64006400u;
    __half2 a = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&lo0), k1032), s2);
    __half2 b = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&hi0), k16th, km72), s2);
    __half2 c = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&lo1), k1032), s2);
    __half2 d = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&hi1), k16th, km72), s2);
    uint4 o;
    o.x = *reinterpret_cast<uint32_t*>(&a);
    o.y = *reinterpret_cast<uint32_t*>(&b);
    o.z = *reinterpret_cast<uint32_t*>(&c);
    o.w = *reinterpret_cast<uint32_t*>(&d);
    return o;
}

struct PfTile { int expert, slot0, ntok, rb, K, nkb, nround; const uint8_t* chunks; int unit_stride; };

__device__ __forceinline__ PfTile pf_tile(const PrefillKArgs& a, int idx) {
    const int4 t = reinterpret_cast<const int4*>(a.tiles + kTileHeader)[idx];
    PfTile r;
    r.expert = t.x; r.slot0 = t.y; r.ntok = t.z; r.rb = t.w;
    const bool sh = t.x >= a.E;
    r.K = sh ? a.Ks : a.K;
    r.nkb = r.K >> 6;
    r.nround = (r.ntok + 15) & ~15;
    const int U = sh ? a.units_s : a.units;
    const int nchunk = r.K / kChunkCols;
    const uint8_t* base = sh ? a.shared_packed : a.packed;
    const int64_t e_local = sh ? 0 : t.x;
    r.chunks = base + ((e_local * U + (int64_t)r.rb * 4) * nchunk) * (int64_t)kChunkBytes;
    r.unit_stride = nchunk * kChunkBytes;
    return r;
}

template <bool GU, int AS, int BS>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_gemm_kernel(const PrefillKArgs a, const __grid_constant__ CUtensorMap tmap_b64,
                    const __grid_constant__ CUtensorMap tmap_b128, const __grid_constant__ CUtensorMap tmap_b256) {
    extern __shared__ uint8_t smem_raw[];
    // the kernel has no static shared memory, so the dynamic window starts 1024-byte aligned (the
    // swizzled tiles need that); checked below, a misaligned base is reported instead of used
    uint8_t* smem = smem_raw;
    uint8_t* sA = smem;                                   // [AS][16 KiB]
    uint8_t* sB = sA + AS * kABytes;                      // [BS][32 KiB]
    uint8_t* sQ = sB + BS * kBBytes;                      // [2][4 chunks]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sQ + 2 * kQBytes);
    uint64_t* full_a = bars;                   // [AS] dequant warps -> MMA
    uint64_t* empty = full_a + AS;             // [AS] MMA commit -> dequant
    uint64_t* full_b = empty + AS;             // [BS] TMA -> MMA
    uint64_t* empty_b = full_b + BS;           // [BS] MMA commit -> producer
    uint64_t* q_full = empty_b + BS;           // [2] bulk copy -> dequant
    uint64_t* q_empty = q_full + 2;            // [2] dequant -> producer
    uint64_t* acc_full = q_empty + 2;          // [2] MMA commit -> epilogue
    uint64_t* acc_empty = acc_full + 2;        // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (smem_u32(smem_raw) & 1023u) {
        if (tid == 0 && atomicCAS(a.status + kStatusCode, 0, GSB_ERR_LAUNCH) == 0) a.status[kStatusWhere] = 199;
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < AS; ++i) { mbar_init(&full_a[i], 4); mbar_init(&empty[i], 1); }
        for (int i = 0; i < BS; ++i) { mbar_init(&full_b[i], 1); mbar_init(&empty_b[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 8); mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int ntiles = a.tiles[0];

    if (warp == 0) {
        // ------------- producer: int4 chunks (bulk copies) and activation tiles (TMA) -------------
        if (lane == 0) {
            uint32_t kc = 0, qc = 0;
            for (int ti = blockIdx.x; ti < ntiles && !*abort_flag; ti += gridDim.x) {
                const PfTile t = pf_tile(a, ti);
                for (int kb = 0; kb < t.nkb; ++kb, ++kc) {
                    if ((kb & 7) == 0) {
                        const uint32_t qs = qc & 1u, qph = (qc >> 1) & 1u;
                        if (!mbar_wait(&q_empty[qs], qph ^ 1u, kPfWaitLimit)) { pf_timeout(a, abort_flag, 1); break; }
                        mbar_arrive_expect_tx(&q_full[qs], kQBytes);
                        const int c = kb >> 3;
#pragma unroll
                        for (int u = 0; u < 4; ++u)
                            bulk_g2s(sQ + qs * kQBytes + u * kChunkBytes,
                                     t.chunks + (int64_t)u * t.unit_stride + (int64_t)c * kChunkBytes, kChunkBytes, &q_full[qs]);
                        ++qc;
                    }
                    const uint32_t s = kc % BS, ph = (kc / BS) & 1u;
                    if (!mbar_wait(&empty_b[s], ph ^ 1u, kPfWaitLimit)) { pf_timeout(a, abort_flag, 2); break; }
                    // the smallest box that covers the tile's rows: a ragged tile does not pull 256 rows
                    const CUtensorMap* tm = t.nround <= 64 ? &tmap_b64 : (t.nround <= 128 ? &tmap_b128 : &tmap_b256);
                    const uint32_t rows = t.nround <= 64 ? 64u : (t.nround <= 128 ? 128u : 256u);
                    mbar_arrive_expect_tx(&full_b[s], rows * 128u);
                    tma_load_2d(sB + s * kBBytes, tm, kb * 64, t.slot0, &full_b[s]);
                }
            }
        }
    } else if (warp == 1) {
        // ------------- MMA issuer -------------
        if (lane == 0) {
            uint32_t kc = 0, tl = 0;
            for (int ti = blockIdx.x; ti < ntiles && !*abort_flag; ti += gridDim.x, ++tl) {
                const PfTile t = pf_tile(a, ti);
                const uint32_t buf = tl & 1u;
                if (!mbar_wait(&acc_empty[buf], ((tl >> 1) & 1u) ^ 1u, kPfWaitLimit)) { pf_timeout(a, abort_flag, 3); break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * 256u;
                const uint32_t idesc = make_idesc((uint32_t)t.nround);
                bool dead = false;
                for (int kb = 0; kb < t.nkb; ++kb, ++kc) {
                    const uint32_t s = kc % AS, ph = (kc / AS) & 1u;
                    const uint32_t sb = kc % BS, phb = (kc / BS) & 1u;
                    if (!mbar_wait(&full_a[s], ph, kPfWaitLimit) || !mbar_wait(&full_b[sb], phb, kPfWaitLimit)) {
                        pf_timeout(a, abort_flag, 4); dead = true; break;
                    }
                    tc_fence_after();
                    const uint64_t ad = make_desc_sw128(smem_u32(sA + s * kABytes));
                    const uint64_t bd = make_desc_sw128(smem_u32(sB + sb * kBBytes));
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4)
                        tc_mma_f16(d_tmem, ad + (uint64_t)(k4 * 2), bd + (uint64_t)(k4 * 2), idesc, (kb | k4) ? 1u : 0u);
                    tc_commit(&empty[s]);
                    tc_commit(&empty_b[sb]);
                }
                if (dead) break;
                tc_commit(&acc_full[buf]);
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ------------- epilogue (warp % 4 selects the TMEM lane quarter) -------------
        const int q = warp & 3;
        uint32_t tl = 0;
        for (int ti = blockIdx.x; ti < ntiles; ti += gridDim.x, ++tl) {
            const PfTile t = pf_tile(a, ti);
            const uint32_t buf = tl & 1u;
            if (*abort_flag || !mbar_wait(&acc_full[buf], (tl >> 1) & 1u, kPfWaitLimit)) {
                if (!*abort_flag) pf_timeout(a, abort_flag, 5);
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * 256u;
            for (int c0 = 0; c0 < t.nround; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(taddr + (uint32_t)c0, r);
                tmem_ld_wait();
                if (GU) {
                    // lanes 0..15 hold gate rows, lanes 16..31 the matching up rows
                    const int feat = t.rb * 64 + q * 16 + (lane & 15);
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
                        const float send = (lane < 16) ? v1 : v0;
                        const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
                        const float g = (lane < 16) ? v0 : recv;
                        const float u = (lane < 16) ? recv : v1;
                        const int n = c0 + j + ((lane < 16) ? 0 : 1);
                        if (n < t.ntok)
                            a.hbuf[(int64_t)(t.slot0 + n) * a.ldh + feat] = __float2half_rn(__fmul_rn(silu_ref(g), u));
                    }
                } else {
                    const int feat = t.rb * 128 + q * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int n = c0 + j;
                        if (n < t.ntok) {
                            __half* yrow = a.ydst ? a.ydst[t.slot0 + n] : a.ybuf + (int64_t)(t.slot0 + n) * a.H;
                            yrow[feat] = __float2half_rn(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    } else if (warp >= 8) {
        // ------------- dequant: int4 chunk pieces -> swizzled fp16 A tile -------------
        // Two groups of four warps take alternate k-blocks, so each group has two MMA periods
        // per k-block; a thread owns one row of the 128-row tile (both 32-column halves).
        const int d = tid - 256;                       // 0..255
        const int grp = d >> 7;                        // 0: even k-blocks, 1: odd
        const int R = d & 127;                         // row of the tile (= TMEM lane)
        const int uu = R >> 5, m = (R >> 4) & 1, h = (R >> 3) & 1, g = R & 7;
        uint32_t kc = grp, qc = 0;
        bool dead = false;
        for (int ti = blockIdx.x; ti < ntiles && !dead; ti += gridDim.x) {
            const PfTile t = pf_tile(a, ti);
            uint32_t qs = 0;
            for (int kb = grp; kb < t.nkb; kb += 2, kc += 2) {
                const int kb8 = kb & 7;
                if (kb8 == grp) {
                    qs = qc & 1u;
                    if (*abort_flag || !mbar_wait(&q_full[qs], (qc >> 1) & 1u, kPfWaitLimit)) {
                        if (!*abort_flag) pf_timeout(a, abort_flag, 6);
                        dead = true; break;
                    }
                    ++qc;
                }
                const int ks = kb8 >> 1, tq0 = grp << 1;
                const uint8_t* chunk = sQ + qs * kQBytes + uu * kChunkBytes;
                const uint4* piece = reinterpret_cast<const uint4*>(chunk + (ks * 2 + m) * 1024 + h * 512 + (g * 4 + tq0) * 16);
                // A row's two 16-byte pieces sit 64 bytes from the next row's, so eight lanes reading
                // "their first piece" fall on two bank groups (4-way conflict).  Rows 2,3,6,7 read
                // their second piece first: four bank groups per load, 2-way - the best this layout
                // allows, since one k-block touches only half of the bank groups.
                const int swp = (g >> 1) & 1;
                const uint4 wa = piece[swp], wb = piece[swp ^ 1];
                const uint4 wv0 = swp ? wb : wa, wv1 = swp ? wa : wb;
                const __half sc = reinterpret_cast<const __half*>(chunk + kChunkWeightBytes)[(ks * 2 + m) * 16 + g + 8 * h];
                const __half2 s2 = __half2half2(sc);
                const uint32_t wq[8] = {wv0.x, wv0.y, wv0.z, wv0.w, wv1.x, wv1.y, wv1.z, wv1.w};
                uint4 dq[8];   // unpacked in registers first: only the stores need the stage to be free
#pragma unroll
                for (int c = 0; c < 8; ++c) dq[c] = dequant8(wq[c], s2);
                const uint32_t s = kc % AS, ph = (kc / AS) & 1u;
                if (!mbar_wait(&empty[s], ph ^ 1u, kPfWaitLimit)) { pf_timeout(a, abort_flag, 7); dead = true; break; }
                uint8_t* arow = sA + s * kABytes + (R >> 3) * 1024 + g * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)             // c = 16-byte piece of the 128-byte row
                    *reinterpret_cast<uint4*>(arow + ((c ^ g) << 4)) = dq[c];
                fence_proxy_async();   // this thread's stores, visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&full_a[s]);
                if (kb8 >= 6) {        // this group's last k-block of the int4 super-stage
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&q_empty[qs]);
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- tile list ------------------------------------------------------------------------
// tiles[0] = count; then int4 {expert (E = shared), first slot, tokens (<= 256), row block}.
// Row block varies fastest so CTAs running together share the token tile through L2.
__global__ void __launch_bounds__(1024)
tile_build_kernel(const int* __restrict__ expert_offsets, int E, int n, int P, int has_shared,
                  int row_blocks, int row_blocks_s, int* __restrict__ tiles) {
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    int cnt = 0, beg = 0;
    if (tid < E) { beg = expert_offsets[tid]; cnt = expert_offsets[tid + 1] - beg; }
    const int ng = (cnt + kBN - 1) / kBN;
    int incl = ng;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    if (lane == 31) wsum[w] = incl;
    __syncthreads();
    int total_routed = 0;
    if (w == 0) {
        const int s = wsum[lane];
        int si = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, si, o);
            if (lane >= o) si += u;
        }
        wsum[lane] = si - s;
        total_routed = __shfl_sync(0xffffffffu, si, 31);
        const int nsh = has_shared ? (n + kBN - 1) / kBN : 0;
        if (lane == 0) { tiles[0] = total_routed * row_blocks + nsh * row_blocks_s; tiles[1] = tiles[2] = tiles[3] = 0; }
    }
    __syncthreads();
    const int base = incl - ng + wsum[w];
    int4* out = reinterpret_cast<int4*>(tiles + kTileHeader);
    for (int j = 0; j < ng; ++j)
        for (int rb = 0; rb < row_blocks; ++rb)
            out[(int64_t)(base + j) * row_blocks + rb] = make_int4(tid, beg + j * kBN, min(kBN, cnt - j * kBN), rb);
}

// Shared-expert tiles appended after the routed tiles (separate tiny kernel keeps the scan simple).
__global__ void tile_append_shared_kernel(const int* __restrict__ expert_offsets, int E, int n, int P,
                                          int row_blocks, int row_blocks_s, int* __restrict__ tiles) {
    // number of routed token tiles
    __shared__ int routed_tiles;
    if (threadIdx.x == 0) {
        int tot = 0;
        for (int e = 0; e < E; ++e) tot += (expert_offsets[e + 1] - expert_offsets[e] + kBN - 1) / kBN;
        routed_tiles = tot;
    }
    __syncthreads();
    const int nsh = (n + kBN - 1) / kBN;
    int4* out = reinterpret_cast<int4*>(tiles + kTileHeader) + (int64_t)routed_tiles * row_blocks;
    for (int i = threadIdx.x; i < nsh * row_blocks_s; i += blockDim.x) {
        const int j = i / row_blocks_s, rb = i - j * row_blocks_s;
        out[i] = make_int4(E, P + j * kBN, min(kBN, n - j * kBN), rb);
    }
}

// Activations into expert order, bf16 -> fp16 (natural feature order for TMA):
// xs[r] = x[sorted_tok[r]] for r < P, xs[P + t] = x[t].
__global__ void __launch_bounds__(256)
gather_x_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ sorted_tok, int P,
                int n, int H, int with_shared, __half* __restrict__ xs) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int gpr = H >> 3;
    const int64_t rows = (int64_t)P + (with_shared ? n : 0);
    if (i >= rows * gpr) return;
    const int64_t r = i / gpr;
    const int grp = (int)(i - r * gpr);
    const int64_t src = r < P ? sorted_tok[r] : r - P;
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + src * H) + grp);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(bp[q]);
        f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
        f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
        const __half2 hh = __floats2half2_rn(f.x, f.y);
        op[q] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    reinterpret_cast<uint4*>(xs + r * H)[grp] = o;
}

// Deterministic combine over fp16 per-slot rows (same order as combine_kernel of the decode
// path: slots k = 0..topk-1, then the shared expert).
__global__ void __launch_bounds__(256)
combine_h_kernel(const __half* __restrict__ ybuf, const int* __restrict__ slot_pos,
                 const float* __restrict__ topk_w, int n, int topk, int H, int P, int has_shared,
                 float* __restrict__ out) {
    const int t = blockIdx.y;
    const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c8 >= (H >> 3)) return;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int k = 0; k <= topk; ++k) {
        if (k == topk && !has_shared) break;
        const int64_t pos = k < topk ? slot_pos[t * topk + k] : (int64_t)P + t;
        const float w = k < topk ? topk_w[t * topk + k] : 1.0f;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(ybuf + pos * H) + c8);
        const __half2* hp = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float2 f = __half22float2(hp[q]);
            acc[2 * q] = __fadd_rn(acc[2 * q], __fmul_rn(w, f.x));
            acc[2 * q + 1] = __fadd_rn(acc[2 * q + 1], __fmul_rn(w, f.y));
        }
    }
    float4* o = reinterpret_cast<float4*>(out + (int64_t)t * H + (c8 << 3));
    o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// fp16 [rows, cols] row-major; box = 64 columns x kBN rows, 128-byte swizzle.
int make_tmap(CUtensorMap* m, const void* base, int64_t rows, int64_t cols, int64_t ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return GSB_ERR_CUDA;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                          estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? GSB_OK : GSB_ERR_CUDA;
}

// Tile list holding only shared-expert tiles over n token rows starting at row 0.
__global__ void tile_shared_only_kernel(int E_marker, int n, int row_blocks, int* __restrict__ tiles) {
    const int nsh = (n + kBN - 1) / kBN;
    if (threadIdx.x == 0) { tiles[0] = nsh * row_blocks; tiles[1] = tiles[2] = tiles[3] = 0; }
    int4* out = reinterpret_cast<int4*>(tiles + kTileHeader);
    for (int i = threadIdx.x; i < nsh * row_blocks; i += blockDim.x) {
        const int j = i / row_blocks, rb = i - j * row_blocks;
        out[i] = make_int4(E_marker, j * kBN, min(kBN, n - j * kBN), rb);
    }
}

constexpr size_t pf_smem(int as, int bs) { return (size_t)as * kABytes + (size_t)bs * kBBytes + 2 * kQBytes + 256; }

}  // namespace

size_t prefill_tile_bytes(int n, int topk, int E, int H, int I) {
    const size_t P = (size_t)n * topk;
    const size_t tok_tiles = (size_t)E + P / kBN + (size_t)n / kBN + 2;
    const size_t rbmax = (size_t)((H / 128 > I / 64) ? H / 128 : I / 64);
    return (kTileHeader + 4 * tok_tiles * rbmax) * sizeof(int);
}

template <int AS, int BS>
static int launch_pair(const PrefillKArgs& g, const PrefillKArgs& w, const CUtensorMap* tm_x, const CUtensorMap* tm_h,
                       int sm_count, cudaStream_t s, cudaEvent_t ev_mid) {
    const size_t smem = pf_smem(AS, BS);
    if (smem > 227 * 1024) return GSB_ERR_UNSUPPORTED;
    if (cudaFuncSetAttribute(prefill_gemm_kernel<true, AS, BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_gemm_kernel<false, AS, BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    prefill_gemm_kernel<true, AS, BS><<<sm_count, kPfThreads, smem, s>>>(g, tm_x[0], tm_x[1], tm_x[2]);
    if (ev_mid) cudaEventRecord(ev_mid, s);
    prefill_gemm_kernel<false, AS, BS><<<sm_count, kPfThreads, smem, s>>>(w, tm_h[0], tm_h[1], tm_h[2]);
    return launch_status();
}

static int run_gemm_pair(const PrefillKArgs& g_in, const PrefillKArgs& w_in, const void* xbase, int64_t xrows,
                         int H, const void* hbase, int64_t hrows, int ldh, int sm_count, cudaStream_t s,
                         cudaEvent_t ev_mid) {
    CUtensorMap tm_x[3], tm_h[3];
    const int boxes[3] = {64, 128, 256};
    for (int i = 0; i < 3; ++i) {
        int st = make_tmap(&tm_x[i], xbase, xrows, H, H, boxes[i]);
        if (st) return st;
        st = make_tmap(&tm_h[i], hbase, hrows, ldh, ldh, boxes[i]);
        if (st) return st;
    }
    // two weight stages and four activation stages measured best on the skewed GLM-scale layer
    return launch_pair<2, 4>(g_in, w_in, tm_x, tm_h, sm_count, s, ev_mid);
}

// Expert parallel, shared expert: this GPU's own tokens through the shared expert, output rows
// into y_shared [n, H] (the tail of the local per-slot row buffer).
int launch_prefill_ep_shared(const PrefillEpArgs& d, cudaStream_t s) {
    if (d.Is <= 0) return GSB_OK;
    gather_x_kernel<<<(unsigned)(((int64_t)d.n * (d.H >> 3) + 255) / 256), 256, 0, s>>>(d.x, nullptr, 0, d.n, d.H, 1, d.xs_local);
    tile_shared_only_kernel<<<1, 256, 0, s>>>(d.El, d.n, d.Is / 64, d.tiles_sh_gu);
    tile_shared_only_kernel<<<1, 256, 0, s>>>(d.El, d.n, d.H / 128, d.tiles_sh_dn);
    PrefillKArgs g{};
    g.packed = nullptr; g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    g.tiles = d.tiles_sh_gu; g.K = d.H; g.Ks = d.H; g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.El;
    g.hbuf = d.hbuf_sh; g.ldh = d.Is; g.ybuf = nullptr; g.H = d.H; g.ydst = nullptr; g.status = d.status;
    PrefillKArgs w = g;
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.tiles = d.tiles_sh_dn; w.K = d.I; w.Ks = d.Is; w.units = d.H / 32; w.units_s = d.H / 32;
    w.hbuf = nullptr; w.ybuf = d.y_shared;
    return run_gemm_pair(g, w, d.xs_local, d.n, d.H, d.hbuf_sh, d.n, d.Is, d.sm_count, s, nullptr);
}

// Expert parallel, routed experts: the rows this GPU received (grouped by local expert in
// recv_x) through its resident experts; the down kernel's epilogue stores every output row
// straight to the GPU that owns the token (ydst) - compute and the return all-to-all in one kernel.
int launch_prefill_ep_routed(const PrefillEpArgs& d, cudaStream_t s) {
    tile_build_kernel<<<1, 1024, 0, s>>>(d.recv_offsets, d.El, 0, 0, 0, d.I / 64, 1, d.tiles_gu);
    tile_build_kernel<<<1, 1024, 0, s>>>(d.recv_offsets, d.El, 0, 0, 0, d.H / 128, 1, d.tiles_dn);
    PrefillKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed); g.shared_packed = nullptr;
    g.tiles = d.tiles_gu; g.K = d.H; g.Ks = d.H; g.units = d.I / 16; g.units_s = 1; g.E = d.El;
    g.hbuf = d.hbuf; g.ldh = d.I; g.ybuf = nullptr; g.H = d.H; g.ydst = nullptr; g.status = d.status;
    PrefillKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed);
    w.tiles = d.tiles_dn; w.K = d.I; w.Ks = d.I; w.units = d.H / 32; w.units_s = 1;
    w.hbuf = nullptr; w.ybuf = nullptr; w.ydst = d.ydst;
    return run_gemm_pair(g, w, d.recv_x, d.recv_cap, d.H, d.hbuf, d.recv_cap, d.I, d.sm_count, s, nullptr);
}

int launch_combine_h(const __half* ybuf, const int* slot_pos, const float* topk_w, int n, int topk, int H,
                     int P, int has_shared, float* out, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    dim3 cgrid((unsigned)(((H >> 3) + 255) / 256), (unsigned)n);
    combine_h_kernel<<<cgrid, 256, 0, s>>>(ybuf, slot_pos, topk_w, n, topk, H, P, has_shared, out);
    return launch_status();
}

int launch_prefill_layer(const PrefillArgs& d, cudaStream_t s) {
    const int P = d.n * d.topk;
    const bool shared = d.Is > 0;
    const int imax = d.I > d.Is ? d.I : d.Is;
    if (d.E > 1024 || d.H % 128 || d.I % 64 || (shared && d.Is % 64)) return GSB_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(d.status, 0, 16, s) != cudaSuccess) return GSB_ERR_CUDA;
    const int64_t rows = (int64_t)P + (shared ? d.n : 0);

    gather_x_kernel<<<(unsigned)((rows * (d.H >> 3) + 255) / 256), 256, 0, s>>>(d.x, d.sorted_tok, P, d.n, d.H,
                                                                              shared ? 1 : 0, d.xs);
    // gate/up tiles: row block = 4 units of (16 gate + 16 up) rows = 64 features
    tile_build_kernel<<<1, 1024, 0, s>>>(d.expert_offsets, d.E, d.n, P, shared ? 1 : 0, d.I / 64, d.Is / 64, d.tiles_gu);
    if (shared) tile_append_shared_kernel<<<1, 256, 0, s>>>(d.expert_offsets, d.E, d.n, P, d.I / 64, d.Is / 64, d.tiles_gu);
    tile_build_kernel<<<1, 1024, 0, s>>>(d.expert_offsets, d.E, d.n, P, shared ? 1 : 0, d.H / 128, d.H / 128, d.tiles_dn);
    if (shared) tile_append_shared_kernel<<<1, 256, 0, s>>>(d.expert_offsets, d.E, d.n, P, d.H / 128, d.H / 128, d.tiles_dn);
    if (d.ev_prep) cudaEventRecord(d.ev_prep, s);

    PrefillKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed);
    g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    g.tiles = d.tiles_gu; g.K = d.H; g.Ks = d.H; g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.E;
    g.hbuf = d.hbuf; g.ldh = imax; g.ybuf = nullptr; g.H = d.H; g.status = d.status;
    PrefillKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed);
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.tiles = d.tiles_dn; w.K = d.I; w.Ks = shared ? d.Is : d.I; w.units = d.H / 32; w.units_s = d.H / 32;
    w.hbuf = nullptr; w.ybuf = d.ybuf;
    const int st = run_gemm_pair(g, w, d.xs, rows, d.H, d.hbuf, rows, imax, d.sm_count, s, d.ev_gate_up);
    if (st) return st;
    if (d.ev_down) cudaEventRecord(d.ev_down, s);

    dim3 cgrid((unsigned)(((d.H >> 3) + 255) / 256), (unsigned)d.n);
    combine_h_kernel<<<cgrid, 256, 0, s>>>(d.ybuf, d.slot_pos, d.topk_w, d.n, d.topk, d.H, P, shared ? 1 : 0, d.out);
    return launch_status();
}

}  // namespace gsb

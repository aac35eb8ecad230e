// Prefill-shaped W4A16 grouped GEMM on the 5th-generation tensor cores (tcgen05 / TMEM).
//
// D[weight row, token] = sum_k W[row, k] * X[token, k] for one tile = (up to 192 token rows of
// one expert) x (128 weight rows = four 32-row units of the tile stream).
//   A operand (M = 128 weight rows): int4 chunks arrive by 1-D bulk copies; eight dequant
//     warps unpack them to fp16 (q - 8) * scale and store them with tcgen05.st straight into
//     TENSOR MEMORY (lane = weight row, one 32-bit column per pair of input columns), a ring of
//     four 64-column k-blocks.  The tensor core reads A from there, so the dequantised weights
//     never touch shared memory: its bandwidth is left to the activation tiles, and a k-block is
//     handed over with one tcgen05.st per thread instead of eight swizzled shared-memory stores
//     and a proxy fence.
//   B operand (N = 16..192 token rows): fp16 activations, gathered into expert order
//     beforehand, loaded by TMA (2-D tiled, 128-byte swizzle, no multicast), five stages.
//   D: fp32 in tensor memory, two buffers of 192 columns so the epilogue of one tile overlaps
//     the main loop of the next.  TMEM columns: [0,192) and [192,384) accumulators, [384,512) A.
// One thread issues tcgen05.mma (cta_group::1, kind::f16, 128 x N x 16, A from TMEM);
// tcgen05.commit releases stages and publishes finished accumulators through mbarriers.
// Epilogue warps read the accumulator with tcgen05.ld: the gate/up kernel pairs gate and up
// rows (lanes l and l^16 of a warp) to fuse SwiGLU and stores fp16 h; the down kernel stores
// the slot's fp16 output row.  Persistent CTAs walk a list of token tiles built on the device.
// All waits are bounded (see mbar_wait); a timeout is recorded in the status word.
#include <cuda.h>

#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

namespace {

constexpr int kDqGroups = 4;           // groups of four unpack warps; group g owns ring stage g
constexpr int kPfThreads = 256 + kDqGroups * 128;   // 4 service warps, 4 epilogue warps, the unpack warps
constexpr int kBN = 192;               // token rows per tile at most (TMA box rows, accumulator columns)
constexpr int kBBytes = kBN * 128;     // one activation stage: 192 token rows x 64 fp16
constexpr int kQBytes = 4 * kChunkBytes;  // one int4 stage: four units x one 512-column chunk
constexpr int kAStages = 4;            // TMEM ring of dequantised k-blocks (32 columns each)
constexpr int kBStages = 6;            // shared-memory ring of activation tiles (deeper: a TMA load takes longer to land
                                       // than three k-blocks take to multiply)
constexpr int kACol0 = 2 * kBN;        // first TMEM column of that ring
constexpr long long kPfWaitLimit = 2000000000LL;
constexpr int kTileHeader = 4;
constexpr int kEpiWarpBytes = 2048;     // per epilogue warp: 32 tokens x 32 features fp16
static_assert(kDqGroups == kAStages && kAStages % 2 == 0 && kBStages % 2 == 0, "an unpack group per ring stage; stages are handed over in pairs");
static_assert(kACol0 + kAStages * 32 <= 512, "accumulators and the A ring must fit the 512 TMEM columns");

struct PrefillKArgs {
    const uint8_t* packed;
    const uint8_t* shared_packed;
    const int* tiles;        // [0] = routed token tiles, [1] = shared-expert token tiles; then int4
                             // {expert, first slot, tokens, 0} per token tile, routed ones first
    int RB, RBs;             // 128-row blocks per routed / shared token tile (tile = token tile x row block)
    int K, Ks;               // input dims (routed / shared)
    int units, units_s;      // 32-row units per expert
    int E;
    __half* hbuf; int ldh;   // gate/up output, natural feature order
    __half* ybuf; int H;     // down output [slots, H]
    __half* const* ydst;     // optional per-row output pointers (expert parallel: rows live on the
                             // token's home GPU and are stored there over NVLink); overrides ybuf
    int* status;
    long long* prof;         // optional [grid][8] wait cycles per role (gsb_prefill_wait_profile)
};

// mbar_wait that also adds the cycles spent waiting to `acc` (try_wait may itself block for a while
// before it answers, so the first call is timed as well)
__device__ __forceinline__ bool mbar_wait_acc(uint64_t* bar, uint32_t parity, long long limit_cycles, long long& acc) {
    const long long start = clock64();
    bool ok = true;
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > limit_cycles) { ok = false; break; }
    }
    acc += clock64() - start;
    return ok;
}

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
// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
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
// One lane of the (converged) warp, the same one every time.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
// This thread's 32 registers -> its TMEM lane, columns taddr .. taddr + 31.
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint4 (&v)[8]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr),
          "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z), "r"(v[1].w),
          "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z), "r"(v[3].w),
          "r"(v[4].x), "r"(v[4].y), "r"(v[4].z), "r"(v[4].w), "r"(v[5].x), "r"(v[5].y), "r"(v[5].z), "r"(v[5].w),
          "r"(v[6].x), "r"(v[6].y), "r"(v[6].z), "r"(v[6].w), "r"(v[7].x), "r"(v[7].y), "r"(v[7].z), "r"(v[7].w)
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

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

// tile idx -> (token tile, row block); row block varies fastest so CTAs running together share
// the token tile through L2
__device__ __forceinline__ PfTile pf_tile(const PrefillKArgs& a, int idx) {
    const int routed = a.tiles[0] * a.RB;
    int tt, rb;
    if (idx < routed) { tt = idx / a.RB; rb = idx - tt * a.RB; }
    else { const int j = idx - routed; const int q = j / a.RBs; tt = a.tiles[0] + q; rb = j - q * a.RBs; }
    const int4 t = reinterpret_cast<const int4*>(a.tiles + kTileHeader)[tt];
    PfTile r;
    r.expert = t.x; r.slot0 = t.y; r.ntok = t.z; r.rb = rb;
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

template <bool GU, int QS>
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_gemm_kernel(const PrefillKArgs a, const __grid_constant__ CUtensorMap tmap_b64,
                    const __grid_constant__ CUtensorMap tmap_b128, const __grid_constant__ CUtensorMap tmap_b192) {
    extern __shared__ uint8_t smem_raw[];
    // the kernel has no static shared memory, so the dynamic window starts 1024-byte aligned (the
    // swizzled tiles need that); checked below, a misaligned base is reported instead of used
    uint8_t* smem = smem_raw;
    constexpr int BS = kBStages;
    uint8_t* sB = smem;                                   // [BS][24 KiB]
    uint8_t* sQ = sB + BS * kBBytes;                      // [QS][4 chunks]
    uint8_t* sE = sQ + QS * kQBytes;                      // [4 epilogue warps][2 KiB] transposition staging
    uint64_t* bars = reinterpret_cast<uint64_t*>(sE + 4 * kEpiWarpBytes);
    // Stages are handed over in PAIRS of k-blocks: the tensor pipe drains and idles while the MMA warp
    // waits, fences and commits, so it does that once per eight MMAs, not once per four.
    uint64_t* full = bars;                     // [kAStages / 2] the pair's 8 unpack warps -> MMA
    uint64_t* empty = full + kAStages / 2;     // [kAStages / 2] MMA commit -> unpack warps
    uint64_t* full_b = empty + kAStages / 2;   // [BS / 2] activation TMA (two loads) -> MMA
    uint64_t* empty_b = full_b + BS / 2;       // [BS / 2] MMA commit -> producer
    uint64_t* q_full = empty_b + BS / 2;       // [QS] bulk copy -> dequant
    uint64_t* q_empty = q_full + QS;           // [QS] dequant -> producer
    uint64_t* acc_full = q_empty + QS;         // [2] MMA commit -> epilogue
    uint64_t* acc_empty = acc_full + 2;        // [2] epilogue -> MMA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (smem_u32(smem_raw) & 1023u) {
        if (tid == 0 && atomicCAS(a.status + kStatusCode, 0, GSB_ERR_LAUNCH) == 0) a.status[kStatusWhere] = 199;
        return;
    }
    if (tid == 0) {
        for (int i = 0; i < kAStages / 2; ++i) { mbar_init(&full[i], 8); mbar_init(&empty[i], 1); }
        for (int i = 0; i < BS / 2; ++i) { mbar_init(&full_b[i], 1); mbar_init(&empty_b[i], 1); }
        for (int i = 0; i < QS; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 4 * kDqGroups); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], 4); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int ntiles = a.tiles[0] * a.RB + a.tiles[1] * a.RBs;

    if (warp == 0) {
        // ------------- producer of the activation tiles (TMA) -------------
        if (lane == 0) {
            uint32_t sb = 0, phb = 0;      // ring position and the parity of its current use
            bool dead = false;
            long long w_b = 0;
            const long long t_begin = clock64();
            for (int ti = blockIdx.x; ti < ntiles && !dead && !*abort_flag; ti += gridDim.x) {
                const PfTile t = pf_tile(a, ti);
                // the smallest box that covers the tile's rows: a ragged tile does not pull 192 rows
                const CUtensorMap* tm = t.nround <= 64 ? &tmap_b64 : (t.nround <= 128 ? &tmap_b128 : &tmap_b192);
                const uint32_t rows = t.nround <= 64 ? 64u : (t.nround <= 128 ? 128u : 192u);
                for (int kb = 0; kb < t.nkb; kb += 2) {   // sb counts pairs of stages
                    if (!mbar_wait_acc(&empty_b[sb], phb ^ 1u, kPfWaitLimit, w_b)) { pf_timeout(a, abort_flag, 2); dead = true; break; }
                    mbar_arrive_expect_tx(&full_b[sb], 2u * rows * 128u);
                    tma_load_2d(sB + (2 * sb) * kBBytes, tm, kb * 64, t.slot0, &full_b[sb]);
                    tma_load_2d(sB + (2 * sb + 1) * kBBytes, tm, kb * 64 + 64, t.slot0, &full_b[sb]);
                    if (++sb == (uint32_t)(BS / 2)) { sb = 0; phb ^= 1u; }
                }
            }
            if (a.prof) { long long* p = a.prof + (size_t)blockIdx.x * 16; p[0] = clock64() - t_begin; p[2] = w_b; }
        }
    } else if (warp == 2) {
        // ------------- producer of the int4 chunks (bulk copies), a thread of its own: it runs ahead by
        // the depth of the int4 ring whatever the state of the activation ring -------------
        if (lane == 0) {
            uint32_t qs = 0, qph = 0;
            bool dead = false;
            long long w_q = 0;
            for (int ti = blockIdx.x; ti < ntiles && !dead && !*abort_flag; ti += gridDim.x) {
                const PfTile t = pf_tile(a, ti);
                for (int c = 0; c < (t.nkb >> 3); ++c) {
                    if (!mbar_wait_acc(&q_empty[qs], qph ^ 1u, kPfWaitLimit, w_q)) { pf_timeout(a, abort_flag, 1); dead = true; break; }
                    mbar_arrive_expect_tx(&q_full[qs], kQBytes);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        bulk_g2s(sQ + qs * kQBytes + u * kChunkBytes,
                                 t.chunks + (int64_t)u * t.unit_stride + (int64_t)c * kChunkBytes, kChunkBytes, &q_full[qs]);
                    if (++qs == (uint32_t)QS) { qs = 0; qph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------- MMA issuer -------------
        // The tensor pipe idles whenever this warp's instruction stream is not at a tcgen05.mma, so the
        // loop is kept short: all 32 lanes run it (warp-uniform values stay in uniform registers; one
        // elected lane issues the tcgen05 instructions), the four ring stages are unrolled (a tile has a
        // multiple of eight k-blocks, so every tile starts at stage 0 and stage numbers are constants),
        // and whether the NEXT stage is full is asked (non-blocking) before this stage's MMAs are issued
        // and looked at after them.
        const bool leader = elect_one();
        uint32_t pha = 0, tl = 0, sb = 0, phb = 0;
        bool dead = false;
        long long w_acc = 0, w_a = 0, w_bf = 0;
        const long long t_begin = clock64();
        const uint32_t a_tmem0 = tmem_base + (uint32_t)kACol0;
        const uint64_t bd0 = make_desc_sw128(smem_u32(sB));
        uint32_t ready_a = mbar_test_wait(&full[0], 0), ready_b = mbar_test_wait(&full_b[0], 0);
        for (int ti = blockIdx.x; ti < ntiles && !dead && !*abort_flag; ti += gridDim.x, ++tl) {
            const PfTile t = pf_tile(a, ti);
            const uint32_t buf = tl & 1u;
            if (!mbar_wait_acc(&acc_empty[buf], ((tl >> 1) & 1u) ^ 1u, kPfWaitLimit, w_acc)) { pf_timeout(a, abort_flag, 3); break; }
            const uint32_t d_tmem = tmem_base + buf * (uint32_t)kBN;
            const uint32_t idesc = make_idesc((uint32_t)t.nround);
            uint32_t acc = 0;    // the tile's first MMA overwrites the accumulator
            for (int kb = 0; kb < t.nkb && !dead; kb += kAStages) {
#pragma unroll
                for (int pr = 0; pr < kAStages / 2; ++pr) {   // pair of ring stages 2 pr, 2 pr + 1; sb counts activation pairs
                    if (!ready_a && !mbar_wait_acc(&full[pr], pha, kPfWaitLimit, w_a)) { pf_timeout(a, abort_flag, 4); dead = true; break; }
                    if (!ready_b && !mbar_wait_acc(&full_b[sb], phb, kPfWaitLimit, w_bf)) { pf_timeout(a, abort_flag, 8); dead = true; break; }
                    tc_fence_after();
                    const uint32_t sbn = sb + 1 == (uint32_t)(BS / 2) ? 0u : sb + 1, phn = sb + 1 == (uint32_t)(BS / 2) ? phb ^ 1u : phb;
                    ready_a = mbar_test_wait(&full[(pr + 1) % (kAStages / 2)], pr + 1 == kAStages / 2 ? pha ^ 1u : pha);
                    ready_b = mbar_test_wait(&full_b[sbn], phn);
                    if (leader) {
                        const uint64_t bd = bd0 + (uint64_t)(sb * (uint32_t)(2 * (kBBytes >> 4)));
#pragma unroll
                        for (int k8 = 0; k8 < 8; ++k8)
                            tc_mma_f16_ts(d_tmem, a_tmem0 + (uint32_t)(pr * 64 + k8 * 8),
                                          bd + (uint64_t)((k8 >> 2) * (kBBytes >> 4) + (k8 & 3) * 2), idesc, k8 ? 1u : acc);
                        tc_commit(&empty[pr]);
                        tc_commit(&empty_b[sb]);
                    }
                    acc = 1u;
                    sb = sbn; phb = phn;
                }
                pha ^= 1u;
            }
            if (dead) break;
            if (leader) tc_commit(&acc_full[buf]);
        }
        if (a.prof && lane == 0) { long long* p = a.prof + (size_t)blockIdx.x * 16; p[3] = w_acc; p[4] = w_a; p[1] = w_bf; p[9] = clock64() - t_begin; }
    } else if (warp >= 4 && warp < 8) {
        // ------------- epilogue (warp % 4 selects the TMEM lane quarter) -------------
        const int q = warp & 3;
        uint32_t tl = 0;
        long long w_full = 0, w_ld = 0;
        const long long t_begin = clock64();
        for (int ti = blockIdx.x; ti < ntiles; ti += gridDim.x, ++tl) {
            const PfTile t = pf_tile(a, ti);
            const uint32_t buf = tl & 1u;
            if (*abort_flag || !mbar_wait_acc(&acc_full[buf], (tl >> 1) & 1u, kPfWaitLimit, w_full)) {
                if (!*abort_flag) pf_timeout(a, abort_flag, 5);
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * (uint32_t)kBN;
            // A lane holds ONE weight row (feature) for 32 tokens, but memory wants a token's features side
            // by side: the chunk goes through this warp's 2 KiB of shared memory as [token][feature], and
            // comes back as 16-byte vectors - eight features of one token per lane, so a store instruction
            // writes 512 bytes instead of 32 two-byte pieces.
            __half* stg = reinterpret_cast<__half*>(sE + q * kEpiWarpBytes);
            for (int c0 = 0; c0 < t.nround; c0 += 32) {
                uint32_t r[32];
                const long long t_l = a.prof ? clock64() : 0;
                tmem_ld32(taddr + (uint32_t)c0, r);
                tmem_ld_wait();
                if (a.prof) w_ld += clock64() - t_l;
                if (GU) {
                    // lanes 0..15 hold gate rows, lanes 16..31 the matching up rows: 16 features per token
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float v0 = __uint_as_float(r[j]), v1 = __uint_as_float(r[j + 1]);
                        const float send = (lane < 16) ? v1 : v0;
                        const float recv = __shfl_xor_sync(0xffffffffu, send, 16);
                        const float g = (lane < 16) ? v0 : recv;
                        const float u = (lane < 16) ? recv : v1;
                        // token j (lanes 0..15) and token j + 1 (lanes 16..31), 32 bytes each, back to back
                        stg[j * 16 + lane] = sat_half(__fmul_rn(silu_ref(g), u));
                    }
                    __syncwarp();
                    const int feat = t.rb * 64 + q * 16 + (lane & 1) * 8;
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int n = c0 + k * 16 + (lane >> 1);
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + (k * 16 + (lane >> 1)) * 16 + (lane & 1) * 8);
                        if (n < t.ntok) *reinterpret_cast<uint4*>(a.hbuf + (int64_t)(t.slot0 + n) * a.ldh + feat) = v;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) stg[j * 32 + lane] = sat_half(__uint_as_float(r[j]));
                    __syncwarp();
                    const int feat = t.rb * 128 + q * 32 + (lane & 3) * 8;
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const int n = c0 + k * 8 + (lane >> 2);
                        const uint4 v = *reinterpret_cast<const uint4*>(stg + (k * 8 + (lane >> 2)) * 32 + (lane & 3) * 8);
                        if (n < t.ntok) {
                            __half* yrow = a.ydst ? a.ydst[t.slot0 + n] : a.ybuf + (int64_t)(t.slot0 + n) * a.H;
                            *reinterpret_cast<uint4*>(yrow + feat) = v;
                        }
                    }
                }
                __syncwarp();   // the staging area is rewritten by the next chunk
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
        if (a.prof && q == 0 && lane == 0) { long long* p = a.prof + (size_t)blockIdx.x * 16; p[10] = w_full; p[11] = w_ld; p[12] = clock64() - t_begin; }
    } else if (warp >= 8) {
        // ------------- dequant: int4 chunk pieces -> fp16 rows of the A ring in TMEM -------------
        // Four groups of four warps; group g unpacks the k-blocks kb with kb % 4 == g into ring stage g
        // (a tile has a multiple of eight k-blocks, so that holds across tiles).  A thread owns one row
        // of the 128-row tile = one TMEM lane (warp % 4 is the lane quarter it may access).  The work of a
        // k-block is a latency chain (shared-memory loads, ~100 ALU operations, the TMEM store), so it
        // takes this many warps in flight to produce a k-block as fast as the tensor core consumes one.
        const int d = tid - 256;
        const int grp = d >> 7;                        // ring stage and k-block residue of this group
        const int R = d & 127;                         // row of the tile (= TMEM lane)
        const int uu = R >> 5, m = (R >> 4) & 1, h = (R >> 3) & 1, g = R & 7;
        const uint32_t a_st = tmem_base + ((uint32_t)(R & ~31) << 16) + (uint32_t)kACol0 + (uint32_t)grp * 32u;
        uint32_t pha = 0;                              // parity of the stage's current use
        uint32_t qs = 0, qph = 0;
        bool dead = false;
        long long w_qf = 0, w_ea = 0, w_alu = 0, w_pub = 0, w_st = 0;
        const long long t_begin = clock64();
        for (int ti = blockIdx.x; ti < ntiles && !dead; ti += gridDim.x) {
            const PfTile t = pf_tile(a, ti);
            for (int kb = grp; kb < t.nkb; kb += kDqGroups) {
                const int kb8 = kb & 7;
                if (kb8 == grp) {
                    if (*abort_flag || !mbar_wait_acc(&q_full[qs], qph, kPfWaitLimit, w_qf)) {
                        if (!*abort_flag) pf_timeout(a, abort_flag, 6);
                        dead = true; break;
                    }
                }
                const long long t0 = a.prof ? clock64() : 0;
                const int ks = kb8 >> 1, tq0 = (kb8 & 1) << 1;
                const uint8_t* chunk = sQ + qs * kQBytes + uu * kChunkBytes;
                const uint4* piece = reinterpret_cast<const uint4*>(chunk + (ks * 2 + m) * 1024 + h * 512 + (g * 4 + tq0) * 16);
                // A row's two 16-byte pieces sit 64 bytes from the next row's, so eight lanes reading "their
                // first piece" fall on two bank groups (4-way conflict).  Rows 2,3,6,7 read their second piece
                // first: four bank groups per load, 2-way - the best this layout allows for one k-block, and
                // it matters: the shared-memory pipe also feeds the tensor core its activation tiles.
                const int swp = (g >> 1) & 1;
                const uint4 wa = piece[swp], wb = piece[swp ^ 1];
                const uint4 wv0 = swp ? wb : wa, wv1 = swp ? wa : wb;
                const __half sc = reinterpret_cast<const __half*>(chunk + kChunkWeightBytes)[(ks * 2 + m) * 16 + g + 8 * h];
                const __half2 s2 = __half2half2(sc);
                const uint32_t wq[8] = {wv0.x, wv0.y, wv0.z, wv0.w, wv1.x, wv1.y, wv1.z, wv1.w};
                uint4 dq[8];   // unpacked in registers first: only the store needs the stage to be free
#pragma unroll
                for (int c = 0; c < 8; ++c) dq[c] = dequant8(wq[c], s2);
                long long t1 = 0;
                if (a.prof) { t1 = clock64(); w_alu += t1 - t0 + (long long)(dq[0].x & 0u); }
                // unpacked in registers before the wait: only the store needs the stage to be free
                if (!mbar_wait_acc(&empty[grp >> 1], pha ^ 1u, kPfWaitLimit, w_ea)) { pf_timeout(a, abort_flag, 7); dead = true; break; }
                const long long t3 = a.prof ? clock64() : 0;
                tc_fence_after();      // the MMAs that read this stage (their commit released it) before the store
                tmem_st32(a_st, dq);
                tmem_st_wait();
                tc_fence_before();     // the store before the MMA thread's reads, across the arrive below
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[grp >> 1]);
                if (a.prof) w_st += clock64() - t3;
                pha ^= 1u;
                if (kb8 >= 4) {        // this group's last k-block of the int4 stage; the store above took the
                                       // unpacked words, so every load from the stage has returned
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&q_empty[qs]);
                    if (++qs == (uint32_t)QS) { qs = 0; qph ^= 1u; }
                }
            }
        }
        if (a.prof && d == 0) { long long* p = a.prof + (size_t)blockIdx.x * 16; p[6] = w_qf; p[7] = w_ea; p[5] = w_alu; p[8] = w_pub; p[13] = w_st; p[14] = clock64() - t_begin; }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem_base, 512);
}

// ---- token-tile list ------------------------------------------------------------------
// tiles[0] = routed token tiles, tiles[1] = shared-expert token tiles, then int4 {expert
// (shared_marker = shared), first slot, tokens (<= 192), 0} per token tile, routed ones first.  Both GEMM kernels
// read the one list (they differ in the row blocks per token tile).  An expert's rows are cut into
// the fewest tiles of at most 192 rows, of equal size up to one row: a 200-row expert becomes
// 100 + 100, not 192 + 8 (a tile pays a full pass of weight unpacking however few rows it has).
__device__ __forceinline__ int4 token_tile(int expert, int beg, int cnt, int nt, int j) {
    const int base = cnt / nt, rem = cnt - base * nt;
    return make_int4(expert, beg + j * base + min(j, rem), base + (j < rem ? 1 : 0), 0);
}

__global__ void __launch_bounds__(1024)
tile_list_kernel(const int* __restrict__ expert_offsets, int E, int shared_marker, int n_shared, int shared_slot0,
                 int* __restrict__ tiles) {
    __shared__ int wsum[32];
    __shared__ int routed_total;
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
    if (w == 0) {
        const int s = wsum[lane];
        int si = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, si, o);
            if (lane >= o) si += u;
        }
        wsum[lane] = si - s;
        if (lane == 31) routed_total = si;
    }
    __syncthreads();
    const int nsh = (n_shared + kBN - 1) / kBN;
    if (tid == 0) { tiles[0] = routed_total; tiles[1] = nsh; tiles[2] = tiles[3] = 0; }
    const int base = incl - ng + wsum[w];
    int4* out = reinterpret_cast<int4*>(tiles + kTileHeader);
    for (int j = 0; j < ng; ++j) out[base + j] = token_tile(tid, beg, cnt, ng, j);
    for (int j = tid; j < nsh; j += 1024) out[routed_total + j] = token_tile(shared_marker, shared_slot0, n_shared, nsh, j);
}

// Activations into expert order (natural feature order for TMA), from the fp16 copy the
// router-logits launch left behind: xs[r] = xh[sorted_tok[r]] for r < P, xs[P + t] = xh[t].
// (Fetching the rows by index in the GEMM's producer instead - TMA gather4, four 128-byte rows per
// instruction - was built and is correct, but 48 such instructions per k-block keep the TMA unit busy
// for ~2200 cycles against the ~380 the tensor core needs: 4x slower than this pass plus tiled loads.)
// Two rows per block, each thread up to four 16-byte groups of each: eight independent loads are in flight
// per thread before the first store (one load per thread left the pass bound by latency, 2.2 TB/s).
__global__ void __launch_bounds__(256)
gather_x_kernel(const __half* __restrict__ xh, const int* __restrict__ sorted_tok, int P,
                int n, int H, int with_shared, __half* __restrict__ xs) {
    const int gpr = H >> 3;
    const int64_t rows = (int64_t)P + (with_shared ? n : 0);
    const int64_t r0 = (int64_t)blockIdx.x * 2;
    const uint4* sp[2];
    uint4* dp[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int64_t r = r0 + j < rows ? r0 + j : r0;            // an odd row count: the last block has one row
        const int64_t src = r < P ? sorted_tok[r] : r - P;
        sp[j] = reinterpret_cast<const uint4*>(xh + src * H);
        dp[j] = reinterpret_cast<uint4*>(xs + r * H);
    }
    const int nj = r0 + 1 < rows ? 2 : 1;
    for (int g0 = threadIdx.x; g0 < gpr; g0 += 4 * 256) {
        uint4 v[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (j < nj && g0 + u * 256 < gpr) v[j][u] = __ldg(sp[j] + g0 + u * 256);
        // streaming stores: the 0.9 GB written here must not push the token-order matrix (which every row is
        // read from top-k times) out of L2
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int u = 0; u < 4; ++u)
                if (j < nj && g0 + u * 256 < gpr) __stcs(dp[j] + g0 + u * 256, v[j][u]);
    }
}

// Deterministic combine over fp16 per-slot rows (same order as combine_kernel of the decode
// path: slots k = 0..topk-1, then the shared expert); with `residual` the layer's pre-norm
// residual add rides the same pass (out = residual + sum).
__global__ void __launch_bounds__(256)
combine_h_kernel(const __half* __restrict__ ybuf, const int* __restrict__ slot_pos,
                 const float* __restrict__ topk_w, int n, int topk, int H, int P, int has_shared,
                 const float* residual, float* out) {
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
    if (residual) {   // hidden + mlp, the layer's sum complete before the add (src/model_gpu.cpp:1502 of the reference)
        const float4* rp = reinterpret_cast<const float4*>(residual + (int64_t)t * H + (c8 << 3));
        const float4 r0 = rp[0], r1 = rp[1];   // out may be the residual itself: read before the stores
        o[0] = make_float4(__fadd_rn(r0.x, acc[0]), __fadd_rn(r0.y, acc[1]), __fadd_rn(r0.z, acc[2]), __fadd_rn(r0.w, acc[3]));
        o[1] = make_float4(__fadd_rn(r1.x, acc[4]), __fadd_rn(r1.y, acc[5]), __fadd_rn(r1.z, acc[6]), __fadd_rn(r1.w, acc[7]));
        return;
    }
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

// fp16 [rows, cols] row-major; box = 64 columns x box_rows rows, 128-byte swizzle.
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

constexpr size_t pf_smem(int qs) { return (size_t)kBStages * kBBytes + (size_t)qs * kQBytes + 4 * kEpiWarpBytes + 256; }
constexpr int kPfQStages = 2;
static_assert(pf_smem(kPfQStages) <= 227 * 1024, "stages exceed the shared memory of an SM");

}  // namespace

size_t prefill_tile_bytes(int n, int topk, int E) {
    const size_t P = (size_t)n * topk;
    const size_t tok_tiles = (size_t)E + P / kBN + (size_t)n / kBN + 2;
    return (kTileHeader + 4 * tok_tiles) * sizeof(int);
}

// optional wait-cycle profile of the two GEMM kernels (see gsb_prefill_wait_profile)
static long long* g_pf_prof = nullptr;

static int run_gemm_pair(const PrefillKArgs& g_in, const PrefillKArgs& w_in, const void* xbase, int64_t xrows,
                         int H, const void* hbase, int64_t hrows, int ldh, int sm_count, cudaStream_t s,
                         cudaEvent_t ev_mid) {
    CUtensorMap tm_x[3], tm_h[3];
    const int boxes[3] = {64, 128, kBN};
    for (int i = 0; i < 3; ++i) {
        int st = make_tmap(&tm_x[i], xbase, xrows, H, H, boxes[i]);
        if (st) return st;
        st = make_tmap(&tm_h[i], hbase, hrows, ldh, ldh, boxes[i]);
        if (st) return st;
    }
    PrefillKArgs g = g_in, w = w_in;
    g.prof = g_pf_prof;
    w.prof = g_pf_prof ? g_pf_prof + 16 * 1024 : nullptr;
    constexpr size_t smem = pf_smem(kPfQStages);
    if (cudaFuncSetAttribute(prefill_gemm_kernel<true, kPfQStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
        cudaFuncSetAttribute(prefill_gemm_kernel<false, kPfQStages>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    prefill_gemm_kernel<true, kPfQStages><<<sm_count, kPfThreads, smem, s>>>(g, tm_x[0], tm_x[1], tm_x[2]);
    if (ev_mid) cudaEventRecord(ev_mid, s);
    prefill_gemm_kernel<false, kPfQStages><<<sm_count, kPfThreads, smem, s>>>(w, tm_h[0], tm_h[1], tm_h[2]);
    return launch_status();
}

// Expert parallel, shared expert: this GPU's own tokens through the shared expert, output rows
// into y_shared [n, H] (the tail of the local per-slot row buffer).
int launch_prefill_ep_shared(const PrefillEpArgs& d, cudaStream_t s) {
    if (d.Is <= 0) return GSB_OK;
    tile_list_kernel<<<1, 1024, 0, s>>>(nullptr, 0, d.El, d.n, 0, d.tiles_sh);
    PrefillKArgs g{};
    g.packed = nullptr; g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    g.tiles = d.tiles_sh; g.RB = 1; g.RBs = d.Is / 64;
    g.K = d.H; g.Ks = d.H; g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.El;
    g.hbuf = d.hbuf_sh; g.ldh = d.Is; g.ybuf = nullptr; g.H = d.H; g.ydst = nullptr; g.status = d.status;
    PrefillKArgs w = g;
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.RBs = d.H / 128; w.K = d.I; w.Ks = d.Is; w.units = d.H / 32; w.units_s = d.H / 32;
    w.hbuf = nullptr; w.ybuf = d.y_shared;
    return run_gemm_pair(g, w, d.xs_local, d.n, d.H, d.hbuf_sh, d.n, d.Is, d.sm_count, s, nullptr);
}

// Expert parallel, routed experts: the rows this GPU received (grouped by local expert in
// recv_x) through its resident experts; the down kernel's epilogue stores every output row
// straight to the GPU that owns the token (ydst) - compute and the return all-to-all in one kernel.
int launch_prefill_ep_routed(const PrefillEpArgs& d, cudaStream_t s, int what) {
    const int e0 = d.e_end > d.e_begin ? d.e_begin : 0, e1 = d.e_end > d.e_begin ? d.e_end : d.El;
    // tile experts count from e0: the offsets and the weight streams are handed over from there
    if (what & 1) tile_list_kernel<<<1, 1024, 0, s>>>(d.recv_offsets + e0, e1 - e0, d.El, 0, 0, d.tiles);
    if (!(what & 2)) return launch_status();
    const size_t gu_expert = (size_t)(d.I / 16) * (d.H / kChunkCols) * kChunkBytes;
    const size_t dn_expert = (size_t)(d.H / 32) * (d.I / kChunkCols) * kChunkBytes;
    PrefillKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed) + (size_t)e0 * gu_expert; g.shared_packed = nullptr;
    g.tiles = d.tiles; g.RB = d.I / 64; g.RBs = 1;
    g.K = d.H; g.Ks = d.H; g.units = d.I / 16; g.units_s = 1; g.E = d.El;
    g.hbuf = d.hbuf; g.ldh = d.I; g.ybuf = nullptr; g.H = d.H; g.ydst = nullptr; g.status = d.status;
    PrefillKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed) + (size_t)e0 * dn_expert;
    w.RB = d.H / 128; w.K = d.I; w.Ks = d.I; w.units = d.H / 32; w.units_s = 1;
    w.hbuf = nullptr; w.ybuf = nullptr; w.ydst = d.ydst;
    return run_gemm_pair(g, w, d.recv_x, d.recv_cap, d.H, d.hbuf, d.recv_cap, d.I, d.sm_count, s, nullptr);
}

int launch_combine_h(const __half* ybuf, const int* slot_pos, const float* topk_w, int n, int topk, int H,
                     int P, int has_shared, const float* residual, float* out, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    dim3 cgrid((unsigned)(((H >> 3) + 255) / 256), (unsigned)n);
    combine_h_kernel<<<cgrid, 256, 0, s>>>(ybuf, slot_pos, topk_w, n, topk, H, P, has_shared, residual, out);
    return launch_status();
}

int launch_prefill_layer(const PrefillArgs& d, cudaStream_t s) {
    const int P = d.n * d.topk;
    const bool shared = d.Is > 0;
    const int Id = d.Id > 0 ? d.Id : d.I, Isd = shared ? (d.Isd > 0 ? d.Isd : d.Is) : Id;
    const int imax = Id > Isd ? Id : Isd;
    if (d.E > 1024 || d.H % 128 || d.I % 64 || (shared && d.Is % 64)) return GSB_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(d.status, 0, 16, s) != cudaSuccess) return GSB_ERR_CUDA;
    const int64_t rows = (int64_t)P + (shared ? d.n : 0);

    if (!d.xh_ready) {
        const int st0 = launch_xprep(d.x, d.xh, d.n, d.H, 1, s);
        if (st0) return st0;
    }
    if (rows > 0)
        gather_x_kernel<<<(unsigned)((rows + 1) / 2), 256, 0, s>>>(d.xh, d.sorted_tok, P, d.n, d.H, shared ? 1 : 0, d.xs);
    tile_list_kernel<<<1, 1024, 0, s>>>(d.expert_offsets, d.E, d.E, shared ? d.n : 0, P, d.tiles);
    if (d.ev_prep) cudaEventRecord(d.ev_prep, s);

    PrefillKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed);
    g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    // gate/up row block = 4 units of (16 gate + 16 up) rows = 64 features; down row block = 128 rows
    g.tiles = d.tiles; g.RB = d.I / 64; g.RBs = shared ? d.Is / 64 : 1;
    g.K = d.H; g.Ks = d.H; g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.E;
    g.hbuf = d.hbuf; g.ldh = imax; g.ybuf = nullptr; g.H = d.H; g.status = d.status;
    PrefillKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed);
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.RB = d.H / 128; w.RBs = d.H / 128;
    w.K = Id; w.Ks = Isd; w.units = d.H / 32; w.units_s = d.H / 32;
    w.hbuf = nullptr; w.ybuf = d.ybuf;
    const int st = run_gemm_pair(g, w, d.xs, rows, d.H, d.hbuf, rows, imax, d.sm_count, s, d.ev_gate_up);
    if (st) return st;
    if (d.ev_down) cudaEventRecord(d.ev_down, s);
    return launch_combine_h(d.ybuf, d.slot_pos, d.topk_w, d.n, d.topk, d.H, P, shared ? 1 : 0, d.residual, d.out, s);
}

}  // namespace gsb

extern "C" int gsb_prefill_wait_profile(long long* device_buffer) {
    gsb::g_pf_prof = device_buffer;
    return GSB_OK;
}

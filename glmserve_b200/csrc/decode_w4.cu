// Decode-shaped W4A16 grouped GEMM: a bandwidth-bound split-K kernel over the tile stream.
//
// One persistent CTA per SM.  Work item = (segment, unit): a segment is up to 8 token rows
// of one expert (the shared expert is expert index E with every token), a unit is 32 weight
// rows over the full input dimension.  Roles inside the CTA:
//   warp 0           producer: one lane streams the item's chunks (16.5 KiB stages, one
//                    contiguous 1-D bulk copy each) into a shared-memory ring, completion
//                    on mbarriers, running ahead across item boundaries
//   warps 1..16      consumers: each owns one (128-column kstep, half unit) of every stage
//                    = split-K across warps; unpacks int4 to exact fp16 integers in
//                    registers, mma.sync m16n8k16 against the segment's fp16 activations
//                    (held in shared memory), applies the fp16 group scale to the fp32
//                    accumulator once per 128 columns
//   warps 17..20     epilogue: sums the 8 K-split partials of each half unit in fixed order,
//                    fuses SwiGLU (gate/up kernel) and stores fp16 h, or stores the fp32
//                    down-projection row of the slot (down kernel)
// Nothing is accumulated with atomics; every reduction order is fixed, so results do not
// depend on the grid or on timing.  Every wait is bounded: on a timeout the CTA records
// where in the status word and all its loops leave.
#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

namespace {

constexpr int kConsumerWarps = 16;
constexpr int kEpiWarps = 4;
constexpr int kDecodeThreads = (1 + kConsumerWarps + kEpiWarps) * 32;  // 672
constexpr int kStageChunks = 2;
constexpr int kStageBytes = kStageChunks * kChunkBytes;  // 16896
constexpr int kMaxStages = 12;
constexpr int kRedBytes = kConsumerWarps * 4 * 32 * 4;   // one partial buffer: 8 KiB
constexpr int kXPad = 64;                                 // bytes of padding per activation row
constexpr long long kWaitLimit = 2000000000LL;              // SM cycles, about one second
constexpr int kSegHeader = 4;                             // ints before the first segment

struct DecodeKArgs {
    const uint8_t* packed;         // routed tile stream
    const uint8_t* shared_packed;  // shared expert tile stream (or null)
    const int* segs;               // [0] = nseg, [1] = n shared segs; then int4 per segment
    const int* sorted_tok;         // gate/up: token of a routed slot
    const __half* bsrc;            // gate/up: xp [n, K]; down: hbuf [P + n, ldb]
    int ldb;                       // row stride of bsrc in halves
    int K;                         // input dim of routed experts
    int Ks;                        // input dim of the shared expert (gate/up: = K)
    int units;                     // units per routed expert
    int units_s;                   // units per shared expert
    int E;                         // routed experts (shared expert id)
    int P;                         // routed slots (n * topk)
    __half* hbuf;                  // gate/up output [P + n, ldh]
    int ldh;
    float* ybuf;                   // down output [P + n, H]
    int H;
    int nstage;
    int* status;
};

struct Item {
    int seg, unit, expert, slot_begin, ntok, K;
    const uint8_t* chunks;  // first chunk of this (expert, unit)
    int nchunk;
};

__device__ __forceinline__ Item decode_item(const DecodeKArgs& a, int64_t it, int nshared_seg) {
    Item r;
    const int64_t shared_items = (int64_t)nshared_seg * a.units_s;
    bool sh = it < shared_items;
    int64_t local = sh ? it : it - shared_items;
    const int U = sh ? a.units_s : a.units;
    r.seg = (int)(local / U) + (sh ? 0 : nshared_seg);
    r.unit = (int)(local % U);
    const int4 sg = reinterpret_cast<const int4*>(a.segs + kSegHeader)[r.seg];
    r.expert = sg.x;
    r.slot_begin = sg.y;
    r.ntok = sg.z;
    r.K = sh ? a.Ks : a.K;
    r.nchunk = r.K / kChunkCols;
    const uint8_t* base = sh ? a.shared_packed : a.packed;
    const int64_t e_local = sh ? 0 : r.expert;
    r.chunks = base + ((e_local * U + r.unit) * (int64_t)r.nchunk) * kChunkBytes;
    return r;
}

__device__ __forceinline__ void record_timeout(const DecodeKArgs& a, volatile int* abort_flag,
                                               int where) {
    *abort_flag = 1;
    if (atomicCAS(a.status + kStatusCode, 0, GSB_ERR_TIMEOUT) == 0) {
        a.status[kStatusWhere] = where;
        a.status[kStatusAux] = (int)blockIdx.x;
    }
}

// eight int4 (one word, tile-stream nibble order) -> four fp16x2 of (q - 8), exact
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t& p01, uint32_t& p23, uint32_t& p45,
                                        uint32_t& p67) {
    const __half2 k1032 = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));
    const __half2 k16th = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));
    const __half2 km72 = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));
    uint32_t lo0 = (w & 0x000f000fu) | 0x64006400u;
    uint32_t hi0 = (w & 0x00f000f0u) | 0x64006400u;
    const uint32_t w8 = w >> 8;
    uint32_t lo1 = (w8 & 0x000f000fu) | 0x64006400u;
    uint32_t hi1 = (w8 & 0x00f000f0u) | 0x64006400u;
    __half2 a = __hsub2(*reinterpret_cast<__half2*>(&lo0), k1032);
    __half2 b = __hfma2(*reinterpret_cast<__half2*>(&hi0), k16th, km72);
    __half2 c = __hsub2(*reinterpret_cast<__half2*>(&lo1), k1032);
    __half2 d = __hfma2(*reinterpret_cast<__half2*>(&hi1), k16th, km72);
    p01 = *reinterpret_cast<uint32_t*>(&a);
    p23 = *reinterpret_cast<uint32_t*>(&b);
    p45 = *reinterpret_cast<uint32_t*>(&c);
    p67 = *reinterpret_cast<uint32_t*>(&d);
}

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(smem_u32(p)));
    return v;
}

// position (in halves) of feature f inside a fragment-ordered row: within each block of
// 128 features the sixteen 8-feature groups are stored transposed (group 4t+j at 4j+t), so
// that the four lanes of a quad read adjacent 16-byte pieces.
__device__ __host__ __forceinline__ int frag_pos(int f) {
    const int kb = f >> 7, kk = f & 127;
    const int t = kk >> 5, j = (kk >> 3) & 3, el = kk & 7;
    return (kb << 7) + (((j << 2) + t) << 3) + el;
}

template <bool GU>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_gemm_kernel(const DecodeKArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int nstage = a.nstage;
    const int Kmax = a.K > a.Ks ? a.K : a.Ks;
    const int xstride = Kmax * 2 + kXPad;  // bytes per activation row in shared memory
    uint8_t* ring = smem;
    uint8_t* xs = ring + (size_t)nstage * kStageBytes;
    float* red = reinterpret_cast<float*>(xs + (size_t)kDecodeTokens * xstride);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + 2 * kRedBytes);
    uint64_t* full = bars;                      // [kMaxStages]
    uint64_t* empty = bars + kMaxStages;        // [kMaxStages]
    uint64_t* red_full = bars + 2 * kMaxStages; // [2]
    uint64_t* red_free = red_full + 2;          // [2]
    uint64_t* xbar = red_free + 2;              // [1]
    volatile int* abort_flag = reinterpret_cast<volatile int*>(xbar + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < nstage; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kConsumerWarps); }
        for (int i = 0; i < 2; ++i) { mbar_init(&red_full[i], kConsumerWarps * 32); mbar_init(&red_free[i], kEpiWarps * 32); }
        mbar_init(xbar, kConsumerWarps * 32);
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    const int nseg = a.segs[0];
    const int nshared_seg = a.segs[1];
    const int64_t total = (int64_t)nshared_seg * a.units_s + (int64_t)(nseg - nshared_seg) * a.units;
    const int64_t it0 = total * blockIdx.x / gridDim.x;
    const int64_t it1 = total * (blockIdx.x + 1) / gridDim.x;

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t q = 0;
            for (int64_t it = it0; it < it1 && !*abort_flag; ++it) {
                const Item im = decode_item(a, it, nshared_seg);
                for (int c0 = 0; c0 < im.nchunk; c0 += kStageChunks, ++q) {
                    const uint32_t slot = q % nstage, ph = (q / nstage) & 1u;
                    if (!mbar_wait(&empty[slot], ph ^ 1u, kWaitLimit)) { record_timeout(a, abort_flag, 1); break; }
                    const int nc = min(kStageChunks, im.nchunk - c0);
                    const uint32_t bytes = (uint32_t)nc * kChunkBytes;
                    mbar_arrive_expect_tx(&full[slot], bytes);
                    bulk_g2s(ring + (size_t)slot * kStageBytes, im.chunks + (size_t)c0 * kChunkBytes, bytes, &full[slot]);
                }
            }
        }
    } else if (warp <= kConsumerWarps) {
        // ---------------- consumers ----------------
        const int cw = warp - 1;
        const int ck = cw >> 3, ks = (cw >> 1) & 3, m = cw & 1;
        const int g = lane >> 2, t = lane & 3;
        const int ctid = tid - 32;  // 0..511
        uint32_t q = 0, xuse = 0, item_local = 0;
        int cur_seg = -1;
        bool dead = false;
        for (int64_t it = it0; it < it1 && !dead; ++it, ++item_local) {
            const Item im = decode_item(a, it, nshared_seg);
            if (im.seg != cur_seg) {
                // every consumer is done with the previous segment's rows before they change
                mbar_arrive(xbar);
                if (!mbar_wait(xbar, xuse & 1u, kWaitLimit)) { record_timeout(a, abort_flag, 2); break; }
                ++xuse;
                const int vec_per_row = im.K >> 3;  // 16-byte pieces per row
                for (int idx = ctid; idx < im.ntok * vec_per_row; idx += kConsumerWarps * 32) {
                    const int j = idx / vec_per_row, v = idx - j * vec_per_row;
                    int64_t row;
                    if (GU) row = (im.slot_begin + j < a.P) ? a.sorted_tok[im.slot_begin + j] : (im.slot_begin + j - a.P);
                    else row = im.slot_begin + j;
                    const uint4 val = __ldg(reinterpret_cast<const uint4*>(a.bsrc + row * a.ldb) + v);
                    *reinterpret_cast<uint4*>(xs + (size_t)j * xstride + (size_t)v * 16) = val;
                }
                mbar_arrive(xbar);
                if (!mbar_wait(xbar, xuse & 1u, kWaitLimit)) { record_timeout(a, abort_flag, 3); break; }
                ++xuse;
                cur_seg = im.seg;
            }
            float tot[4] = {0.f, 0.f, 0.f, 0.f};
            for (int c0 = 0; c0 < im.nchunk; c0 += kStageChunks, ++q) {
                const uint32_t slot = q % nstage, ph = (q / nstage) & 1u;
                if (*abort_flag || !mbar_wait(&full[slot], ph, kWaitLimit)) {
                    if (!*abort_flag) record_timeout(a, abort_flag, 4);
                    dead = true;
                    break;
                }
                if (c0 + ck < im.nchunk) {
                    const uint8_t* chunk = ring + (size_t)slot * kStageBytes + (size_t)ck * kChunkBytes;
                    const uint8_t* blk = chunk + (ks * 2 + m) * 1024;
                    const uint4 w0 = lds128(blk + lane * 16);
                    const uint4 w1 = lds128(blk + 512 + lane * 16);
                    const __half* sc = reinterpret_cast<const __half*>(chunk + kChunkWeightBytes) + (ks * 2 + m) * 16;
                    const float s0 = __half2float(sc[g]), s1 = __half2float(sc[g + 8]);
                    const int kb = (c0 + ck) * 4 + ks;  // 128-column block index along K
                    const uint8_t* xrow = xs + (size_t)g * xstride + (size_t)kb * 256 + t * 16;
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w};
                    const uint32_t wb[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 xv = lds128(xrow + j * 64);
                        uint32_t a01, a23, a45, a67, b01, b23, b45, b67;
                        unpack8(wa[j], a01, a23, a45, a67);
                        unpack8(wb[j], b01, b23, b45, b67);
                        mma_16816(acc, a01, b01, a23, b23, xv.x, xv.y);
                        mma_16816(acc, a45, b45, a67, b67, xv.z, xv.w);
                    }
                    tot[0] = fmaf(s0, acc[0], tot[0]);
                    tot[1] = fmaf(s0, acc[1], tot[1]);
                    tot[2] = fmaf(s1, acc[2], tot[2]);
                    tot[3] = fmaf(s1, acc[3], tot[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }
            if (dead) break;
            const uint32_t rb = item_local & 1u;
            if (!mbar_wait(&red_free[rb], ((item_local >> 1) & 1u) ^ 1u, kWaitLimit)) { record_timeout(a, abort_flag, 5); break; }
            float* r = red + (size_t)rb * (kRedBytes / 4) + (size_t)cw * 128 + lane;
            r[0] = tot[0]; r[32] = tot[1]; r[64] = tot[2]; r[96] = tot[3];
            mbar_arrive(&red_full[rb]);
        }
    } else {
        // ---------------- epilogue ----------------
        const int et = tid - (1 + kConsumerWarps) * 32;  // 0..127
        const int r = et & 15, n = et >> 4;              // row in half unit, token
        const int L = ((r & 7) << 2) + (n >> 1);
        const int c = ((r >> 3) << 1) + (n & 1);
        uint32_t item_local = 0;
        for (int64_t it = it0; it < it1; ++it, ++item_local) {
            const Item im = decode_item(a, it, nshared_seg);
            const uint32_t rb = item_local & 1u;
            if (*abort_flag || !mbar_wait(&red_full[rb], (item_local >> 1) & 1u, kWaitLimit)) {
                if (!*abort_flag) record_timeout(a, abort_flag, 6);
                break;
            }
            const float* rbuf = red + (size_t)rb * (kRedBytes / 4) + c * 32 + L;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int j = 0; j < kConsumerWarps / 2; ++j) {
                s0 += rbuf[(size_t)(2 * j) * 128];
                s1 += rbuf[(size_t)(2 * j + 1) * 128];
            }
            if (n < im.ntok) {
                const int64_t slot = im.slot_begin + n;
                if (GU) {
                    const float h = __fmul_rn(silu_ref(s0), s1);
                    a.hbuf[slot * a.ldh + frag_pos(im.unit * 16 + r)] = __float2half_rn(h);
                } else {
                    float* y = a.ybuf + slot * a.H + im.unit * 32 + r;
                    y[0] = s0;
                    y[16] = s1;
                }
            }
            mbar_arrive(&red_free[rb]);
        }
    }
}

// ---- segment list ---------------------------------------------------------------------
// segs[0] = number of segments, segs[1] = number of shared-expert segments (these come
// first), then int4 {expert, first slot, tokens (<= 8), 0} per segment.  Built on the device
// from the dispatch offsets - no host synchronisation.
__global__ void __launch_bounds__(1024)
seg_build_kernel(const int* __restrict__ expert_offsets, int E, int n, int P, int has_shared,
                 int* __restrict__ segs) {
    __shared__ int wsum[32];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    const int nsh = has_shared ? (n + kDecodeTokens - 1) / kDecodeTokens : 0;
    int cnt = 0, beg = 0;
    if (tid < E) { beg = expert_offsets[tid]; cnt = expert_offsets[tid + 1] - beg; }
    const int ng = (cnt + kDecodeTokens - 1) / kDecodeTokens;
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
        if (lane == 31) { segs[0] = nsh + si; segs[1] = nsh; segs[2] = 0; segs[3] = 0; }
    }
    __syncthreads();
    const int base = nsh + incl - ng + wsum[w];
    int4* out = reinterpret_cast<int4*>(segs + kSegHeader);
    for (int j = 0; j < ng; ++j)
        out[base + j] = make_int4(tid, beg + j * kDecodeTokens, min(kDecodeTokens, cnt - j * kDecodeTokens), 0);
    for (int j = tid; j < nsh; j += blockDim.x)
        out[j] = make_int4(E, P + j * kDecodeTokens, min(kDecodeTokens, n - j * kDecodeTokens), 0);
}

// bf16 activations -> fp16 in fragment order (exact for |x| in the fp16 normal range; values
// beyond +-65504 saturate to the largest finite fp16).
__global__ void __launch_bounds__(256)
xprep_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ xp, int64_t n, int H) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 8-feature group each
    const int gpr = H >> 3;
    if (i >= n * gpr) return;
    const int64_t row = i / gpr;
    const int grp = (int)(i - row * gpr);
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + row * H) + grp);
    const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&v);
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float2 f = __bfloat1622float2(bp[q]);
        f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
        f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
        const __half2 h = __floats2half2_rn(f.x, f.y);
        op[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(xp + row * H + frag_pos(grp << 3)) = o;
}

// Deterministic weighted combine (replaces the in-kernel slot sum of
// cuda/moe_expert.cu:201-221 and moe_down_reduce_kernel, cuda/qgemm.cu:943-954):
// out[t] = ((0 + w0*y0) + w1*y1 ...) + y_shared, product and sum rounded separately like the
// CPU reference (src/model_glm52.cpp:1141, :1151).
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ ybuf, const int* __restrict__ slot_pos,
               const float* __restrict__ topk_w, int n, int topk, int H, int P, int has_shared,
               float* __restrict__ out) {
    const int t = blockIdx.y;
    const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c4 >= (H >> 2)) return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < topk; ++k) {
        const int pos = slot_pos[t * topk + k];
        const float w = topk_w[t * topk + k];
        const float4 y = __ldg(reinterpret_cast<const float4*>(ybuf + (int64_t)pos * H) + c4);
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, y.x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(w, y.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, y.z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(w, y.w));
    }
    if (has_shared) {
        const float4 y = __ldg(reinterpret_cast<const float4*>(ybuf + (int64_t)(P + t) * H) + c4);
        acc.x = __fadd_rn(acc.x, y.x);
        acc.y = __fadd_rn(acc.y, y.y);
        acc.z = __fadd_rn(acc.z, y.z);
        acc.w = __fadd_rn(acc.w, y.w);
    }
    reinterpret_cast<float4*>(out + (int64_t)t * H)[c4] = acc;
}

size_t decode_smem_bytes(int Kmax, int nstage) {
    return (size_t)nstage * kStageBytes + (size_t)kDecodeTokens * (Kmax * 2 + kXPad) + 2 * kRedBytes +
           (2 * kMaxStages + 5) * sizeof(uint64_t) + 16;
}

int pick_stages(int Kmax) {
    const size_t limit = 227 * 1024;
    int ns = kMaxStages;
    while (ns >= 3 && decode_smem_bytes(Kmax, ns) > limit) --ns;
    return ns >= 3 ? ns : 0;
}

}  // namespace

size_t decode_seg_bytes(int n, int topk, int E) {
    const size_t P = (size_t)n * topk;
    const size_t max_segs = (size_t)E + (P + kDecodeTokens - 1) / kDecodeTokens +
                            ((size_t)n + kDecodeTokens - 1) / kDecodeTokens + 1;
    return (kSegHeader + 4 * max_segs) * sizeof(int);
}

int launch_decode_layer(const DecodeArgs& d, cudaStream_t s) {
    const int P = d.n * d.topk;
    const bool shared = d.Is > 0;
    const int imax = d.I > d.Is ? d.I : d.Is;
    if (d.E > 1024) return GSB_ERR_UNSUPPORTED;
    if (cudaMemsetAsync(d.status, 0, 16, s) != cudaSuccess) return GSB_ERR_CUDA;

    xprep_kernel<<<(unsigned)(((int64_t)d.n * (d.H >> 3) + 255) / 256), 256, 0, s>>>(d.x, d.xp, d.n, d.H);
    seg_build_kernel<<<1, 1024, 0, s>>>(d.expert_offsets, d.E, d.n, P, shared ? 1 : 0, d.segs);
    if (d.ev_prep) cudaEventRecord(d.ev_prep, s);

    DecodeKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed);
    g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    g.segs = d.segs; g.sorted_tok = d.sorted_tok;
    g.bsrc = d.xp; g.ldb = d.H; g.K = d.H; g.Ks = d.H;
    g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.E; g.P = P;
    g.hbuf = d.hbuf; g.ldh = imax; g.ybuf = nullptr; g.H = d.H; g.status = d.status;
    g.nstage = pick_stages(d.H);
    if (!g.nstage) return GSB_ERR_UNSUPPORTED;
    size_t smem = decode_smem_bytes(d.H, g.nstage);
    if (cudaFuncSetAttribute(decode_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    decode_gemm_kernel<true><<<d.sm_count, kDecodeThreads, smem, s>>>(g);
    if (d.ev_gate_up) cudaEventRecord(d.ev_gate_up, s);

    DecodeKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed);
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.bsrc = d.hbuf; w.ldb = imax; w.K = d.I; w.Ks = shared ? d.Is : d.I;
    w.units = d.H / 32; w.units_s = d.H / 32;
    w.hbuf = nullptr; w.ybuf = d.ybuf;
    w.nstage = pick_stages(imax);
    if (!w.nstage) return GSB_ERR_UNSUPPORTED;
    smem = decode_smem_bytes(imax, w.nstage);
    if (cudaFuncSetAttribute(decode_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    decode_gemm_kernel<false><<<d.sm_count, kDecodeThreads, smem, s>>>(w);
    if (d.ev_down) cudaEventRecord(d.ev_down, s);

    dim3 cgrid((unsigned)(((d.H >> 2) + 255) / 256), (unsigned)d.n);
    combine_kernel<<<cgrid, 256, 0, s>>>(d.ybuf, d.slot_pos, d.topk_w, d.n, d.topk, d.H, P,
                                         shared ? 1 : 0, d.out);
    return launch_status();
}

}  // namespace gsb

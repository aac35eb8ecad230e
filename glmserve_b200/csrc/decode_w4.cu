// Decode-shaped W4A16 grouped GEMM: a bandwidth-bound split-K kernel over the tile stream.
//
// One persistent CTA per SM.  Work item = (segment, unit): a segment is up to 8 token rows
// of one expert (the shared expert is expert index E with every token), a unit is 32 weight
// rows over the full input dimension.  Roles inside the CTA:
//   warp 0           producer: one lane streams the item's chunks (16.5 KiB stages, one
//                    contiguous 1-D bulk copy each) into a shared-memory ring, completion
//                    on mbarriers, running ahead across item boundaries
//   warps 1..16      consumers: each owns one (128-column kstep, half unit) of every stage
//                    = split-K across warps.  A nibble n masked in place IS the fp16
//                    subnormal n * 2^-24 (n * 2^-20 for the odd nibble), so unpacking is one
//                    AND per fp16 pair; mma.sync m16n8k16 against the segment's fp16
//                    activations (in shared memory) gives sum x*n exactly in fp32, and once
//                    per 128 columns the zero point (-8 * sum x, from a per-segment table)
//                    and the fp16 group scale are applied to the accumulator
//   warps 17..20     epilogue: sums the 8 K-split partials of each half unit in fixed order,
//                    fuses SwiGLU (gate/up kernel) and stores fp16 h, or stores the fp32
//                    down-projection row of the slot (down kernel)
// Nothing is accumulated with atomics; every reduction order is fixed, so results do not
// depend on the grid or on timing.  Every wait is bounded: on a timeout the CTA records
// where in the status word and all its loops leave.

#include <cooperative_groups.h>

#include "common.cuh"
#include "launchers.cuh"
#include "route_device.cuh"

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
    float* const* ydst;            // optional per-slot output row pointers (expert parallel: a routed row lives on the
                                   // token's home GPU and is stored there over NVLink); overrides ybuf
    int H;
    int nstage;
    int* status;
    int pdl_trigger;               // 1: let the next launch start early (programmatic dependent launch)
    int pdl_wait;                  // 1: launched early: wait for the previous grid before reading its output
    int pdl_wait_all;              // 1: launched early and every warp needs the previous grid's output at once
    const int* xsegs;              // expert list of the register-resident variant (see xseg_* below)
    int x_which;                   // 0: gate/up item numbering, 1: down
};

struct Item {
    int seg, unit, expert, slot_begin, ntok, K;
    const uint8_t* chunks;  // first chunk of this (expert, unit)
    int nchunk;
};

// Walks the flat item list [shared segments x units_s | routed segments x units] without a
// division per item: (segment, unit) advance incrementally, the segment record is re-read
// only when the segment changes.
struct ItemIter {
    int seg, unit, U, nshared_seg;
    int4 rec;
    __device__ __forceinline__ void init(const DecodeKArgs& a, long long it, int nshared) {
        nshared_seg = nshared;
        const long long shared_items = (long long)nshared * a.units_s;
        if (it < shared_items) { U = a.units_s; seg = (int)(it / U); unit = (int)(it - (long long)seg * U); }
        else {
            const long long l = it - shared_items;
            U = a.units; const int sg = (int)(l / U); unit = (int)(l - (long long)sg * U); seg = sg + nshared;
        }
        rec = reinterpret_cast<const int4*>(a.segs + kSegHeader)[seg];
    }
    __device__ __forceinline__ void next(const DecodeKArgs& a) {
        if (++unit == U) {
            unit = 0;
            ++seg;
            if (seg == nshared_seg) U = a.units;
            rec = reinterpret_cast<const int4*>(a.segs + kSegHeader)[seg];  // one past the end is padding
        }
    }
    __device__ __forceinline__ Item get(const DecodeKArgs& a) const {
        Item r;
        const bool sh = seg < nshared_seg;
        r.seg = seg; r.unit = unit; r.expert = rec.x; r.slot_begin = rec.y; r.ntok = rec.z;
        r.K = sh ? a.Ks : a.K;
        r.nchunk = r.K / kChunkCols;
        const uint8_t* base = sh ? a.shared_packed : a.packed;
        const long long e_local = sh ? 0 : rec.x;
        r.chunks = base + ((e_local * U + unit) * (long long)r.nchunk) * kChunkBytes;
        return r;
    }
};

// A maximal run of consecutive items inside one segment: units [ubeg, uend) of segment seg.
// A CTA's item range splits into a handful of runs, so the per-item work of the inner loops
// is a counter increment (the units of a segment are contiguous in the tile stream).
struct SegRun {
    int seg, ubeg, uend, expert, slot_begin, ntok;
    const uint8_t* chunks;  // first chunk of unit ubeg
};
// ---- expert list (register-resident variant) ----------------------------------------------
// One entry per expert that has tokens (the shared expert first, then the routed experts in order):
//   xsegs[0] = entries, [1] / [2] = total items of the gate/up / down kernel, [3] = grid size,
//   entries from [kXHeader]: {expert, first slot, tokens, groups of 8 tokens, first gate/up item,
//   first down item, 0, 0}, then cta_start[2][grid + 1]: the entry each CTA's first item falls in.
// An expert with G > 1 token groups enumerates its items group by group (all units of group 0,
// then of group 1, ...).  Interleaving the groups over small blocks of units, so that a block's
// weights come from L2 for every group after the first, measured slower: each switch of group
// reloads the group's activation fragments (as many bytes as one unit of weights) and drains
// the pipeline.
constexpr int kXHeader = 4;
constexpr int kXEntry = 8;

template <bool GU>
__device__ __forceinline__ bool next_run_x(const DecodeKArgs& a, long long& it, long long it1, int& cur,
                                           int nchunk, SegRun& r) {
    if (it >= it1) return false;
    const int* ent = a.xsegs + kXHeader + cur * kXEntry;
    int U, G;
    long long ib;
    for (;;) {
        U = ent[0] >= a.E ? a.units_s : a.units;
        G = ent[3];
        ib = ent[GU ? 4 : 5];
        if (it < ib + (long long)U * G) break;
        ++cur;
        ent += kXEntry;
    }
    const int l = (int)(it - ib);
    const long long left = it1 - it;
    const int g = G == 1 ? 0 : l / U;
    const int unit = l - g * U;
    const int uend = (long long)(U - unit) < left ? U : unit + (int)left;
    r.seg = cur * 4096 + g;
    r.ubeg = unit; r.uend = uend;
    r.expert = ent[0];
    r.slot_begin = ent[1] + g * kDecodeTokens;
    r.ntok = min(kDecodeTokens, ent[2] - g * kDecodeTokens);
    const bool sh = ent[0] >= a.E;
    const uint8_t* base = sh ? a.shared_packed : a.packed;
    const long long e_local = sh ? 0 : ent[0];
    r.chunks = base + ((e_local * U + unit) * (long long)nchunk) * kChunkBytes;
    it += uend - unit;
    return true;
}

__device__ __forceinline__ void record_timeout(const DecodeKArgs& a, volatile int* abort_flag,
                                               int where) {
    *abort_flag = 1;
    if (atomicCAS(a.status + kStatusCode, 0, GSB_ERR_TIMEOUT) == 0) {
        a.status[kStatusWhere] = where;
        a.status[kStatusAux] = (int)blockIdx.x;
    }
}

// Eight int4 of one word (tile-stream nibble order) as fp16 SUBNORMAL bit patterns: a nibble n
// left in bits 0..3 of a half is n * 2^-24, in bits 4..7 it is n * 2^-20.  lo* hold columns
// (k0,k1) / (k4,k5), hi* hold (k2,k3) / (k6,k7).
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t& lo0, uint32_t& hi0, uint32_t& lo1,
                                        uint32_t& hi1) {
    lo0 = w & 0x000f000fu;
    hi0 = w & 0x00f000f0u;
    const uint32_t w8 = w >> 8;
    lo1 = w8 & 0x000f000fu;
    hi1 = w8 & 0x00f000f0u;
}

// d = a * b (no accumulator input: the first product of a chain needs no zeroed registers)
__device__ __forceinline__ void mma_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                                uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
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

template <bool GU>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_gemm_kernel(const DecodeKArgs a) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const int nstage = a.nstage;
    const int Kmax = a.K > a.Ks ? a.K : a.Ks;
    const int xstride = Kmax * 2 + kXPad;  // bytes per activation row in shared memory
    uint8_t* ring = smem;
    uint8_t* xs = ring + (size_t)nstage * kStageBytes;
    float* sx = reinterpret_cast<float*>(xs + (size_t)kDecodeTokens * xstride);  // [K/128][8] row sums
    float* red = sx + (size_t)(Kmax >> 7) * kDecodeTokens;
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
        for (int i = 0; i < 2; ++i) { mbar_init(&red_full[i], kConsumerWarps); mbar_init(&red_free[i], kEpiWarps); }
        mbar_init(xbar, kConsumerWarps * 32);
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    const int nseg = a.segs[0];
    const int nshared_seg = a.segs[1];
    const long long total = (long long)nshared_seg * a.units_s + (long long)(nseg - nshared_seg) * a.units;
    const long long it0 = total * blockIdx.x / gridDim.x;
    const long long it1 = total * (blockIdx.x + 1) / gridDim.x;
    if (it0 >= it1) return;
    ItemIter iter;
    iter.init(a, it0, nshared_seg);

    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            uint32_t q = 0;
            for (long long it = it0; it < it1 && !*abort_flag; ++it, iter.next(a)) {
                const Item im = iter.get(a);
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
        const uint32_t w_off = (uint32_t)ck * kChunkBytes + (ks * 2 + m) * 1024 + lane * 16;
        const uint32_t sc_off = (uint32_t)ck * kChunkBytes + kChunkWeightBytes + ((ks * 2 + m) * 16 + g) * 2;
        const uint8_t* xlane = xs + (size_t)g * xstride + t * 16;
        uint32_t q = 0, xuse = 0, item_local = 0;
        int cur_seg = -1;
        bool dead = false;
        for (long long it = it0; it < it1 && !dead; ++it, ++item_local, iter.next(a)) {
            const Item im = iter.get(a);
            if (im.seg != cur_seg) {
                // every consumer is done with the previous segment's rows before they change
                mbar_arrive(xbar);
                if (!mbar_wait(xbar, xuse & 1u, kWaitLimit)) { record_timeout(a, abort_flag, 2); break; }
                ++xuse;
                const int vec_per_row = im.K >> 3;  // 16-byte pieces per row
                for (int idx = ctid; idx < im.ntok * vec_per_row; idx += kConsumerWarps * 32) {
                    const int j = idx / vec_per_row, v = idx - j * vec_per_row;
                    long long row;
                    if (GU) row = (im.slot_begin + j < a.P) ? a.sorted_tok[im.slot_begin + j] : (im.slot_begin + j - a.P);
                    else row = im.slot_begin + j;
                    const uint4 val = __ldg(reinterpret_cast<const uint4*>(a.bsrc + row * a.ldb) + v);
                    *reinterpret_cast<uint4*>(xs + (size_t)j * xstride + (size_t)v * 16) = val;
                }
                mbar_arrive(xbar);
                if (!mbar_wait(xbar, xuse & 1u, kWaitLimit)) { record_timeout(a, abort_flag, 3); break; }
                ++xuse;
                // per (token, 128-column block) sums of the activations: the zero-point term
                const int nkb = im.K >> 7;
                for (int idx = ctid; idx < nkb * kDecodeTokens; idx += kConsumerWarps * 32) {
                    const int n = idx & (kDecodeTokens - 1), kb = idx >> 3;
                    float acc = 0.f;
                    if (n < im.ntok) {
                        const uint4* src = reinterpret_cast<const uint4*>(xs + (size_t)n * xstride + (size_t)kb * 256);
#pragma unroll 4
                        for (int v = 0; v < 16; ++v) {
                            const uint4 u = src[v];
                            const __half2* hp = reinterpret_cast<const __half2*>(&u);
#pragma unroll
                            for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(hp[e]); acc += f.x; acc += f.y; }
                        }
                    }
                    sx[idx] = acc;
                }
                mbar_arrive(xbar);
                if (!mbar_wait(xbar, xuse & 1u, kWaitLimit)) { record_timeout(a, abort_flag, 7); break; }
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
                    const uint8_t* stage = ring + (size_t)slot * kStageBytes;
                    const uint4 w0 = lds128(stage + w_off);
                    const uint4 w1 = lds128(stage + w_off + 512);
                    const __half* sc = reinterpret_cast<const __half*>(stage + sc_off);
                    const float s0 = __half2float(sc[0]), s1 = __half2float(sc[8]);
                    const int kb = (c0 + ck) * 4 + ks;  // 128-column block index along K
                    const float2 sxv = *reinterpret_cast<const float2*>(sx + kb * kDecodeTokens + 2 * t);
                    const uint8_t* xrow = xlane + (size_t)kb * 256;
                    float alo[4] = {0.f, 0.f, 0.f, 0.f}, ahi[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w};
                    const uint32_t wb[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint4 xv = lds128(xrow + j * 64);
                        uint32_t al0, ah0, al1, ah1, bl0, bh0, bl1, bh1;
                        unpack8(wa[j], al0, ah0, al1, ah1);
                        unpack8(wb[j], bl0, bh0, bl1, bh1);
                        // columns (k0,k1)+(k4,k5) carry weight n*2^-24, (k2,k3)+(k6,k7) carry n*2^-20
                        mma_16816(alo, al0, bl0, al1, bl1, xv.x, xv.z);
                        mma_16816(ahi, ah0, bh0, ah1, bh1, xv.y, xv.w);
                    }
                    // sum x*(n-8) = 2^24*alo + 2^20*ahi - 8*sum(x); then the group scale
                    const float s0a = s0 * 16777216.f, s0b = s0 * 1048576.f, s0c = s0 * -8.f;
                    const float s1a = s1 * 16777216.f, s1b = s1 * 1048576.f, s1c = s1 * -8.f;
                    tot[0] = fmaf(s0a, alo[0], fmaf(s0b, ahi[0], fmaf(s0c, sxv.x, tot[0])));
                    tot[1] = fmaf(s0a, alo[1], fmaf(s0b, ahi[1], fmaf(s0c, sxv.y, tot[1])));
                    tot[2] = fmaf(s1a, alo[2], fmaf(s1b, ahi[2], fmaf(s1c, sxv.x, tot[2])));
                    tot[3] = fmaf(s1a, alo[3], fmaf(s1b, ahi[3], fmaf(s1c, sxv.y, tot[3])));
                }
                fence_proxy_async();  // as in the register-resident kernel: this warp's reads before the refill
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }
            if (dead) break;
            const uint32_t rb = item_local & 1u;
            if (!mbar_wait(&red_free[rb], ((item_local >> 1) & 1u) ^ 1u, kWaitLimit)) { record_timeout(a, abort_flag, 5); break; }
            float* r = red + (size_t)rb * (kRedBytes / 4) + (size_t)cw * 128 + lane;
            r[0] = tot[0]; r[32] = tot[1]; r[64] = tot[2]; r[96] = tot[3];
            __syncwarp();  // orders every lane's partials before the one release-arrive below
            if (lane == 0) mbar_arrive(&red_full[rb]);
        }
    } else {
        // ---------------- epilogue ----------------
        const int et = tid - (1 + kConsumerWarps) * 32;  // 0..127
        const int r = et & 15, n = et >> 4;              // row in half unit, token
        const int L = ((r & 7) << 2) + (n >> 1);
        const int c = ((r >> 3) << 1) + (n & 1);
        uint32_t item_local = 0;
        for (long long it = it0; it < it1; ++it, ++item_local, iter.next(a)) {
            const Item im = iter.get(a);
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
                const long long slot = im.slot_begin + n;
                if (GU) {
                    const float h = __fmul_rn(silu_ref(s0), s1);
                    a.hbuf[slot * a.ldh + frag_pos(im.unit * 16 + r)] = sat_half(h);
                } else {
                    float* y = (a.ydst ? a.ydst[slot] : a.ybuf + slot * a.H) + im.unit * 32 + r;
                    y[0] = s0;
                    y[16] = s1;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&red_free[rb]);
        }
    }
}

// ---- register-resident variant ------------------------------------------------------------
// Same work split and arithmetic, for input dims that are multiples of 2048 (NKB = K / 2048
// <= 3): a stage is four chunks (33 KiB, one bulk copy), consumer warp (ck, ks) owns chunk ck
// and kstep ks of every stage and BOTH half units, and keeps the activation fragments it will
// ever need for the segment - NKB x 4 x 16 bytes per lane - and their per-group sums in
// registers.  No activation copy in shared memory (the whole 227 KiB minus the partial-sum
// buffers is ring: more bytes in flight per SM), no CTA-wide synchronisation when the
// segment changes, a quarter fewer instructions per byte.
constexpr int kRConsumerWarps = 16;
// epilogue warps / partial-sum buffers: the down kernel finishes an item per stage and has
// twice the outputs per item, so it gets three warps and three buffers; gate/up one and two
// Warp roles (warpgroup aligned so register budgets can be moved with setmaxnreg):
// warps 0..15 consumers, warp 16 producer, warps 17..19 epilogue.
template <bool GU> struct RCfg { static constexpr int kEpiWarps = 3; static constexpr int kRed = GU ? 2 : 3;
                                 static constexpr int kThreads = (16 + 1 + kEpiWarps) * 32; };
// setmaxnreg moves registers between the warps of ONE CTA: what the consumers gain must have been
// given up by the helper warps out of the CTA's launch allocation (640 threads x 96 registers); an
// increase beyond that waits for ever.  16 x 32 x (104 - 96) = 4096 <= 4 x 32 x (96 - 64) = 4096.
constexpr int kRLaunchRegs = 96;
constexpr int kRConsumerRegs = 104;
constexpr int kRHelperRegs = 64;
static_assert(16 * (kRConsumerRegs - kRLaunchRegs) <= 4 * (kRLaunchRegs - kRHelperRegs),
              "consumer warps would wait for registers the helper warps never release");
constexpr int kRStageChunks = 4;
constexpr int kRStageBytes = kRStageChunks * kChunkBytes;           // 33792
constexpr int kRRedFloats = kRConsumerWarps * 8 * 32;               // 16 KiB per buffer
constexpr int kRMaxStages = 6;

// Sums the sixteen consumer warps' partials of one item and writes the item's outputs (gate/up:
// silu(gate) * up as fp16 in fragment order; down: fp32 rows of the slot buffer).
// A warp's partials lie as [m][c][lane] (c = accumulator register, lane = 4*g + t: row
// g + 8*(c>>1) of the half unit, token 2t + (c&1)).  A thread takes V adjacent lanes (same g,
// tokens two apart), so a warp reads consecutive words of each consumer warp's block: no bank
// conflicts, sixteen vector loads per thread.
template <bool GU, int UPS>
__device__ __forceinline__ void reduce_item(const DecodeKArgs& a, const float* __restrict__ redbuf, int et,
                                         int unit0, int slot_begin, int ntok) {
    constexpr int V = GU ? 2 : 4;
    constexpr int WPU = kRConsumerWarps / UPS;           // consumer warps that split one unit's input dim
    if (et >= 64) return;
    const int q = et * V;                              // first float of the m-block(s)
    const int m = GU ? 0 : q >> 7;
    const int c = (q >> 5) & 3, L0 = q & 31;
    const int r = (L0 >> 2) + ((c >> 1) << 3);
    const int n0 = ((L0 & 3) << 1) + (c & 1);
#pragma unroll
    for (int us = 0; us < UPS; ++us) {                 // the units of a stage (one, unless the input dim is short)
        const float* rbuf = redbuf + us * WPU * 256 + q;
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[2] = {0.f, 0.f};
#pragma unroll
        for (int w = 0; w < WPU; ++w) {
            if (GU) {
                const float2 p0 = *reinterpret_cast<const float2*>(rbuf + w * 256);
                const float2 p1 = *reinterpret_cast<const float2*>(rbuf + w * 256 + 128);
                s0[0] += p0.x; s0[1] += p0.y; s1[0] += p1.x; s1[1] += p1.y;
            } else {
                const float4 p0 = *reinterpret_cast<const float4*>(rbuf + w * 256);
                s0[0] += p0.x; s0[1] += p0.y; s0[2] += p0.z; s0[3] += p0.w;
            }
        }
        const int unit = unit0 * UPS + us;
#pragma unroll
        for (int v = 0; v < V; ++v) {
            const int n = n0 + 2 * v;
            if (n >= ntok) continue;
            const long long slot = slot_begin + n;
            if (GU) a.hbuf[slot * a.ldh + frag_pos(unit * 16 + r)] = sat_half(__fmul_rn(silu_ref(s0[v]), s1[v & 1]));
            else (a.ydst ? a.ydst[slot] : a.ybuf + slot * a.H)[unit * 32 + m * 16 + r] = s0[v];
        }
    }
}

// UPS > 1 (NKB = 1 only): the input dim is 2048 / UPS, so a 33 KiB stage holds UPS complete units (they are
// contiguous in the tile stream); an "item" is then a stage = UPS units, consumer warp (ck, ks) works on
// unit ck / (4 / UPS) of the stage, and the K-split of a unit runs over 16 / UPS warps.  Without this a
// tensor-parallel shard's 512-column down projection would be one 8 KiB chunk per item: all hand-offs.
template <bool GU, int NKB, int UPS>
__global__ void __launch_bounds__(RCfg<GU>::kThreads, 1)
decode_reg_kernel(const DecodeKArgs a) {
    static_assert(UPS == 1 || NKB == 1, "several units per stage only when a unit fits one stage");
    constexpr int CPU = kRStageChunks / UPS;          // chunks of one unit inside a stage
    constexpr int kREpiWarps = RCfg<GU>::kEpiWarps;
    constexpr int kRed = RCfg<GU>::kRed;
    extern __shared__ __align__(1024) uint8_t smem[];
    const int nstage = a.nstage;
    uint8_t* ring = smem;
    float* red = reinterpret_cast<float*>(ring + (size_t)nstage * kRStageBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + kRed * kRRedFloats);
    uint64_t* full = bars;
    uint64_t* empty = bars + kRMaxStages;
    uint64_t* red_full = bars + 2 * kRMaxStages;
    uint64_t* red_free = red_full + 4;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(red_free + 4);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < nstage; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], kRConsumerWarps); }
        for (int i = 0; i < kRed; ++i) { mbar_init(&red_full[i], kRConsumerWarps); mbar_init(&red_free[i], kREpiWarps); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();

    // Programmatic dependent launch along routing -> gate/up -> down -> combine: a grid lets its
    // successor be scheduled as SMs free up, and the successor waits (griddepcontrol.wait = the
    // predecessor has completed and its writes are visible) before it touches the predecessor's
    // output.  Gate/up needs the work lists at once, so all of it waits; the down kernel's producer
    // warp streams weights under gate/up's tail and only its consumers wait (pdl_wait below).  Every
    // grid waits before it ends, so completion is transitive along the chain.
    if (a.pdl_wait_all) asm volatile("griddepcontrol.wait;" ::: "memory");   // the work lists come from the previous grid
    if (a.pdl_trigger) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const long long total = a.xsegs[1 + a.x_which];
    const long long it0 = total * blockIdx.x / gridDim.x;
    const long long it1 = total * (blockIdx.x + 1) / gridDim.x;
    if (it0 >= it1) return;
    long long it = it0;
    int cur = a.xsegs[kXHeader + a.xsegs[0] * kXEntry + a.x_which * ((int)gridDim.x + 1) + blockIdx.x];
    SegRun run;

    if (warp < kRConsumerWarps) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRConsumerRegs));
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRHelperRegs));

    if (warp == kRConsumerWarps) {
        if (lane == 0) {  // register-resident variant: producer
            uint32_t slot = 0, ph = 0;   // ring position and the parity of its current use
            bool dead = false;
            while (!dead && !*abort_flag && next_run_x<GU>(a, it, it1, cur, NKB * 4, run)) {
                const uint8_t* src = run.chunks;
                const int nst = (run.uend - run.ubeg) * NKB;  // the run's units are contiguous in memory
                for (int i = 0; i < nst; ++i, src += kRStageBytes) {
                    if (!mbar_wait(&empty[slot], ph ^ 1u, kWaitLimit)) { record_timeout(a, abort_flag, 11); dead = true; break; }
                    mbar_arrive_expect_tx(&full[slot], kRStageBytes);
                    bulk_g2s(ring + (size_t)slot * kRStageBytes, src, kRStageBytes, &full[slot]);
                    if (++slot == (uint32_t)nstage) { slot = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp < kRConsumerWarps) {
        const int cw = warp;
        const int ck = cw >> 2, ks = cw & 3;
        const int g = lane >> 2, t = lane & 3;
        const uint32_t w_off = (uint32_t)ck * kChunkBytes + (ks * 2) * 1024 + lane * 16;
        const uint32_t sc_off = (uint32_t)ck * kChunkBytes + kChunkWeightBytes + ((ks * 2) * 16 + g) * 2;
        float* red_lane = red + (size_t)cw * 256 + lane;
        uint4 xf[NKB][4];
        float2 sxv[NKB];
        uint32_t slot = 0, ph = 0;   // ring position and parity, stepped instead of divided out
        uint32_t rb = 0, rph = 0;    // partial-sum buffer and the parity of its current use
        bool dead = false;
        int cur_key = -1;
        if (a.pdl_wait) asm volatile("griddepcontrol.wait;" ::: "memory");   // the activations come from the previous grid
        while (!dead && next_run_x<GU>(a, it, it1, cur, NKB * 4, run)) {
            if (run.seg != cur_key) {   // this group's activation fragments and sums, into registers
                cur_key = run.seg;
                const bool valid = g < run.ntok;
                long long row = 0;
                if (valid) {
                    if (GU) row = (run.slot_begin + g < a.P) ? a.sorted_tok[run.slot_begin + g] : (run.slot_begin + g - a.P);
                    else row = run.slot_begin + g;
                }
                const uint4* src = reinterpret_cast<const uint4*>(a.bsrc + row * a.ldb);
#pragma unroll
                for (int st = 0; st < NKB; ++st) {
                    const int kb = (st * kRStageChunks + (UPS == 1 ? ck : ck % CPU)) * 4 + ks;
                    float sg = 0.f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        xf[st][j] = valid ? __ldg(src + kb * 16 + j * 4 + t) : make_uint4(0u, 0u, 0u, 0u);
                        const __half2* hp = reinterpret_cast<const __half2*>(&xf[st][j]);
#pragma unroll
                        for (int e = 0; e < 4; ++e) { const float2 f = __half22float2(hp[e]); sg += f.x; sg += f.y; }
                    }
                    sg += __shfl_xor_sync(0xffffffffu, sg, 1);
                    sg += __shfl_xor_sync(0xffffffffu, sg, 2);
                    sxv[st].x = -8.f * __shfl_sync(0xffffffffu, sg, (2 * t) * 4);      // the zero-point term
                    sxv[st].y = -8.f * __shfl_sync(0xffffffffu, sg, (2 * t + 1) * 4);
                }
            }
            for (int unit = run.ubeg; unit < run.uend && !dead; ++unit) {
                float tot[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                for (int st = 0; st < NKB; ++st) {
                    if (!mbar_wait(&full[slot], ph, kWaitLimit)) { record_timeout(a, abort_flag, 14); dead = true; break; }
                    __syncwarp();  // lanes leave the poll loop one by one; mma.sync wants them together
                    const uint8_t* stage = ring + (size_t)slot * kRStageBytes;
#pragma unroll
                    for (int m = 0; m < 2; ++m) {
                        const uint4 w0 = lds128(stage + w_off + m * 1024);
                        const uint4 w1 = lds128(stage + w_off + m * 1024 + 512);
                        const __half* sc = reinterpret_cast<const __half*>(stage + sc_off + m * 32);
                        const float s0 = __half2float(sc[0]), s1 = __half2float(sc[8]);
                        float alo[4], ahi[4];
                        const uint32_t wa[4] = {w0.x, w0.y, w0.z, w0.w};
                        const uint32_t wb[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint32_t al0, ah0, al1, ah1, bl0, bh0, bl1, bh1;
                            unpack8(wa[j], al0, ah0, al1, ah1);
                            unpack8(wb[j], bl0, bh0, bl1, bh1);
                            if (j == 0) {
                                mma_16816_first(alo, al0, bl0, al1, bl1, xf[st][j].x, xf[st][j].z);
                                mma_16816_first(ahi, ah0, bh0, ah1, bh1, xf[st][j].y, xf[st][j].w);
                            } else {
                                mma_16816(alo, al0, bl0, al1, bl1, xf[st][j].x, xf[st][j].z);
                                mma_16816(ahi, ah0, bh0, ah1, bh1, xf[st][j].y, xf[st][j].w);
                            }
                        }
                        // sum x*(n-8) = 2^24*(alo + ahi/16) - 8*sum(x), then the group scale;
                        // sxv holds -8*sum(x)
                        tot[m][0] = fmaf(s0, fmaf(fmaf(ahi[0], 0.0625f, alo[0]), 16777216.f, sxv[st].x), tot[m][0]);
                        tot[m][1] = fmaf(s0, fmaf(fmaf(ahi[1], 0.0625f, alo[1]), 16777216.f, sxv[st].y), tot[m][1]);
                        tot[m][2] = fmaf(s1, fmaf(fmaf(ahi[2], 0.0625f, alo[2]), 16777216.f, sxv[st].x), tot[m][2]);
                        tot[m][3] = fmaf(s1, fmaf(fmaf(ahi[3], 0.0625f, alo[3]), 16777216.f, sxv[st].y), tot[m][3]);
                    }
                    // The stage goes back to the producer, whose bulk copy writes it through the async
                    // proxy.  Loads of this warp that are still in flight (the scale words feed only
                    // `tot`, which nothing needs before the unit ends) are generic-proxy accesses: only
                    // a proxy fence before the release orders them ahead of that copy.  Without it a
                    // layer whose weights sit in L2 returned wrong sums in up to 40% of its forwards.
                    fence_proxy_async();  // generic-proxy reads of the stage before the async-proxy refill
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&empty[slot]);
                    if (++slot == (uint32_t)nstage) { slot = 0; ph ^= 1u; }
                }
                if (dead) break;
                if (!mbar_wait(&red_free[rb], rph ^ 1u, kWaitLimit)) { record_timeout(a, abort_flag, 15); dead = true; break; }
                float* r = red_lane + (size_t)rb * kRRedFloats;
#pragma unroll
                for (int m = 0; m < 2; ++m)
#pragma unroll
                    for (int c = 0; c < 4; ++c) r[m * 128 + c * 32] = tot[m][c];
                __syncwarp();  // orders every lane's partials before the one release-arrive below
                if (lane == 0) mbar_arrive(&red_full[rb]);
                if (++rb == (uint32_t)kRed) { rb = 0; rph ^= 1u; }
            }
        }
    } else {
        const int et = tid - (1 + kRConsumerWarps) * 32;
        uint32_t rb = 0, rph = 0;
        bool dead = false;
        while (!dead && next_run_x<GU>(a, it, it1, cur, NKB * 4, run)) {
            for (int unit = run.ubeg; unit < run.uend; ++unit) {
                if (*abort_flag || !mbar_wait(&red_full[rb], rph, kWaitLimit)) {
                    if (!*abort_flag) record_timeout(a, abort_flag, 16);
                    dead = true;
                    break;
                }
                reduce_item<GU, UPS>(a, red + (size_t)rb * kRRedFloats, et, unit, run.slot_begin, run.ntok);
                __syncwarp();
                if (lane == 0) mbar_arrive(&red_free[rb]);
                if (++rb == (uint32_t)kRed) { rb = 0; rph ^= 1u; }
            }
        }
    }
}

// ---- segment list ---------------------------------------------------------------------
// segs[0] = number of segments, segs[1] = number of shared-expert segments (these come
// first), then int4 {expert, first slot, tokens (<= 8), 0} per segment.  Built on the device
// from the dispatch offsets - no host synchronisation.
__device__ __forceinline__ void seg_build_block(const int* __restrict__ expert_offsets, int E, int n, int P,
                                                int has_shared, int* __restrict__ segs, int* __restrict__ xsegs,
                                                int units_gu, int units_gu_s, int units_dn, int grid) {
    __shared__ int wsum[32];
    __shared__ int pre_s[1025];   // exclusive prefix of token groups over routed experts
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
    for (int j = tid; j < nsh; j += 1024)
        out[j] = make_int4(E, P + j * kDecodeTokens, min(kDecodeTokens, n - j * kDecodeTokens), 0);
    if (!xsegs) return;
    // expert list of the register-resident variant: experts that received tokens only, so that
    // a CTA stepping from one expert to the next never walks over empty entries
    __shared__ int nz_w[32];
    const int gpre = incl - ng + wsum[w];             // groups of the routed experts before this one
    const int nz = ng > 0 ? 1 : 0;
    int nzi = nz;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, nzi, o);
        if (lane >= o) nzi += u;
    }
    if (lane == 31) nz_w[w] = nzi;
    __syncthreads();
    if (w == 0) {
        const int v = nz_w[lane];
        int vi = v;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, vi, o);
            if (lane >= o) vi += u;
        }
        nz_w[lane] = vi - v;
        if (lane == 31) pre_s[1024] = vi;             // experts with tokens
    }
    __syncthreads();
    const int nnz = pre_s[1024];
    const int ci = nzi - nz + nz_w[w];                // this expert's place among those with tokens
    __syncthreads();                                  // pre_s[1024] is read before it may be rewritten
    if (nz) pre_s[ci] = gpre;
    if (tid == E - 1) pre_s[nnz] = gpre + ng;
    __syncthreads();
    const int groups = pre_s[nnz];
    const int nent = has_shared + nnz;
    const long long sh_gu = (long long)nsh * units_gu_s, sh_dn = (long long)nsh * units_dn;
    if (nz) {
        int* e8 = xsegs + kXHeader + (has_shared + ci) * kXEntry;
        e8[0] = tid; e8[1] = beg; e8[2] = cnt; e8[3] = ng;
        e8[4] = (int)(sh_gu + (long long)gpre * units_gu);
        e8[5] = (int)(sh_dn + (long long)gpre * units_dn);
        e8[6] = e8[7] = 0;
    }
    if (tid == 0) {
        if (has_shared) {
            int* e8 = xsegs + kXHeader;
            e8[0] = E; e8[1] = P; e8[2] = n; e8[3] = nsh; e8[4] = 0; e8[5] = 0; e8[6] = e8[7] = 0;
        }
        xsegs[0] = nent;
        xsegs[1] = (int)(sh_gu + (long long)groups * units_gu);
        xsegs[2] = (int)(sh_dn + (long long)groups * units_dn);
        xsegs[3] = grid;
    }
    // entry in which each CTA's first item falls (largest entry whose first item <= target)
    int* cta = xsegs + kXHeader + nent * kXEntry;
    for (int job = tid; job < 2 * (grid + 1); job += 1024) {
        const int which = job / (grid + 1), c = job - which * (grid + 1);
        const long long U = which ? units_dn : units_gu, shi = which ? sh_dn : sh_gu;
        const long long total = shi + (long long)groups * U;
        const long long target = total * c / grid;
        int ent = 0;
        if (!(has_shared && target < shi) && nnz > 0) {
            int lo = 0, hi = nnz - 1;   // last listed routed expert with first item <= target
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (shi + (long long)pre_s[mid] * U <= target) lo = mid; else hi = mid - 1;
            }
            ent = has_shared + lo;
        }
        cta[job] = ent;
    }
}

__global__ void __launch_bounds__(1024)
seg_build_kernel(const int* __restrict__ expert_offsets, int E, int n, int P, int has_shared,
                 int* __restrict__ segs, int* __restrict__ xsegs, int units_gu, int units_gu_s, int units_dn,
                 int grid) {
    seg_build_block(expert_offsets, E, n, P, has_shared, segs, xsegs, units_gu, units_gu_s, units_dn, grid);
}

// Decode-sized batches (decode_route_fusable): top-k selection, dispatch and the work lists of
// both GEMM kernels in ONE launch - a cluster of 8 blocks for the top-k, its first block for the
// rest; three launches and their drain/fill gaps less per layer.  Each step is the stand-alone kernel's body, so ids, weights,
// permutation and lists are the same bits.
struct RouteFusedArgs {
    const float* scores; const float* e_bias;
    int n, E, topk, norm_topk; float routed_scale;
    int* ids; float* w;
    int* expert_offsets; int* sorted_tok; int* sorted_row; int* slot_pos;
    int has_shared; int* segs; int* xsegs; int units_gu, units_gu_s, units_dn, grid;
    int* status;
};

constexpr int kRouteCluster = 8;   // CTAs that share the top-k phase

// CL = 1: up to 32 tokens a single block has a warp per token and needs no cluster (and no cluster barrier).
template <int CL>
__device__ __forceinline__ void route_fused_body(const RouteFusedArgs& a, int rank) {
    extern __shared__ int route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    asm volatile("griddepcontrol.wait;" ::: "memory");                // launched under the logits kernel's tail
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");   // gate/up may be scheduled; it waits for this grid
    if (rank == 0 && threadIdx.x < 4) a.status[threadIdx.x] = 0;
    // top-k: a warp per token over the whole cluster (one block alone spends 15 us on 64 tokens)
    for (int t = rank + CL * warp; t < a.n; t += CL * 32)   // tokens dealt round-robin to the CTAs
        topk_token<8, true>(a.scores + (size_t)t * a.E, a.e_bias, a.E, a.topk, a.norm_topk, a.routed_scale, lane,
                            a.ids + (size_t)t * a.topk, a.w + (size_t)t * a.topk);
}
__device__ __forceinline__ void route_fused_tail(const RouteFusedArgs& a) {
    extern __shared__ int route_smem[];
    dispatch_block(a.ids, a.n * a.topk, a.topk, a.E, a.expert_offsets, a.sorted_tok, a.sorted_row, a.slot_pos, route_smem);
    __syncthreads();   // the block's own global writes (expert_offsets) are visible to it from here
    seg_build_block(a.expert_offsets, a.E, a.n, a.n * a.topk, a.has_shared, a.segs, a.xsegs, a.units_gu,
                    a.units_gu_s, a.units_dn, a.grid);
}

__global__ void __cluster_dims__(kRouteCluster, 1, 1) __launch_bounds__(1024)
route_fused_kernel(const RouteFusedArgs a) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    route_fused_body<kRouteCluster>(a, rank);
    cluster.sync();    // hardware barrier with release/acquire: every CTA's ids are visible to CTA 0
    if (rank != 0) return;
    route_fused_tail(a);
}

__global__ void __launch_bounds__(1024)
route_fused_small_kernel(const RouteFusedArgs a) {
    route_fused_body<1>(a, 0);
    __syncthreads();   // the block's own global writes (ids) are visible to it from here
    route_fused_tail(a);
}

// bf16 activations -> fp16 in fragment order or natural order (exact for |x| in the fp16 normal
// range; values beyond +-65504 saturate to the largest finite fp16).
__global__ void __launch_bounds__(256)
xprep_kernel(const __nv_bfloat16* __restrict__ x, __half* __restrict__ xp, int64_t n, int H, int natural) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 8-feature group each
    const int gpr = H >> 3;
    if (i >= n * gpr) return;
    const int64_t row = i / gpr;
    xprep_group(x, xp, row, (int)(i - row * gpr), H, natural);
}

// Deterministic weighted combine (replaces the in-kernel slot sum of
// cuda/moe_expert.cu:201-221 and moe_down_reduce_kernel, cuda/qgemm.cu:943-954):
// out[t] = ((0 + w0*y0) + w1*y1 ...) + y_shared, product and sum rounded separately like the
// CPU reference (src/model_glm52.cpp:1141, :1151).
__global__ void __launch_bounds__(256)
combine_kernel(const float* __restrict__ ybuf, const int* __restrict__ slot_pos,
               const float* __restrict__ topk_w, int n, int topk, int H, int P, int has_shared,
               const float* residual, float* out, int pdl_wait) {
    const int t = blockIdx.y;
    const int c4 = blockIdx.x * blockDim.x + threadIdx.x;
    if (c4 >= (H >> 2)) return;
    // Positions and weights come from the routing step, which completed before the down kernel could even
    // be scheduled, so they are read while that kernel still runs; only the rows need the wait below.
    int pos[8];
    float w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        pos[j] = j < topk ? slot_pos[t * topk + j] : 0;
        w[j] = j < topk ? topk_w[t * topk + j] : 0.f;
    }
    if (pdl_wait) asm volatile("griddepcontrol.wait;" ::: "memory");   // launched under the down kernel's tail
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 ys = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_shared) ys = __ldg(reinterpret_cast<const float4*>(ybuf + (int64_t)(P + t) * H) + c4);
    // eight slots' rows are asked for before the first is used: one slot at a time is a chain of
    // position -> row round trips (5.7 us for a single token); the sums keep their slot order
    for (int k0 = 0; k0 < topk; k0 += 8) {
        float4 y[8];
        if (k0) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                pos[j] = k0 + j < topk ? slot_pos[t * topk + k0 + j] : 0;
                w[j] = k0 + j < topk ? topk_w[t * topk + k0 + j] : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (k0 + j < topk) y[j] = __ldg(reinterpret_cast<const float4*>(ybuf + (int64_t)pos[j] * H) + c4);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (k0 + j < topk) {
                acc.x = __fadd_rn(acc.x, __fmul_rn(w[j], y[j].x));
                acc.y = __fadd_rn(acc.y, __fmul_rn(w[j], y[j].y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w[j], y[j].z));
                acc.w = __fadd_rn(acc.w, __fmul_rn(w[j], y[j].w));
            }
        }
    }
    if (has_shared) {
        const float4 y = ys;
        acc.x = __fadd_rn(acc.x, y.x);
        acc.y = __fadd_rn(acc.y, y.y);
        acc.z = __fadd_rn(acc.z, y.z);
        acc.w = __fadd_rn(acc.w, y.w);
    }
    if (residual) {   // hidden + mlp with the layer's sum complete before the add (src/model_gpu.cpp:1502);
                      // out may be the residual itself: each thread reads its element before it writes it
        const float4 r = reinterpret_cast<const float4*>(residual + (int64_t)t * H)[c4];
        acc = make_float4(__fadd_rn(r.x, acc.x), __fadd_rn(r.y, acc.y), __fadd_rn(r.z, acc.z), __fadd_rn(r.w, acc.w));
    }
    reinterpret_cast<float4*>(out + (int64_t)t * H)[c4] = acc;
}

size_t decode_smem_bytes(int Kmax, int nstage) {
    return (size_t)nstage * kStageBytes + (size_t)kDecodeTokens * (Kmax * 2 + kXPad) +
           (size_t)(Kmax >> 7) * kDecodeTokens * sizeof(float) + 2 * kRedBytes +
           (2 * kMaxStages + 5) * sizeof(uint64_t) + 16;
}

int pick_stages(int Kmax) {
    const size_t limit = 227 * 1024;
    int ns = kMaxStages;
    while (ns >= 3 && decode_smem_bytes(Kmax, ns) > limit) --ns;
    return ns >= 3 ? ns : 0;
}

}  // namespace

// fp32 activations (the reference's operator surface) -> fp16 rows, saturating, in either order
__global__ void __launch_bounds__(256)
xprep_f32_kernel(const float* __restrict__ x, __half* __restrict__ xp, int64_t n, int H, int natural) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 8-feature group each
    const int gpr = H >> 3;
    if (i >= n * gpr) return;
    const int64_t row = i / gpr;
    const int grp = (int)(i - row * gpr);
    const float4* src = reinterpret_cast<const float4*>(x + row * H) + 2 * grp;
    const float4 a = __ldg(src), b = __ldg(src + 1);
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const __half2 h = __halves2half2(sat_half(v[2 * q]), sat_half(v[2 * q + 1]));
        op[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(xp + row * H + (natural ? (grp << 3) : frag_pos(grp << 3))) = o;
}

int launch_xprep_f32(const float* x, __half* xp, int64_t n, int H, int natural, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    if (H % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return GSB_ERR_UNSUPPORTED;
    xprep_f32_kernel<<<(unsigned)((n * (H >> 3) + 255) / 256), 256, 0, s>>>(x, xp, n, H, natural);
    return launch_status();
}

int launch_xprep(const __nv_bfloat16* x, __half* xp, int64_t n, int H, int natural, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    xprep_kernel<<<(unsigned)((n * (H >> 3) + 255) / 256), 256, 0, s>>>(x, xp, n, H, natural);
    return launch_status();
}

// slots = routed rows the lists may have to cover, n_shared = rows of the shared expert, E = routed experts
static size_t seg_max(size_t slots, size_t n_shared, int E) {
    return (size_t)E + (slots + kDecodeTokens - 1) / kDecodeTokens + (n_shared + kDecodeTokens - 1) / kDecodeTokens + 1;
}
static size_t xsegs_offset_raw(size_t slots, size_t n_shared, int E) {
    return (kSegHeader + 4 * (seg_max(slots, n_shared, E) + 1) + 3) / 4 * 4;
}
size_t decode_seg_bytes_raw(size_t slots, size_t n_shared, int E) {
    const size_t x_ints = kXHeader + ((size_t)E + 1) * kXEntry + 2 * (1024 + 1);
    return (xsegs_offset_raw(slots, n_shared, E) + x_ints) * sizeof(int);
}
size_t decode_seg_bytes(int n, int topk, int E) { return decode_seg_bytes_raw((size_t)n * topk, (size_t)n, E); }
static size_t xsegs_offset_ints(int n, int topk, int E) { return xsegs_offset_raw((size_t)n * topk, (size_t)n, E); }

constexpr size_t decode_reg_smem(int nstage, int nred) {
    return (size_t)nstage * kRStageBytes + (size_t)nred * kRRedFloats * sizeof(float) + (2 * kRMaxStages + 8) * sizeof(uint64_t) + 16;
}

// nkb: 2048-column stages per unit (1..3), or 0 with ups = 2 / 4: units of 1024 / 512 columns, ups per stage
template <bool GU>
static int launch_reg(const DecodeKArgs& k, int nkb, int grid, cudaStream_t s, int ups = 1) {
    DecodeKArgs a = k;
    a.nstage = 5;
    const size_t smem = decode_reg_smem(a.nstage, RCfg<GU>::kRed);
#define GSB_LAUNCH_REG(N, U)                                                                           \
    {                                                                                                  \
        if (cudaFuncSetAttribute(decode_reg_kernel<GU, N, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                 (int)smem) != cudaSuccess)                                            \
            return GSB_ERR_CUDA;                                                                       \
        if (a.pdl_wait || a.pdl_wait_all) {                                                            \
            cudaLaunchConfig_t cfg = {};                                                               \
            cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(RCfg<GU>::kThreads);               \
            cfg.dynamicSmemBytes = smem; cfg.stream = s;                                               \
            cudaLaunchAttribute at[1];                                                                 \
            at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;                             \
            at[0].val.programmaticStreamSerializationAllowed = 1;                                      \
            cfg.attrs = at; cfg.numAttrs = 1;                                                          \
            if (cudaLaunchKernelEx(&cfg, decode_reg_kernel<GU, N, U>, a) != cudaSuccess) return GSB_ERR_LAUNCH; \
        } else {                                                                                       \
            decode_reg_kernel<GU, N, U><<<grid, RCfg<GU>::kThreads, smem, s>>>(a);                     \
        }                                                                                              \
        return GSB_OK;                                                                                 \
    }
    if (ups == 1) {
        if (nkb == 1) GSB_LAUNCH_REG(1, 1)
        if (nkb == 2) GSB_LAUNCH_REG(2, 1)
        if (nkb == 3) GSB_LAUNCH_REG(3, 1)
        return GSB_ERR_UNSUPPORTED;
    }
    if constexpr (!GU) {   // short input dims occur for the down projection of tensor-parallel shards
        if (ups == 2) GSB_LAUNCH_REG(1, 2)
        if (ups == 4) GSB_LAUNCH_REG(1, 4)
    }
    return GSB_ERR_UNSUPPORTED;
#undef GSB_LAUNCH_REG
}

// Register-resident form of the down kernel for this input dim: 0 = none, else units per stage.
static int down_reg_ups(int K) {
    if (K % 2048 == 0 && K / 2048 <= 3) return 1;
    if (K == 1024) return 2;
    if (K == 512) return 4;
    return 0;
}

int launch_decode_layer(const DecodeArgs& d, cudaStream_t s) {
    const int P = d.n * d.topk;
    const bool shared = d.Is > 0;
    // input dims of the down projections as packed (zero-weight columns beyond I / Is, see DecodeArgs)
    const int Id = d.Id > 0 ? d.Id : d.I, Isd = shared ? (d.Isd > 0 ? d.Isd : d.Is) : Id;
    const int imax = Id > Isd ? Id : Isd;
    const int ups = (!d.force_smem_variant && Isd == Id) ? down_reg_ups(Id) : 0;   // register-resident down kernel?
    const int units_dn = ups ? (d.H / 32) / ups : d.H / 32;                         // its items per expert
    if (d.E > 1024) return GSB_ERR_UNSUPPORTED;
    if (d.sm_count > 1024) return GSB_ERR_UNSUPPORTED;
    if (!d.xp_ready) {
        const int st0 = launch_xprep(d.x, d.xp, d.n, d.H, 0, s);
        if (st0) return st0;
    }
    int* xsegs = d.segs + xsegs_offset_ints(d.n, d.topk, d.E);
    if (d.fused_route) {
        if (!decode_route_fusable(d.n, d.topk, d.E)) return GSB_ERR_INVALID_ARG;
        RouteFusedArgs r{};
        r.scores = d.scores; r.e_bias = d.e_bias; r.n = d.n; r.E = d.E; r.topk = d.topk;
        r.norm_topk = d.norm_topk; r.routed_scale = d.routed_scale; r.ids = d.ids; r.w = d.w_out;
        r.expert_offsets = const_cast<int*>(d.expert_offsets); r.sorted_tok = const_cast<int*>(d.sorted_tok);
        r.sorted_row = d.sorted_row; r.slot_pos = const_cast<int*>(d.slot_pos);
        r.has_shared = shared ? 1 : 0; r.segs = d.segs; r.xsegs = xsegs;
        r.units_gu = d.I / 16; r.units_gu_s = shared ? d.Is / 16 : 1; r.units_dn = units_dn; r.grid = d.sm_count;
        r.status = d.status;
        const size_t smem = (size_t)(kDispWarps * d.E + 1024) * sizeof(int);   // 36 KiB at 256 experts
        cudaLaunchConfig_t cfg = {};
        const bool small = d.n <= 32;
        cfg.gridDim = dim3(small ? 1 : kRouteCluster); cfg.blockDim = dim3(1024); cfg.dynamicSmemBytes = smem; cfg.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // the logits kernel triggers at its start
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        if ((small ? cudaLaunchKernelEx(&cfg, route_fused_small_kernel, r) : cudaLaunchKernelEx(&cfg, route_fused_kernel, r)) != cudaSuccess)
            return GSB_ERR_LAUNCH;
    } else {
        if (cudaMemsetAsync(d.status, 0, 16, s) != cudaSuccess) return GSB_ERR_CUDA;
        seg_build_kernel<<<1, 1024, 0, s>>>(d.expert_offsets, d.E, d.n, P, shared ? 1 : 0, d.segs, xsegs, d.I / 16,
                                            shared ? d.Is / 16 : 1, units_dn, d.sm_count);
    }
    if (d.ev_prep) cudaEventRecord(d.ev_prep, s);

    DecodeKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed);
    g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    g.segs = d.segs; g.sorted_tok = d.sorted_tok;
    g.bsrc = d.xp; g.ldb = d.H; g.K = d.H; g.Ks = d.H;
    g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.E; g.P = P;
    g.hbuf = d.hbuf; g.ldh = imax; g.ybuf = nullptr; g.H = d.H; g.status = d.status;
    g.xsegs = xsegs; g.x_which = 0;
    // register-resident variant when the input dim is a multiple of 2048 (at most 3 x 2048)
    const bool gu_reg = !d.force_smem_variant && d.H % 2048 == 0 && d.H / 2048 <= 3;
    const bool dn_reg_ok = ups != 0;
    const bool pdl = gu_reg && dn_reg_ok;   // both register-resident: the down kernel starts under gate/up's tail
    g.pdl_trigger = pdl ? 1 : 0;
    g.pdl_wait_all = (pdl && d.fused_route) ? 1 : 0;   // the fused routing kernel is the one that triggers
    if (gu_reg) {
        const int st = launch_reg<true>(g, d.H / 2048, d.sm_count, s);
        if (st) return st;
    } else {
        g.nstage = pick_stages(d.H);
        if (!g.nstage) return GSB_ERR_UNSUPPORTED;
        const size_t smem = decode_smem_bytes(d.H, g.nstage);
        if (cudaFuncSetAttribute(decode_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return GSB_ERR_CUDA;
        decode_gemm_kernel<true><<<d.sm_count, kDecodeThreads, smem, s>>>(g);
    }
    if (d.ev_gate_up) cudaEventRecord(d.ev_gate_up, s);

    DecodeKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed);
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.bsrc = d.hbuf; w.ldb = imax; w.K = Id; w.Ks = Isd;
    w.units = units_dn; w.units_s = units_dn;
    w.hbuf = nullptr; w.ybuf = d.ybuf; w.x_which = 1;
    w.pdl_trigger = pdl ? 1 : 0; w.pdl_wait = pdl ? 1 : 0; w.pdl_wait_all = 0;
    const bool dn_reg = dn_reg_ok;
    if (dn_reg) {
        const int st = launch_reg<false>(w, ups == 1 ? Id / 2048 : 0, d.sm_count, s, ups);
        if (st) return st;
    } else {
        w.nstage = pick_stages(imax);
        if (!w.nstage) return GSB_ERR_UNSUPPORTED;
        const size_t smem = decode_smem_bytes(imax, w.nstage);
        if (cudaFuncSetAttribute(decode_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return GSB_ERR_CUDA;
        decode_gemm_kernel<false><<<d.sm_count, kDecodeThreads, smem, s>>>(w);
    }
    if (d.ev_down) cudaEventRecord(d.ev_down, s);

    dim3 cgrid((unsigned)(((d.H >> 2) + 255) / 256), (unsigned)d.n);
    if (pdl && dn_reg) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = cgrid; cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = 0; cfg.stream = s;
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, combine_kernel, (const float*)d.ybuf, (const int*)d.slot_pos,
                               (const float*)d.topk_w, d.n, d.topk, d.H, P, shared ? 1 : 0, (const float*)d.residual,
                               d.out, 1) != cudaSuccess)
            return GSB_ERR_LAUNCH;
    } else {
        combine_kernel<<<cgrid, 256, 0, s>>>(d.ybuf, d.slot_pos, d.topk_w, d.n, d.topk, d.H, P,
                                             shared ? 1 : 0, d.residual, d.out, 0);
    }
    return launch_status();
}

// Expert parallel on the split-K kernels: the rows this GPU received (already in expert order, fragment
// order, in xbuf rows [0, recv_cap)) through its resident experts, and its own n tokens (xbuf rows
// [recv_cap, recv_cap + n)) through the shared expert, as ONE pair of launches.  With P = 0 the gate/up
// kernel takes slot s from xbuf row s; the down kernel's epilogue stores every output row through ydst
// (received rows: a row of the token's home GPU over NVLink; shared rows: this GPU's own row buffer).
// `what`: 1 = the work lists only (they need the plan's receive offsets, not the rows: the caller builds them while
// the rows are still in flight), 2 = the two GEMM kernels only, 3 = both.
int launch_decode_ep(const DecodeEpArgs& d, cudaStream_t s, int what) {
    const bool shared = d.Is > 0;
    const int imax = d.I > d.Is ? d.I : d.Is;
    if (d.El > 1024 || d.sm_count > 1024) return GSB_ERR_UNSUPPORTED;
    const int ups = (!shared || d.Is == d.I) ? down_reg_ups(d.I) : 0;
    const int units_dn = ups ? (d.H / 32) / ups : d.H / 32;
    int* xsegs = d.segs + xsegs_offset_raw((size_t)d.recv_cap, (size_t)d.n, d.El);
    if (what & 1)
        seg_build_kernel<<<1, 1024, 0, s>>>(d.recv_offsets, d.El, d.n, d.recv_cap, shared ? 1 : 0, d.segs, xsegs, d.I / 16,
                                            shared ? d.Is / 16 : 1, units_dn, d.sm_count);
    if (!(what & 2)) return launch_status();
    DecodeKArgs g{};
    g.packed = reinterpret_cast<const uint8_t*>(d.gate_up_packed);
    g.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_gate_up_packed);
    g.segs = d.segs; g.sorted_tok = nullptr;
    g.bsrc = d.xbuf; g.ldb = d.H; g.K = d.H; g.Ks = d.H;
    g.units = d.I / 16; g.units_s = d.Is / 16; g.E = d.El; g.P = 0;
    g.hbuf = d.hbuf; g.ldh = imax; g.ybuf = nullptr; g.ydst = nullptr; g.H = d.H; g.status = d.status;
    g.xsegs = xsegs; g.x_which = 0;
    const bool gu_reg = d.H % 2048 == 0 && d.H / 2048 <= 3;
    // both register-resident: the down kernel is scheduled as gate/up's CTAs leave and streams its weights
    // under gate/up's tail (its consumers wait for gate/up's completion before they read h)
    const bool pdl = gu_reg && ups != 0;
    g.pdl_trigger = pdl ? 1 : 0;
    if (gu_reg) {
        const int st = launch_reg<true>(g, d.H / 2048, d.sm_count, s);
        if (st) return st;
    } else {
        g.nstage = pick_stages(d.H);
        if (!g.nstage) return GSB_ERR_UNSUPPORTED;
        const size_t smem = decode_smem_bytes(d.H, g.nstage);
        if (cudaFuncSetAttribute(decode_gemm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GSB_ERR_CUDA;
        decode_gemm_kernel<true><<<d.sm_count, kDecodeThreads, smem, s>>>(g);
    }
    DecodeKArgs w = g;
    w.packed = reinterpret_cast<const uint8_t*>(d.down_packed);
    w.shared_packed = reinterpret_cast<const uint8_t*>(d.shared_down_packed);
    w.bsrc = d.hbuf; w.ldb = imax; w.K = d.I; w.Ks = shared ? d.Is : d.I;
    w.units = units_dn; w.units_s = units_dn;
    w.hbuf = nullptr; w.ybuf = nullptr; w.ydst = d.ydst; w.x_which = 1;
    w.pdl_trigger = 0; w.pdl_wait = pdl ? 1 : 0; w.pdl_wait_all = 0;
    if (ups) {
        const int st = launch_reg<false>(w, ups == 1 ? d.I / 2048 : 0, d.sm_count, s, ups);
        if (st) return st;
    } else {
        w.nstage = pick_stages(imax);
        if (!w.nstage) return GSB_ERR_UNSUPPORTED;
        const size_t smem = decode_smem_bytes(imax, w.nstage);
        if (cudaFuncSetAttribute(decode_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GSB_ERR_CUDA;
        decode_gemm_kernel<false><<<d.sm_count, kDecodeThreads, smem, s>>>(w);
    }
    return launch_status();
}

// A dense W4A16 projection y[n, rows] = x[n, K] W^T on the split-K down kernel: W packed like one expert's
// down matrix, the n rows as one expert's tokens (xf: fp16 rows in fragment order), fp32 rows out.
// zero2: two zero ints (the dispatch offsets of a routed expert without tokens).
int launch_decode_dense(const void* packed, const __half* xf, int n, int K, int rows, float* y, int* segs,
                        const int* zero2, int* status, int sm_count, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    if (K % 512 || rows % 32 || sm_count > 1024) return GSB_ERR_UNSUPPORTED;
    const int ups = down_reg_ups(K);
    if (ups > 1 && (rows / 32) % ups) return GSB_ERR_UNSUPPORTED;
    const int units = ups ? (rows / 32) / ups : rows / 32;
    int* xsegs = segs + xsegs_offset_raw(0, (size_t)n, 1);
    if (cudaMemsetAsync(status, 0, 16, s) != cudaSuccess) return GSB_ERR_CUDA;
    seg_build_kernel<<<1, 1024, 0, s>>>(zero2, 1, n, 0, 1, segs, xsegs, 1, 1, units, sm_count);
    DecodeKArgs w{};
    w.packed = nullptr; w.shared_packed = reinterpret_cast<const uint8_t*>(packed);
    w.segs = segs; w.sorted_tok = nullptr; w.bsrc = xf; w.ldb = K; w.K = K; w.Ks = K;
    w.units = units; w.units_s = units; w.E = 1; w.P = 0;
    w.hbuf = nullptr; w.ybuf = y; w.ydst = nullptr; w.H = rows; w.status = status;
    w.xsegs = xsegs; w.x_which = 1;
    if (ups) return launch_reg<false>(w, ups == 1 ? K / 2048 : 0, sm_count, s, ups);
    w.nstage = pick_stages(K);
    if (!w.nstage) return GSB_ERR_UNSUPPORTED;
    const size_t smem = decode_smem_bytes(K, w.nstage);
    if (cudaFuncSetAttribute(decode_gemm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    decode_gemm_kernel<false><<<sm_count, kDecodeThreads, smem, s>>>(w);
    return launch_status();
}

int launch_combine_f32(const float* ybuf, const int* slot_pos, const float* topk_w, int n, int topk, int H, int P,
                       int has_shared, const float* residual, float* out, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    dim3 cgrid((unsigned)(((H >> 2) + 255) / 256), (unsigned)n);
    combine_kernel<<<cgrid, 256, 0, s>>>(ybuf, slot_pos, topk_w, n, topk, H, P, has_shared, residual, out, 0);
    return launch_status();
}

}  // namespace gsb

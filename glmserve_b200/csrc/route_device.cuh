// Device-side bodies of the routing steps, shared by their stand-alone kernels and by the
// single-block kernel that runs all of them for a decode-sized batch.
#pragma once

#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

// sigmoid evaluated so it reproduces the CPU reference's 1.0f / (1.0f + std::exp(-x)):
// exp in double then rounded once to float (what a correctly rounded expf returns), an
// IEEE add and an IEEE divide.  No fast-math intrinsics on purpose.
__device__ __forceinline__ float sigmoid_ref(float x) {
    const float e = static_cast<float>(exp(static_cast<double>(-x)));
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, e));
}

// One warp per token.  Lane l owns experts l, l+32, ...; NS = slots per lane.
// FROM_SCORES: the input already holds sigmoid scores (written by the logits kernel's
// epilogue with the same sigmoid_ref), so no transcendental is evaluated here.
template <int NS, bool FROM_SCORES>
__device__ __forceinline__ void topk_token(const float* __restrict__ lt, const float* __restrict__ e_bias, int E,
                                           int topk, int norm_topk, float routed_scale, int lane,
                                           int* __restrict__ ids_row, float* __restrict__ w_row) {
    float score[NS], key[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        const int e = lane + (j << 5);
        if (e < E) {
            const float sc = FROM_SCORES ? lt[e] : sigmoid_ref(lt[e]);
            score[j] = sc;
            key[j] = __fadd_rn(sc, e_bias ? e_bias[e] : 0.0f);
        } else {
            score[j] = 0.0f;
            key[j] = 0.0f;
        }
    }
    uint32_t taken = 0;  // bit j: slot j already selected
    float wsum = 0.0f;
    float myw = 0.0f;    // lane k keeps the weight and the id of selection k (topk <= 32)
    int myid = 0;
    for (int k = 0; k < topk; ++k) {
        // lane-local best among the slots still free: ascending j = ascending expert id,
        // strict > keeps the smaller id on equal keys.
        int be = 0x7fffffff;
        float bk = 0.0f, bs = 0.0f;
#pragma unroll
        for (int j = 0; j < NS; ++j) {
            const int e = lane + (j << 5);
            const bool ok = (e < E) && !((taken >> j) & 1u);
            if (ok && (be == 0x7fffffff || key[j] > bk)) { be = e; bk = key[j]; bs = score[j]; }
        }
        // warp winner: largest key, then smallest expert id among the lanes that hold it.  Keys
        // are compared as order-preserving integers (the float order for everything but NaN and
        // the sign of zero, neither of which sigmoid + bias produces), so two hardware warp
        // reductions replace fifteen shuffles per round.
        const uint32_t kb = __float_as_uint(bk);
        const uint32_t uk = be == 0x7fffffff ? 0u : ((kb & 0x80000000u) ? ~kb : (kb | 0x80000000u));
        const uint32_t mk = __reduce_max_sync(0xffffffffu, uk);
        const uint32_t me = __reduce_min_sync(0xffffffffu, (uk == mk && be != 0x7fffffff) ? (uint32_t)be : 0xffffffffu);
        const bool none = me == 0xffffffffu;
        be = none ? 0x7fffffff : (int)me;
        bs = __shfl_sync(0xffffffffu, bs, none ? 0 : (int)(me & 31u));   // the owning lane's best IS that expert
        if (none) bs = 0.0f;
        // every lane now holds the same winner
        if ((be & 31) == lane && be != 0x7fffffff) taken |= 1u << (be >> 5);
        if (lane == k) { myid = be == 0x7fffffff ? 0 : be; myw = bs; }
        wsum = __fadd_rn(wsum, bs);
    }
    if (lane < topk) {
        float v = myw;
        if (norm_topk && wsum > 0.0f) v = __fdiv_rn(v, wsum);
        w_row[lane] = __fmul_rn(v, routed_scale);
        ids_row[lane] = myid;
    }
}

constexpr int kDispWarps = 32;

// The dispatch in three phases, so that one block (decode-sized batches) or many blocks (prefill)
// can run it.  A block owns the contiguous slot range [b0, b1); its 32 warps own contiguous
// sub-ranges.  smem holds kDispWarps * E + 1024 ints: hist [kDispWarps][E], tot [E].

struct DispRange { int beg, end; };

__device__ __forceinline__ DispRange dispatch_warp_range(int b0, int b1) {
    int chunk = (b1 - b0 + kDispWarps - 1) / kDispWarps;
    chunk = (chunk + 31) & ~31;
    const int w = threadIdx.x >> 5;
    DispRange r;
    r.beg = min(b1, b0 + w * chunk);
    r.end = min(b1, r.beg + chunk);
    return r;
}

// Phase 1: per-warp histograms (no atomics: the lowest lane of each group of equal ids adds the
// group size), then per expert an exclusive scan over the block's warps.  On return
// hist[w][e] = slots of expert e owned by warps < w of this block, tot[e] = the block's count.
__device__ __forceinline__ void dispatch_hist(const int* __restrict__ topk_ids, int b0, int b1, int E, int* smem) {
    int* hist = smem;
    int* tot = smem + kDispWarps * E;
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    for (int i = tid; i < kDispWarps * E; i += (kDispWarps * 32)) hist[i] = 0;
    __syncthreads();
    const DispRange r = dispatch_warp_range(b0, b1);
    const uint32_t lt_mask = (1u << lane) - 1u;
    int* myhist = hist + w * E;
    for (int base = r.beg; base < r.end; base += 32) {
        const int i = base + lane;
        int id = (i < r.end) ? topk_ids[i] : -1;
        const bool valid = id >= 0 && id < E;
        const int key = valid ? id : (-1 - lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid && (peers & lt_mask) == 0) myhist[id] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    for (int e = tid; e < E; e += (kDispWarps * 32)) {
        int run = 0;
        for (int ww = 0; ww < kDispWarps; ++ww) {
            const int c = hist[ww * E + e];
            hist[ww * E + e] = run;
            run += c;
        }
        tot[e] = run;
    }
    __syncthreads();
}

// Exclusive scan of v over the block's first E threads (E <= 1024 = blockDim); every thread calls.
__device__ __forceinline__ int dispatch_block_scan(int v, int* total) {
    __shared__ int warp_sums[32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
    }
    if (lane == 31) warp_sums[w] = incl;
    __syncthreads();
    if (w == 0) {
        const int s = warp_sums[lane];
        int si = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, si, o);
            if (lane >= o) si += u;
        }
        warp_sums[lane] = si - s;
        if (lane == 31 && total) *total = si;
    }
    __syncthreads();
    const int excl = incl - v + warp_sums[w];
    __syncthreads();   // warp_sums may be reused by a later call
    return excl;
}

// Phase 3: hist[w][e] already holds the absolute start of (warp, expert); every warp walks its range
// again in the same order.  A slot's position is that start + the equal ids in lower lanes, and the
// group leader advances the start.  No position depends on an atomic or on timing.
__device__ __forceinline__ void dispatch_scatter(const int* __restrict__ topk_ids, int b0, int b1, int topk, int E,
                                                 int* __restrict__ sorted_token_ids, int* __restrict__ sorted_row,
                                                 int* __restrict__ slot_pos, int* smem) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const DispRange r = dispatch_warp_range(b0, b1);
    const uint32_t lt_mask = (1u << lane) - 1u;
    int* myhist = smem + w * E;
    for (int base = r.beg; base < r.end; base += 32) {
        const int i = base + lane;
        int id = (i < r.end) ? topk_ids[i] : -1;
        const bool valid = id >= 0 && id < E;
        const int key = valid ? id : (-1 - lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid) {
            const int dst = myhist[id] + __popc(peers & lt_mask);
            sorted_token_ids[dst] = i / topk;
            sorted_row[dst] = i - (i / topk) * topk;
            if (slot_pos) slot_pos[i] = dst;
        }
        __syncwarp();
        if (valid && (peers & lt_mask) == 0) myhist[id] += __popc(peers);
        __syncwarp();
    }
}

// The whole dispatch in one block.
__device__ __forceinline__ void dispatch_block(const int* __restrict__ topk_ids, int P, int topk, int E,
                                               int* __restrict__ expert_offsets, int* __restrict__ sorted_token_ids,
                                               int* __restrict__ sorted_row, int* __restrict__ slot_pos, int* smem) {
    int* hist = smem;
    int* tot = smem + kDispWarps * E;
    const int tid = threadIdx.x;
    dispatch_hist(topk_ids, 0, P, E, smem);
    const int v = tid < E ? tot[tid] : 0;
    const int excl = dispatch_block_scan(v, nullptr);
    if (tid < E) {
        tot[tid] = excl;
        expert_offsets[tid] = excl;
        if (tid == E - 1) expert_offsets[E] = excl + v;
    }
    __syncthreads();
    for (int i = tid; i < kDispWarps * E; i += (kDispWarps * 32)) hist[i] += tot[i % E];
    __syncthreads();
    dispatch_scatter(topk_ids, 0, P, topk, E, sorted_token_ids, sorted_row, slot_pos, smem);
}

}  // namespace gsb

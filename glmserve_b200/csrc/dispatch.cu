// Token permutation into per-expert contiguous segments.
//
// Same result as the reference's single-thread counting sort (cuda/moe_dispatch.cu:24-38):
// a STABLE sort of the flat slots i = t*topk + k by expert id.  Here 32 warps each own a
// contiguous range of i.  Pass 1: every warp builds its own histogram with __match_any_sync
// (the lowest lane of each group of equal ids adds the group size - addresses within a warp
// step are distinct, so no atomics).  A prefix scan over (expert, warp) turns the counts
// into start positions.  Pass 2: every warp walks its range again in the same order; a
// slot's position is start[warp][expert] + number of equal ids in lower lanes, and the
// group leader advances the start.  No position depends on an atomic or on timing.
#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

constexpr int kDispWarps = 32;

__global__ void __launch_bounds__(kDispWarps * 32)
dispatch_kernel(const int* __restrict__ topk_ids, int P, int topk, int E,
                int* __restrict__ expert_offsets, int* __restrict__ sorted_token_ids,
                int* __restrict__ sorted_row, int* __restrict__ slot_pos) {
    extern __shared__ int smem[];
    int* hist = smem;                        // [kDispWarps][E]
    int* tot = smem + kDispWarps * E;        // [E rounded to 1024]
    __shared__ int warp_sums[32];
    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
    for (int i = tid; i < kDispWarps * E; i += blockDim.x) hist[i] = 0;
    __syncthreads();

    int chunk = (P + kDispWarps - 1) / kDispWarps;
    chunk = (chunk + 31) & ~31;
    const int beg = min(P, w * chunk), end = min(P, beg + chunk);
    const uint32_t lt_mask = (1u << lane) - 1u;
    int* myhist = hist + w * E;

    for (int base = beg; base < end; base += 32) {
        const int i = base + lane;
        int id = (i < end) ? topk_ids[i] : -1;
        const bool valid = id >= 0 && id < E;
        const int key = valid ? id : (-1 - lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, key);
        if (valid && (peers & lt_mask) == 0) myhist[id] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();

    // per expert: exclusive scan over warps, total into tot[]
    for (int e = tid; e < E; e += blockDim.x) {
        int run = 0;
        for (int ww = 0; ww < kDispWarps; ++ww) {
            const int c = hist[ww * E + e];
            hist[ww * E + e] = run;
            run += c;
        }
        tot[e] = run;
    }
    __syncthreads();
    // exclusive scan of tot[0..E) (E <= 1024 = blockDim): warp scans + scan of warp sums
    {
        const int v = tid < E ? tot[tid] : 0;
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
        }
        __syncthreads();
        const int excl = incl - v + warp_sums[w];
        if (tid < E) {
            tot[tid] = excl;
            expert_offsets[tid] = excl;
            if (tid == E - 1) expert_offsets[E] = excl + v;
        }
    }
    __syncthreads();
    for (int i = tid; i < kDispWarps * E; i += blockDim.x) hist[i] += tot[i % E];
    __syncthreads();

    for (int base = beg; base < end; base += 32) {
        const int i = base + lane;
        int id = (i < end) ? topk_ids[i] : -1;
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

int launch_dispatch(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                    int* sorted_token_ids, int* sorted_row, int* slot_pos, cudaStream_t s) {
    if (E > 1024) return GSB_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(kDispWarps * E + 1024) * sizeof(int);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    dispatch_kernel<<<1, kDispWarps * 32, smem, s>>>(topk_ids, n * topk, topk, E, expert_offsets,
                                                     sorted_token_ids, sorted_row, slot_pos);
    return launch_status();
}

}  // namespace gsb

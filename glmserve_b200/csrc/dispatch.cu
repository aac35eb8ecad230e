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
#include "route_device.cuh"

namespace gsb {

__global__ void __launch_bounds__(kDispWarps * 32)
dispatch_kernel(const int* __restrict__ topk_ids, int P, int topk, int E,
                int* __restrict__ expert_offsets, int* __restrict__ sorted_token_ids,
                int* __restrict__ sorted_row, int* __restrict__ slot_pos) {
    extern __shared__ int smem[];
    dispatch_block(topk_ids, P, topk, E, expert_offsets, sorted_token_ids, sorted_row, slot_pos, smem);
}

// Many-block form for prefill-sized batches: block b owns kDispBlockSlots consecutive slots.
//   count:   per-block expert counts                       -> blk[b][e]
//   offsets: per expert an exclusive scan over the blocks, then over the experts
//            -> expert_offsets and blk[b][e] = absolute start of (block, expert)
//   scatter: every block rebuilds its warp histograms and places its slots
// Same permutation as the one-block form: positions are (expert, block, warp, lane) ordered, which
// is the order of the flat slot index.
constexpr int kDispBlockSlots = 4096;

__global__ void __launch_bounds__(kDispWarps * 32)
dispatch_count_kernel(const int* __restrict__ topk_ids, int P, int E, int* __restrict__ blk) {
    extern __shared__ int smem[];
    const int b0 = blockIdx.x * kDispBlockSlots, b1 = min(P, b0 + kDispBlockSlots);
    dispatch_hist(topk_ids, b0, b1, E, smem);
    const int* tot = smem + kDispWarps * E;
    for (int e = threadIdx.x; e < E; e += kDispWarps * 32) blk[(size_t)blockIdx.x * E + e] = tot[e];
}

__global__ void __launch_bounds__(kDispWarps * 32)
dispatch_offsets_kernel(int nblk, int E, int* __restrict__ blk, int* __restrict__ expert_offsets) {
    const int tid = threadIdx.x;
    int total = 0;
    if (tid < E)
        for (int b = 0; b < nblk; ++b) {
            const int c = blk[(size_t)b * E + tid];
            blk[(size_t)b * E + tid] = total;
            total += c;
        }
    const int excl = dispatch_block_scan(total, nullptr);
    if (tid < E) {
        expert_offsets[tid] = excl;
        if (tid == E - 1) expert_offsets[E] = excl + total;
        for (int b = 0; b < nblk; ++b) blk[(size_t)b * E + tid] += excl;
    }
}

__global__ void __launch_bounds__(kDispWarps * 32)
dispatch_scatter_kernel(const int* __restrict__ topk_ids, int P, int topk, int E, const int* __restrict__ blk,
                        int* __restrict__ sorted_token_ids, int* __restrict__ sorted_row,
                        int* __restrict__ slot_pos) {
    extern __shared__ int smem[];
    const int b0 = blockIdx.x * kDispBlockSlots, b1 = min(P, b0 + kDispBlockSlots);
    dispatch_hist(topk_ids, b0, b1, E, smem);
    for (int i = threadIdx.x; i < kDispWarps * E; i += kDispWarps * 32)
        smem[i] += blk[(size_t)blockIdx.x * E + i % E];
    __syncthreads();
    dispatch_scatter(topk_ids, b0, b1, topk, E, sorted_token_ids, sorted_row, slot_pos, smem);
}

size_t dispatch_scratch_bytes(int n, int topk, int E) {
    const size_t P = (size_t)n * topk;
    const size_t nblk = (P + kDispBlockSlots - 1) / kDispBlockSlots;
    return nblk * (size_t)E * sizeof(int);
}

int launch_dispatch(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                    int* sorted_token_ids, int* sorted_row, int* slot_pos, cudaStream_t s, int* scratch) {
    if (E > 1024) return GSB_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(kDispWarps * E + 1024) * sizeof(int);
    const int P = n * topk;
    const int nblk = (P + kDispBlockSlots - 1) / kDispBlockSlots;
    if (scratch && nblk > 2) {
        if (smem > 48 * 1024 &&
            (cudaFuncSetAttribute(dispatch_count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess ||
             cudaFuncSetAttribute(dispatch_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess))
            return GSB_ERR_CUDA;
        dispatch_count_kernel<<<nblk, kDispWarps * 32, smem, s>>>(topk_ids, P, E, scratch);
        dispatch_offsets_kernel<<<1, kDispWarps * 32, 0, s>>>(nblk, E, scratch, expert_offsets);
        dispatch_scatter_kernel<<<nblk, kDispWarps * 32, smem, s>>>(topk_ids, P, topk, E, scratch, sorted_token_ids,
                                                                   sorted_row, slot_pos);
        return launch_status();
    }
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    dispatch_kernel<<<1, kDispWarps * 32, smem, s>>>(topk_ids, n * topk, topk, E, expert_offsets,
                                                     sorted_token_ids, sorted_row, slot_pos);
    return launch_status();
}

}  // namespace gsb

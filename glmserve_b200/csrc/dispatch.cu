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

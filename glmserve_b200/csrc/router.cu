// Router: logits GEMM (bf16 x bf16 -> fp32) and sigmoid top-k selection.
//
// Selection semantics are those of the reference CPU loop (src/model_glm52.cpp:1113-1129)
// and of its warp kernel (cuda/moe_router.cu:17-79): key = sigmoid(logit) + bias, larger key
// first, equal keys to the smaller expert id; weight = the un-biased sigmoid; the weights
// are summed in selection order, divided by the sum when asked, and scaled.
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
template <int NS>
__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ e_bias, int n,
                   int E, int topk, int norm_topk, float routed_scale, int* __restrict__ topk_ids,
                   float* __restrict__ topk_w) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= n) return;
    const float* lt = logits + (size_t)t * E;
    float score[NS], key[NS];
#pragma unroll
    for (int j = 0; j < NS; ++j) {
        const int e = lane + (j << 5);
        if (e < E) {
            const float sc = sigmoid_ref(lt[e]);
            score[j] = sc;
            key[j] = __fadd_rn(sc, e_bias ? e_bias[e] : 0.0f);
        } else {
            score[j] = 0.0f;
            key[j] = 0.0f;
        }
    }
    uint32_t taken = 0;  // bit j: slot j already selected
    float wsum = 0.0f;
    float myw = 0.0f;    // lane k keeps the weight of selection k (topk <= 32)
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
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const int oe = __shfl_xor_sync(0xffffffffu, be, off);
            const float ok = __shfl_xor_sync(0xffffffffu, bk, off);
            const float os = __shfl_xor_sync(0xffffffffu, bs, off);
            const bool take = (oe != 0x7fffffff) &&
                              (be == 0x7fffffff || ok > bk || (ok == bk && oe < be));
            if (take) { be = oe; bk = ok; bs = os; }
        }
        // every lane now holds the same winner
        if ((be & 31) == lane && be != 0x7fffffff) taken |= 1u << (be >> 5);
        if (lane == 0) topk_ids[(size_t)t * topk + k] = be == 0x7fffffff ? 0 : be;
        wsum = __fadd_rn(wsum, bs);
        if (lane == k) myw = bs;
    }
    if (lane < topk) {
        float v = myw;
        if (norm_topk && wsum > 0.0f) v = __fdiv_rn(v, wsum);
        topk_w[(size_t)t * topk + lane] = __fmul_rn(v, routed_scale);
    }
}

int launch_router_topk(const float* logits, const float* e_bias, int n, int E, int topk,
                       int norm_topk, float routed_scale, int* ids, float* w, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    const int warps = 4;
    const unsigned grid = (unsigned)((n + warps - 1) / warps);
    if (E <= 256)
        router_topk_kernel<8><<<grid, warps * 32, 0, s>>>(logits, e_bias, n, E, topk, norm_topk,
                                                         routed_scale, ids, w);
    else
        router_topk_kernel<32><<<grid, warps * 32, 0, s>>>(logits, e_bias, n, E, topk, norm_topk,
                                                          routed_scale, ids, w);
    return launch_status();
}

// ---- router logits -----------------------------------------------------------------
// logits[t,e] = sum_i x[t,i] * Wr[e,i], bf16 inputs, fp32 accumulation.  A block stages TT
// token rows in shared memory once, then each of its 8 warps owns one expert row: lanes
// stride over the input dim 8 elements (16 bytes) at a time with the weight loads unrolled
// so several are in flight; partial sums are combined with a fixed xor tree.  The result
// for a (token, expert) does not depend on n or on the grid (the property the reference
// wants from its n-invariant gemv, cuda/gemm.cu:37-44).
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        f[2 * q] = __uint_as_float(u[q] << 16);
        f[2 * q + 1] = __uint_as_float(u[q] & 0xffff0000u);
    }
}

template <int TT>
__global__ void __launch_bounds__(256)
router_logits_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr,
                     int n, int H, int E, float* __restrict__ logits) {
    extern __shared__ uint4 xsm[];  // [TT][H/8]
    const int e = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int t0 = blockIdx.y * TT;
    const int lane = threadIdx.x & 31;
    const int nvec = H >> 3;
    for (int idx = threadIdx.x; idx < TT * nvec; idx += blockDim.x) {
        const int j = idx / nvec, v = idx - j * nvec;
        xsm[idx] = (t0 + j < n) ? __ldg(reinterpret_cast<const uint4*>(x + (size_t)(t0 + j) * H) + v)
                                : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads();
    if (e >= E) return;
    float acc[TT];
#pragma unroll
    for (int j = 0; j < TT; ++j) acc[j] = 0.0f;
    const uint4* wrow = reinterpret_cast<const uint4*>(wr + (size_t)e * H);
#pragma unroll 4
    for (int v = lane; v < nvec; v += 32) {
        float wf[8];
        bf16x8_to_f32(__ldg(wrow + v), wf);
#pragma unroll
        for (int j = 0; j < TT; ++j) {
            float xf[8];
            bf16x8_to_f32(xsm[j * nvec + v], xf);
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[j] = fmaf(xf[q], wf[q], acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < TT; ++j) {
        const float v = warp_sum(acc[j]);
        if (lane == 0 && t0 + j < n) logits[(size_t)(t0 + j) * E + e] = v;
    }
}

int launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* wr, int n, int H, int E,
                         float* logits, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    if (H % 8 != 0) return GSB_ERR_UNSUPPORTED;
    constexpr int TT = 8;
    const size_t smem = (size_t)TT * H * 2;
    if (smem > 200 * 1024) return GSB_ERR_UNSUPPORTED;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(router_logits_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    dim3 grid((unsigned)((E + 7) / 8), (unsigned)((n + TT - 1) / TT));
    router_logits_kernel<TT><<<grid, 256, smem, s>>>(x, wr, n, H, E, logits);
    return launch_status();
}

}  // namespace gsb

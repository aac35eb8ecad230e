// Direct-layout kernels: they read the reference's resident weight layout as it is
// (u8 [rows, in/2] two nibbles per byte, low nibble = even column; scales [rows, in/group])
// for ANY shape the quantiser allows.  They are the operator-surface implementation of
// moe_expert_ffn(_w4a16) / gemm_w4a16 and the path the native layer takes for shapes the
// tile-stream kernels do not cover.  fp32 accumulation throughout.
#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

// Warp-cooperative dot of one int4 row with an fp32 vector in shared memory.
// W[c] = (nibble(c) - 8) * sc[c / group]   (src/tensor.cpp:53-63 of the reference).
// in % 8 == 0, group % 8 == 0.  Returns the full sum in every lane.
template <typename ST>
__device__ __forceinline__ float dot_w4_row(const uint8_t* __restrict__ qrow,
                                            const ST* __restrict__ srow, const float* xs, int in,
                                            int group, int lane) {
    const uint32_t* q32 = reinterpret_cast<const uint32_t*>(qrow);
    const int nwords = in >> 3;
    float acc = 0.0f;
    for (int v = lane; v < nwords; v += 32) {
        const uint32_t wv = __ldg(q32 + v);
        const float sc = to_f32<ST>(srow[(v << 3) / group]);
        const float* xp = xs + (v << 3);
        float part = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int qv = (int)((wv >> (4 * j)) & 0xFu) - 8;
            part = fmaf((float)qv, xp[j], part);
        }
        acc = fmaf(part, sc, acc);
    }
    return warp_sum(acc);
}

__device__ __forceinline__ float dot_f32_row(const float* __restrict__ wrow, const float* xs,
                                             int in, int lane) {
    float acc = 0.0f;
    for (int i = lane; i < in; i += 32) acc = fmaf(__ldg(wrow + i), xs[i], acc);
    return warp_sum(acc);
}

// One block per token (the launch shape of the reference kernel, cuda/moe_expert.cu:132-244).
// For slot k = 0..topk-1 (then the shared expert): h = silu(gate x) * up x into shared
// memory, y = down h, acc[o] = acc[o] + w_k * y[o] with product and sum rounded separately,
// which is the reference CPU's accumulation (src/model_glm52.cpp:1141, :1151).
template <typename XT, typename ST, bool W4>
__global__ void __launch_bounds__(256)
generic_expert_kernel(GenericExpertArgs a) {
    extern __shared__ float sm[];
    float* xs = sm;               // [H]
    float* acc = sm + a.H;        // [H]
    float* hb = sm + 2 * a.H;     // [max(I, Is)]
    const int t = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const XT* xr = reinterpret_cast<const XT*>(a.x) + (size_t)t * a.H;
    for (int i = tid; i < a.H; i += blockDim.x) {
        xs[i] = to_f32<XT>(xr[i]);
        acc[i] = 0.0f;
    }
    __syncthreads();
    const int nslots = a.topk + (a.sg ? 1 : 0);
    for (int k = 0; k < nslots; ++k) {
        const bool shared = k >= a.topk;
        const int I = shared ? a.Is : a.I;
        const int e = shared ? 0 : a.ids[(size_t)t * a.topk + k];
        const float wk = shared ? 1.0f : a.w[(size_t)t * a.topk + k];
        if (!shared && (e < 0 || e >= a.E)) continue;  // caller error: contribute nothing
        const int ngh = a.H / a.group, ngi = I / a.group;
        for (int r = warp; r < I; r += nwarp) {
            float g, u;
            if (W4) {
                const uint8_t* gq = shared ? a.sg : reinterpret_cast<const uint8_t*>(a.gate) + (size_t)e * I * (a.H / 2);
                const uint8_t* uq = shared ? a.su : reinterpret_cast<const uint8_t*>(a.up) + (size_t)e * I * (a.H / 2);
                const ST* gs = shared ? reinterpret_cast<const ST*>(a.sg_sc) : reinterpret_cast<const ST*>(a.gate_sc) + (size_t)e * I * ngh;
                const ST* us = shared ? reinterpret_cast<const ST*>(a.su_sc) : reinterpret_cast<const ST*>(a.up_sc) + (size_t)e * I * ngh;
                g = dot_w4_row<ST>(gq + (size_t)r * (a.H / 2), gs + (size_t)r * ngh, xs, a.H, a.group, lane);
                u = dot_w4_row<ST>(uq + (size_t)r * (a.H / 2), us + (size_t)r * ngh, xs, a.H, a.group, lane);
            } else {
                g = dot_f32_row(reinterpret_cast<const float*>(a.gate) + ((size_t)e * I + r) * a.H, xs, a.H, lane);
                u = dot_f32_row(reinterpret_cast<const float*>(a.up) + ((size_t)e * I + r) * a.H, xs, a.H, lane);
            }
            if (lane == 0) hb[r] = __fmul_rn(silu_ref(g), u);
        }
        __syncthreads();
        for (int o = warp; o < a.H; o += nwarp) {
            float y;
            if (W4) {
                const uint8_t* dq = shared ? a.sd : reinterpret_cast<const uint8_t*>(a.down) + (size_t)e * a.H * (I / 2);
                const ST* ds = shared ? reinterpret_cast<const ST*>(a.sd_sc) : reinterpret_cast<const ST*>(a.down_sc) + (size_t)e * a.H * ngi;
                y = dot_w4_row<ST>(dq + (size_t)o * (I / 2), ds + (size_t)o * ngi, hb, I, a.group, lane);
            } else {
                y = dot_f32_row(reinterpret_cast<const float*>(a.down) + ((size_t)e * a.H + o) * I, hb, I, lane);
            }
            if (lane == 0) acc[o] = __fadd_rn(acc[o], __fmul_rn(wk, y));
        }
        __syncthreads();
    }
    float* orow = a.out + (size_t)t * a.H;
    const float* rrow = a.residual ? a.residual + (size_t)t * a.H : nullptr;
    for (int i = tid; i < a.H; i += blockDim.x) orow[i] = rrow ? __fadd_rn(rrow[i], acc[i]) : acc[i];
}

template <typename XT, typename ST, bool W4>
static int launch_generic_expert_t(const GenericExpertArgs& a, cudaStream_t s) {
    if (a.n == 0) return GSB_OK;
    const int imax = a.I > a.Is ? a.I : a.Is;
    const size_t smem = (size_t)(2 * a.H + imax) * sizeof(float);
    if (smem > 227 * 1024) return GSB_ERR_UNSUPPORTED;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(generic_expert_kernel<XT, ST, W4>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    generic_expert_kernel<XT, ST, W4><<<(unsigned)a.n, 256, smem, s>>>(a);
    return launch_status();
}

// xt: 0 = float, 1 = bf16.  st: 0 = float scales, 1 = fp16 scales.
int launch_generic_expert(const GenericExpertArgs& a, int xt, int st, bool w4, cudaStream_t s) {
    if (w4) {
        if (a.H % 8 || a.I % 8 || a.group % 8 || a.H % a.group || a.I % a.group) return GSB_ERR_UNSUPPORTED;
        if (a.sg && (a.Is % 8 || a.Is % a.group)) return GSB_ERR_UNSUPPORTED;
        if (xt == 0 && st == 0) return launch_generic_expert_t<float, float, true>(a, s);
        if (xt == 1 && st == 1) return launch_generic_expert_t<__nv_bfloat16, __half, true>(a, s);
        if (xt == 0 && st == 1) return launch_generic_expert_t<float, __half, true>(a, s);
        return GSB_ERR_UNSUPPORTED;
    }
    if (xt == 0) return launch_generic_expert_t<float, float, false>(a, s);
    return GSB_ERR_UNSUPPORTED;
}

// y[t,o] = sum_i W[o,i] x[t,i] (+ bias[o]); one warp per output row, TT tokens per pass.
template <int TT>
__global__ void __launch_bounds__(256)
generic_gemm_w4_kernel(const float* __restrict__ x, const uint8_t* __restrict__ qW,
                       const float* __restrict__ scales, const float* __restrict__ bias,
                       float* __restrict__ y, int64_t n, int64_t in, int64_t out, int group) {
    const int64_t o = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (o >= out) return;
    const uint32_t* q32 = reinterpret_cast<const uint32_t*>(qW + o * (in / 2));
    const float* srow = scales + o * (in / group);
    const int nwords = (int)(in >> 3);
    for (int64_t t0 = (int64_t)blockIdx.y * TT; t0 < n; t0 += (int64_t)gridDim.y * TT) {
        float acc[TT];
#pragma unroll
        for (int j = 0; j < TT; ++j) acc[j] = 0.0f;
        for (int v = lane; v < nwords; v += 32) {
            const uint32_t wv = __ldg(q32 + v);
            const float sc = srow[(v << 3) / group];
            float wf[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) wf[j] = (float)((int)((wv >> (4 * j)) & 0xFu) - 8) * sc;
#pragma unroll
            for (int j = 0; j < TT; ++j) {
                if (t0 + j < n) {
                    const float* xp = x + (t0 + j) * in + ((int64_t)v << 3);
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc[j] = fmaf(wf[q], xp[q], acc[j]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < TT; ++j) {
            const float v = warp_sum(acc[j]);
            if (lane == 0 && t0 + j < n) y[(t0 + j) * out + o] = bias ? v + bias[o] : v;
        }
    }
}

int launch_generic_gemm_w4(const float* x, const uint8_t* qW, const float* scales,
                           const float* bias, float* y, int64_t n, int64_t in, int64_t out,
                           int64_t group, cudaStream_t s) {
    if (n == 0 || out == 0) return GSB_OK;
    if (in % 8 || group % 8 || in % group) return GSB_ERR_UNSUPPORTED;
    constexpr int TT = 4;
    int64_t gy = (n + TT - 1) / TT;
    if (gy > 4096) gy = 4096;
    dim3 grid((unsigned)((out + 7) / 8), (unsigned)gy);
    generic_gemm_w4_kernel<TT><<<grid, 256, 0, s>>>(x, qW, scales, bias, y, n, in, out, (int)group);
    return launch_status();
}

// ---- glue ----------------------------------------------------------------------------
__global__ void silu_mul_kernel(const float* g, const float* u, float* out, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fmul_rn(silu_ref(g[i]), u[i]);
}
__global__ void add_inplace_kernel(float* y, const float* x, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __fadd_rn(y[i], x[i]);
}
__global__ void add_bias_rows_kernel(float* y, const float* __restrict__ bias, int64_t total, int64_t cols) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) y[i] = __fadd_rn(y[i], bias[i % cols]);
}
int launch_add_bias_rows(float* y, const float* bias, int64_t n, int64_t cols, cudaStream_t s) {
    if (n * cols == 0) return GSB_OK;
    add_bias_rows_kernel<<<(unsigned)((n * cols + 255) / 256), 256, 0, s>>>(y, bias, n * cols, cols);
    return launch_status();
}
int launch_silu_mul(const float* g, const float* u, float* out, int64_t n, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(g, u, out, n);
    return launch_status();
}
int launch_add_inplace(float* y, const float* x, int64_t n, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    add_inplace_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(y, x, n);
    return launch_status();
}

// Row RMSNorm with the CPU reference's arithmetic (src/model_glm52.cpp:61-71): sum of
// squares in double, inv = (float)(1/sqrt(ss/dim + eps)), y = x*inv*w.  The double sum is
// taken in a fixed tree order, so it can differ from the sequential CPU sum only in the
// last bits of a double - far below float resolution.  OT = float or bf16 output.
template <typename OT>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, OT* __restrict__ out,
               int64_t d, float eps) {
    __shared__ double red[8];
    __shared__ float inv_s;
    const float* xr = x + (int64_t)blockIdx.x * d;
    double ss = 0.0;
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) ss += (double)xr[i] * (double)xr[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
        double tot = 0.0;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) tot += red[i];
        inv_s = (float)(1.0 / sqrt(tot / (double)d + (double)eps));
    }
    __syncthreads();
    const float inv = inv_s;
    OT* orow = out + (int64_t)blockIdx.x * d;
    for (int64_t i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = __fmul_rn(__fmul_rn(xr[i], inv), w[i]);
        if constexpr (sizeof(OT) == 4) orow[i] = v; else orow[i] = __float2bfloat16_rn(v);
    }
}
int launch_rmsnorm_f32(const float* x, const float* w, float* out, int64_t n, int64_t d, float eps,
                       cudaStream_t s) {
    if (n == 0) return GSB_OK;
    rmsnorm_kernel<float><<<(unsigned)n, 256, 0, s>>>(x, w, out, d, eps);
    return launch_status();
}
int launch_rmsnorm_bf16(const float* x, const float* w, __nv_bfloat16* out, int64_t n, int64_t d,
                        float eps, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    rmsnorm_kernel<__nv_bfloat16><<<(unsigned)n, 256, 0, s>>>(x, w, out, d, eps);
    return launch_status();
}

// Per-32 absmax int8 activation quantiser (cuda/qgemm.cu:569-587 of the reference).
__global__ void quantize_act_q8_kernel(const float* __restrict__ x, int64_t nblocks,
                                       int8_t* __restrict__ xq, float* __restrict__ xs) {
    const int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (b >= nblocks) return;
    const int lane = threadIdx.x & 31;
    const float v = x[b * 32 + lane];
    float amax = fabsf(v);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sx = amax / 127.0f;
    const float id = sx > 0.0f ? 1.0f / sx : 0.0f;
    xq[b * 32 + lane] = (int8_t)__float2int_rn(v * id);
    if (lane == 0) xs[b] = sx;
}
int launch_quantize_act_q8(const float* x, int64_t n, int64_t in, int8_t* xq, float* xs,
                           cudaStream_t s) {
    if (in % 32) return GSB_ERR_UNSUPPORTED;
    const int64_t nblocks = n * (in >> 5);
    if (nblocks == 0) return GSB_OK;
    quantize_act_q8_kernel<<<(unsigned)((nblocks + 7) / 8), 256, 0, s>>>(x, nblocks, xq, xs);
    return launch_status();
}

__global__ void f32_to_bf16_kernel(const float* x, __nv_bfloat16* y, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = __float2bfloat16_rn(x[i]);
}
int launch_f32_to_bf16(const float* x, __nv_bfloat16* y, int64_t n, cudaStream_t s) {
    if (n == 0) return GSB_OK;
    f32_to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(x, y, n);
    return launch_status();
}

}  // namespace gsb

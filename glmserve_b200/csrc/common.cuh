// Shared device/host helpers for the sm_100a MoE kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/glmserve_b200.h"

namespace gsb {

constexpr int kWarp = 32;

// Status word layout in the workspace header (device memory, int32[8]).
enum StatusSlot { kStatusCode = 0, kStatusWhere = 1, kStatusAux = 2 };

inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? GSB_OK : GSB_ERR_LAUNCH;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// silu exactly as the CPU reference writes it (src/model_glm52.cpp:95): x / (1 + exp(-x)).
__device__ __forceinline__ float silu_ref(float x) { return __fdiv_rn(x, 1.0f + expf(-x)); }

// largest finite fp16 instead of infinity: an intermediate beyond +-65504 must not turn into
// inf and then NaN (inf * 0) further down; the fp32 reference has no such cliff
__device__ __forceinline__ __half sat_half(float v) {
    return __float2half_rn(fminf(fmaxf(v, -65504.f), 65504.f));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier + bulk-copy wrappers (all waits are bounded by the caller) -------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while before it answers).
__device__ __forceinline__ uint32_t mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok;
}
// Bounded wait: gives up after `limit_cycles` SM clock cycles and returns false (the caller
// records the error and leaves); a wait that would otherwise hang the GPU ends in about a
// second instead.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit_cycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - start > limit_cycles) return false;
    }
    return true;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
            "r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// position (in halves) of feature f inside a fragment-ordered row: within each block of
// 128 features the sixteen 8-feature groups are stored transposed (group 4t+j at 4j+t), so
// that the four lanes of a quad read adjacent 16-byte pieces.
__device__ __host__ __forceinline__ int frag_pos(int f) {
    const int kb = f >> 7, kk = f & 127;
    const int t = kk >> 5, j = (kk >> 3) & 3, el = kk & 7;
    return (kb << 7) + (((j << 2) + t) << 3) + el;
}

// Four bf16 pairs -> fp16 (exact for |x| in the fp16 normal range; values beyond +-65504
// saturate to the largest finite fp16).
__device__ __forceinline__ uint4 bf16x8_to_half8(const uint4& v) {
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
    return o;
}

// Eight fp32 values (a0, a1) normalised as the CPU reference does (src/model_glm52.cpp:61-71:
// x * inv * w, each product rounded) and rounded to bf16, as four packed pairs.
__device__ __forceinline__ uint4 norm8_bf16(const uint4& a0, const uint4& a1, const uint4& w0, const uint4& w1, float inv) {
    const float xv[8] = {__uint_as_float(a0.x), __uint_as_float(a0.y), __uint_as_float(a0.z), __uint_as_float(a0.w),
                         __uint_as_float(a1.x), __uint_as_float(a1.y), __uint_as_float(a1.z), __uint_as_float(a1.w)};
    const float wv[8] = {__uint_as_float(w0.x), __uint_as_float(w0.y), __uint_as_float(w0.z), __uint_as_float(w0.w),
                         __uint_as_float(w1.x), __uint_as_float(w1.y), __uint_as_float(w1.z), __uint_as_float(w1.w)};
    uint4 o;
    uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(__fmul_rn(__fmul_rn(xv[2 * q], inv), wv[2 * q]),
                                                       __fmul_rn(__fmul_rn(xv[2 * q + 1], inv), wv[2 * q + 1]));
        op[q] = *reinterpret_cast<const uint32_t*>(&b);
    }
    return o;
}

// One 8-feature group of a bf16 row -> fp16, at its fragment-order position or (natural != 0) in place.
__device__ __forceinline__ void xprep_group(const __nv_bfloat16* __restrict__ x, __half* __restrict__ xp,
                                            int64_t row, int grp, int H, int natural = 0) {
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + row * H) + grp);
    *reinterpret_cast<uint4*>(xp + row * H + (natural ? (grp << 3) : frag_pos(grp << 3))) = bf16x8_to_half8(v);
}
// The same from an fp32 hidden state through the pre-norm: fp16(bf16(x * inv * w)).
__device__ __forceinline__ void xprep_group_norm(const float* __restrict__ hidden, const float* __restrict__ norm_w,
                                                 float inv, __half* __restrict__ xp, int64_t row, int grp, int H,
                                                 int natural) {
    const uint4* hp = reinterpret_cast<const uint4*>(hidden + row * H) + 2 * grp;
    const uint4* wp = reinterpret_cast<const uint4*>(norm_w) + 2 * grp;
    const uint4 v = norm8_bf16(__ldg(hp), __ldg(hp + 1), __ldg(wp), __ldg(wp + 1), inv);
    *reinterpret_cast<uint4*>(xp + row * H + (natural ? (grp << 3) : frag_pos(grp << 3))) = bf16x8_to_half8(v);
}

}  // namespace gsb

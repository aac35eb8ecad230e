// Router: logits GEMM (bf16 x bf16 -> fp32) and sigmoid top-k selection.
//
// Selection semantics are those of the reference CPU loop (src/model_glm52.cpp:1113-1129)
// and of its warp kernel (cuda/moe_router.cu:17-79): key = sigmoid(logit) + bias, larger key
// first, equal keys to the smaller expert id; weight = the un-biased sigmoid; the weights
// are summed in selection order, divided by the sum when asked, and scaled.
#include "common.cuh"
#include "launchers.cuh"
#include "route_device.cuh"

namespace gsb {

// One warp per token.
template <int NS, bool FROM_SCORES>
__global__ void __launch_bounds__(128)
router_topk_kernel(const float* __restrict__ logits, const float* __restrict__ e_bias, int n,
                   int E, int topk, int norm_topk, float routed_scale, int* __restrict__ topk_ids,
                   float* __restrict__ topk_w) {
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= n) return;
    topk_token<NS, FROM_SCORES>(logits + (size_t)t * E, e_bias, E, topk, norm_topk, routed_scale, threadIdx.x & 31,
                                topk_ids + (size_t)t * topk, topk_w + (size_t)t * topk);
}

int launch_router_topk(const float* logits, const float* e_bias, int n, int E, int topk,
                       int norm_topk, float routed_scale, int* ids, float* w, cudaStream_t s,
                       bool from_scores) {
    if (n == 0) return GSB_OK;
    const int warps = 4;
    const unsigned grid = (unsigned)((n + warps - 1) / warps);
#define GSB_TOPK(NS, FS) router_topk_kernel<NS, FS><<<grid, warps * 32, 0, s>>>(logits, e_bias, n, E, topk, norm_topk, routed_scale, ids, w)
    if (E <= 256) { if (from_scores) GSB_TOPK(8, true); else GSB_TOPK(8, false); }
    else { if (from_scores) GSB_TOPK(32, true); else GSB_TOPK(32, false); }
#undef GSB_TOPK
    return launch_status();
}

// Router-less layers (a dense MLP cut into topk slices): slot k of every token is expert k, weight 1.
__global__ void fixed_routing_kernel(int64_t total, int topk, int* __restrict__ ids, float* __restrict__ w) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < total) { ids[i] = (int)(i % topk); w[i] = 1.0f; }
}

int launch_fixed_routing(int n, int topk, int* ids, float* w, cudaStream_t s) {
    const int64_t total = (int64_t)n * topk;
    if (total == 0) return GSB_OK;
    fixed_routing_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(total, topk, ids, w);
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

// Tensor-core form for input dims that are multiples of 256: mma.sync m16n8k16 (bf16 in,
// fp32 accumulate) with 16 experts as M and 8 tokens as N.  Both operands come straight from
// global memory as 16-byte loads: lane (g,t) reads columns 8t..8t+7 of every 32-column block
// of expert rows g, g+8 and of token g, and the two k16 steps of the block use the first and
// second half of those 16 bytes - the k index of an mma is only a label, so any assignment
// of columns works as long as A and B use the same one.
// The 8 warps of a block split the input dim and their partial tiles are added in warp order
// through shared memory, so even a few tokens make many blocks:
//   MT = 1, NT = 1 (n <= 128): 16 experts x 8 tokens per block;
//   MT = 4, NT = 4 (n > 128): 64 experts x 32 tokens per block - a quarter of the re-reads of the
//     activations from L2 (at 8192 tokens 132 us; a warp that walks the whole input dim alone
//     waits on every load and took 600 us).
// The result for a (token, expert) depends only on the variant, never on n or the grid.
// The epilogue also stores sigmoid(logit) (scores, nullable) for the fused top-k.
// ORDERED = false lets the compiler move loads across the mma (the small tiling batches its loads and
// needs that freedom); the large tiling keeps the volatile form, whose schedule fits 128 registers
// without spills.
template <bool ORDERED>
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    if (ORDERED)
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
            "{%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NORM: the activations are bf16(rmsnorm(hidden)) of an fp32 hidden state (the layer's pre-norm,
// src/model_gpu.cpp:1430 of the reference, folded into this launch): every block first takes the
// inverse RMS of its token rows - the same thread-strided double sums in the same order as
// rmsnorm_kernel, so the normalised values are the bits a separate norm pass would produce - and
// normalises and rounds to bf16 as it loads.
template <int MT, int NT, int KSPLIT, bool NORM>
__global__ void __launch_bounds__(256)
router_logits_mma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wr,
                         int n, int H, int E, float* __restrict__ logits, float* __restrict__ scores,
                         __half* __restrict__ xp, int xp_natural, const float* __restrict__ hidden,
                         const float* __restrict__ norm_w, float eps) {
    extern __shared__ float red[];   // KSPLIT > 1: [8 warps][MT][NT][4][32] partial tiles
    __shared__ double nred[8];
    __shared__ float inv_s[8 * NT];
    // the routing kernel that follows may be scheduled now; it waits for this grid before it reads
    // (a no-op unless that launch asks for programmatic serialization)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (NORM) {
        const int rows = min(8 * NT, n - (int)blockIdx.y * (8 * NT));
        for (int r = 0; r < rows; ++r) {
            const float* xr = hidden + ((int64_t)blockIdx.y * (8 * NT) + r) * H;
            double ss = 0.0;
            for (int i = threadIdx.x; i < H; i += 256) ss += (double)xr[i] * (double)xr[i];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if ((threadIdx.x & 31) == 0) nred[threadIdx.x >> 5] = ss;
            __syncthreads();
            if (threadIdx.x == 0) {
                double tot = 0.0;
                for (int i = 0; i < 8; ++i) tot += nred[i];
                inv_s[r] = (float)(1.0 / sqrt(tot / (double)H + (double)eps));
            }
            __syncthreads();
        }
    }
    if (xp && (int)blockIdx.x * (16 * MT) >= E) {
        // one column of blocks beyond the experts: this block's token rows as fp16 for the expert
        // GEMMs - in the decode kernels' fragment order or in natural order (tcgen05 path) - which
        // saves a launch; the logits blocks read the same rows anyway
        const int gpr = H >> 3, rows = min(8 * NT, n - (int)blockIdx.y * (8 * NT));
        for (int i = threadIdx.x; i < rows * gpr; i += 256) {
            const int r = i / gpr;
            const int64_t row = (int64_t)blockIdx.y * (8 * NT) + r;
            if (NORM) xprep_group_norm(hidden, norm_w, inv_s[r], xp, row, i - r * gpr, H, xp_natural);
            else xprep_group(x, xp, row, i - r * gpr, H, xp_natural);
        }
        return;
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int egroup = KSPLIT > 1 ? blockIdx.x : blockIdx.x * 8 + warp;
    const int e0 = egroup * (16 * MT);
    const int t0 = blockIdx.y * (8 * NT);
    const int kslice = H / KSPLIT;
    const int kbeg = KSPLIT > 1 ? warp * kslice : 0;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint4* pa[MT];
    const uint4* pb[MT];
    bool ra_ok[MT], rb_ok[MT];
#pragma unroll
    for (int j = 0; j < MT; ++j) {
        ra_ok[j] = e0 + j * 16 + g < E;
        rb_ok[j] = e0 + j * 16 + g + 8 < E;
        pa[j] = reinterpret_cast<const uint4*>(wr + (size_t)(ra_ok[j] ? e0 + j * 16 + g : 0) * H + kbeg) + t;
        pb[j] = reinterpret_cast<const uint4*>(wr + (size_t)(rb_ok[j] ? e0 + j * 16 + g + 8 : 0) * H + kbeg) + t;
    }
    const uint4* px[NT];
    bool x_ok[NT];
    float xinv[NT];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
        const int tok = t0 + i * 8 + g;
        x_ok[i] = tok < n;
        if (NORM) {
            px[i] = reinterpret_cast<const uint4*>(hidden + (size_t)(x_ok[i] ? tok : 0) * H + kbeg) + 2 * t;
            xinv[i] = x_ok[i] ? inv_s[i * 8 + g] : 0.f;
        } else {
            px[i] = reinterpret_cast<const uint4*>(x + (size_t)(x_ok[i] ? tok : 0) * H + kbeg) + t;
            xinv[i] = 0.f;
        }
    }
    const uint4* pnw = reinterpret_cast<const uint4*>(norm_w + (NORM ? kbeg : 0)) + 2 * t;
    // eight activations of a 32-column block as bf16: loaded as such, or normalised from fp32
    auto load_x = [&](int i, int it) -> uint4 {
        if (!NORM) return __ldg(px[i] + it * 4);
        const uint4 a0 = __ldg(px[i] + it * 8), a1 = __ldg(px[i] + it * 8 + 1);
        const uint4 w0 = __ldg(pnw + it * 8), w1 = __ldg(pnw + it * 8 + 1);
        return norm8_bf16(a0, a1, w0, w1, xinv[i]);
    };
    float acc[MT][NT][4];
#pragma unroll
    for (int j = 0; j < MT; ++j)
#pragma unroll
        for (int i = 0; i < NT; ++i) { acc[j][i][0] = acc[j][i][1] = acc[j][i][2] = acc[j][i][3] = 0.f; }
    const int iters = kslice >> 5;
    if (e0 < E) {
        // kBatch iterations' loads are issued before their mma: the loop is a chain of L2 round
        // trips otherwise (a 16-expert x 8-token block has only three loads per iteration)
        constexpr int kBatch = MT * NT >= 8 ? 1 : (MT * NT >= 4 ? 2 : 8);
        if (kBatch == 1) {
#pragma unroll 1
            for (int it = 0; it < iters; ++it) {
                uint4 va[MT], vb[MT], vx[NT];
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    va[j] = ra_ok[j] ? __ldg(pa[j] + it * 4) : zero;
                    vb[j] = rb_ok[j] ? __ldg(pb[j] + it * 4) : zero;
                }
#pragma unroll
                for (int i = 0; i < NT; ++i) vx[i] = x_ok[i] ? load_x(i, it) : zero;
#pragma unroll
                for (int j = 0; j < MT; ++j)
#pragma unroll
                    for (int i = 0; i < NT; ++i) {
                        mma_bf16_16816<true>(acc[j][i], va[j].x, vb[j].x, va[j].y, vb[j].y, vx[i].x, vx[i].y);
                        mma_bf16_16816<true>(acc[j][i], va[j].z, vb[j].z, va[j].w, vb[j].w, vx[i].z, vx[i].w);
                    }
            }
        } else
        for (int it0 = 0; it0 < iters; it0 += kBatch) {
            uint4 va[kBatch][MT], vb[kBatch][MT], vx[kBatch][NT];
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                const int it = it0 + u;
                const bool in = it < iters;
#pragma unroll
                for (int j = 0; j < MT; ++j) {
                    va[u][j] = (in && ra_ok[j]) ? __ldg(pa[j] + it * 4) : zero;
                    vb[u][j] = (in && rb_ok[j]) ? __ldg(pb[j] + it * 4) : zero;
                }
#pragma unroll
                for (int i = 0; i < NT; ++i) vx[u][i] = (in && x_ok[i]) ? load_x(i, it) : zero;
            }
#pragma unroll
            for (int u = 0; u < kBatch; ++u) {
                if (it0 + u >= iters) break;   // zeros would add nothing, but keep the count exact
#pragma unroll
                for (int j = 0; j < MT; ++j)
#pragma unroll
                    for (int i = 0; i < NT; ++i) {
                        mma_bf16_16816<false>(acc[j][i], va[u][j].x, vb[u][j].x, va[u][j].y, vb[u][j].y, vx[u][i].x, vx[u][i].y);
                        mma_bf16_16816<false>(acc[j][i], va[u][j].z, vb[u][j].z, va[u][j].w, vb[u][j].w, vx[u][i].z, vx[u][i].w);
                    }
            }
        }
    }
    if (KSPLIT > 1) {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) red[(((warp * MT + j) * NT + i) * 4 + c) * 32 + lane] = acc[j][i][c];
        __syncthreads();
        for (int o = threadIdx.x; o < MT * NT * 128; o += 256) {
            const int c = (o >> 5) & 3, i = (o >> 7) % NT, j = (o >> 7) / NT;   // lane keeps its (g,t)
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) v += red[(((w * MT + j) * NT + i) * 4 + c) * 32 + lane];
            const int e = e0 + j * 16 + g + ((c >> 1) << 3), tok = t0 + i * 8 + 2 * t + (c & 1);
            if (e < E && tok < n) {
                logits[(size_t)tok * E + e] = v;
                if (scores) scores[(size_t)tok * E + e] = sigmoid_ref(v);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int e = e0 + j * 16 + g + ((c >> 1) << 3), tok = t0 + i * 8 + 2 * t + (c & 1);
                    if (e < E && tok < n) {
                        logits[(size_t)tok * E + e] = acc[j][i][c];
                        if (scores) scores[(size_t)tok * E + e] = sigmoid_ref(acc[j][i][c]);
                    }
                }
    }
}

__global__ void sigmoid_scores_kernel(const float* __restrict__ logits, float* __restrict__ scores, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) scores[i] = sigmoid_ref(logits[i]);
}

template <bool NORM>
static int launch_logits_mma(const __nv_bfloat16* x, const __nv_bfloat16* wr, int n, int H, int E, float* logits,
                             float* scores, cudaStream_t s, __half* xp, int xp_natural, const float* hidden,
                             const float* norm_w, float eps) {
    if (n <= 128) {
        dim3 grid((unsigned)((E + 15) / 16) + (xp ? 1u : 0u), (unsigned)((n + 7) / 8));
        router_logits_mma_kernel<1, 1, 8, NORM><<<grid, 256, 8 * 512, s>>>(x, wr, n, H, E, logits, scores, xp, xp_natural,
                                                                         hidden, norm_w, eps);
    } else {
        constexpr int smem = 8 * 4 * 4 * 512;   // 64 KiB of partial tiles
        if (cudaFuncSetAttribute(router_logits_mma_kernel<4, 4, 8, NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem) != cudaSuccess)
            return GSB_ERR_CUDA;
        dim3 grid((unsigned)((E + 63) / 64) + (xp ? 1u : 0u), (unsigned)((n + 31) / 32));
        router_logits_mma_kernel<4, 4, 8, NORM><<<grid, 256, smem, s>>>(x, wr, n, H, E, logits, scores, xp, xp_natural,
                                                                      hidden, norm_w, eps);
    }
    return launch_status();
}

// x (bf16) or, when `hidden` is given, bf16(rmsnorm(hidden, norm_w, eps)) computed on the fly.
// xp (nullable, input dims that are multiples of 256 only): the same activations as fp16 rows for the
// expert GEMMs, in fragment order (xp_natural = 0) or natural order (1).
int launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* wr, int n, int H, int E,
                         float* logits, float* scores, cudaStream_t s, __half* xp, int xp_natural,
                         const float* hidden, const float* norm_w, float eps) {
    if (n == 0) return GSB_OK;
    if (H % 8 != 0) return GSB_ERR_UNSUPPORTED;
    if (H % 256 == 0) {
        if (hidden) return launch_logits_mma<true>(nullptr, wr, n, H, E, logits, scores, s, xp, xp_natural, hidden, norm_w, eps);
        return launch_logits_mma<false>(x, wr, n, H, E, logits, scores, s, xp, xp_natural, nullptr, nullptr, 0.f);
    }
    if (xp || hidden) return GSB_ERR_INVALID_ARG;
    constexpr int TT = 8;
    const size_t smem = (size_t)TT * H * 2;
    if (smem > 200 * 1024) return GSB_ERR_UNSUPPORTED;
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(router_logits_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return GSB_ERR_CUDA;
    dim3 grid((unsigned)((E + 7) / 8), (unsigned)((n + TT - 1) / TT));
    router_logits_kernel<TT><<<grid, 256, smem, s>>>(x, wr, n, H, E, logits);
    if (scores) sigmoid_scores_kernel<<<(unsigned)(((int64_t)n * E + 255) / 256), 256, 0, s>>>(logits, scores, (int64_t)n * E);
    return launch_status();
}

}  // namespace gsb

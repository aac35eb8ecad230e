// Header-only shim: the reference's operator names (namespace glmserve::cuda, declared in
// cuda/kernels.cuh of the reference) implemented on the C ABI of libglmserve_b200.so, with the
// same parameter lists and default arguments, so that the reference's caller
// (src/model_gpu.cpp, tests/test_moe_router.cpp, tests/test_qgemm.cpp) compiles and links
// unchanged once the matching declarations/definitions are taken from here instead of
// cuda/moe_router.cu, cuda/moe_dispatch.cu, cuda/moe_expert.cu, cuda/int4_gemm.cu and the MoE
// part of cuda/qgemm.cu.
//
// Error convention: the reference's wrappers return void and the caller polls
// cudaGetLastError() once per forward (src/model_gpu.cpp:393-398).  The shim keeps a sticky
// status: the first non-zero status of any call is remembered and can be read (and cleared)
// with glmserve::cuda::b200_last_status(); a maintainer adds that read to cuda_check().
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "glmserve_b200.h"

namespace glmserve {
namespace cuda {

inline int& b200_sticky_status() {
    static thread_local int st = GSB_OK;
    return st;
}
inline void b200_note(int st) {
    if (st != GSB_OK && b200_sticky_status() == GSB_OK) b200_sticky_status() = st;
}
// Returns the first error since the last call and clears it (GSB_OK = none).
inline int b200_last_status() {
    const int st = b200_sticky_status();
    b200_sticky_status() = GSB_OK;
    return st;
}

// Not in the reference: switches on the fast path behind moe_expert_ffn_w4a16 / gemm_w4a16 (weights repacked
// once per set of pointers, tile-stream kernels from then on; see gsb_operator_cache_enable).  A maintainer
// calls it once after the weights are uploaded (src/model_gpu.cpp:948-1000), with the bytes of int4 weights
// the engine is willing to hold twice; without it every call runs the direct-layout kernels.
inline void b200_enable_operator_cache(size_t max_weight_bytes) { b200_note(gsb_operator_cache_enable(max_weight_bytes)); }

// cuda/kernels.cuh:243-245
inline void moe_router(const float* logits, const float* e_bias, int n, int E, int topk,
                       bool norm_topk, float routed_scale, int* topk_ids, float* topk_weights,
                       cudaStream_t s = 0) {
    b200_note(gsb_moe_router(logits, e_bias, n, E, topk, norm_topk ? 1 : 0, routed_scale, topk_ids,
                             topk_weights, s));
}

// cuda/kernels.cuh:249-250
inline void moe_dispatch(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                         int* sorted_token_ids, int* sorted_row, cudaStream_t s = 0) {
    b200_note(gsb_moe_dispatch(topk_ids, n, topk, E, expert_offsets, sorted_token_ids, sorted_row, s));
}

// cuda/kernels.cuh:254-257
inline void moe_expert_ffn(const float* x, const int* topk_ids, const float* topk_weights,
                           const float* gate_w, const float* up_w, const float* down_w, int n,
                           int topk, int hidden, int moe_inter, int E, float* out,
                           cudaStream_t s = 0) {
    b200_note(gsb_moe_expert_ffn(x, topk_ids, topk_weights, gate_w, up_w, down_w, n, topk, hidden,
                                 moe_inter, E, out, s));
}

// cuda/kernels.cuh:259-268
inline void moe_expert_ffn_w4a16(const float* x, const int* topk_ids, const float* topk_weights,
                                 const uint8_t* gate_q, const float* gate_sc, const uint8_t* up_q,
                                 const float* up_sc, const uint8_t* down_q, const float* down_sc,
                                 int n, int topk, int hidden, int moe_inter, int E, int group_size,
                                 float* out, cudaStream_t s = 0) {
    b200_note(gsb_moe_expert_ffn_w4a16(x, topk_ids, topk_weights, gate_q, gate_sc, up_q, up_sc, down_q,
                                       down_sc, n, topk, hidden, moe_inter, E, group_size, out, s));
}

// cuda/kernels.cuh:48-52
inline void gemm_w4a16(const float* x, const uint8_t* qW, const float* scales, const float* bias,
                       float* y, int64_t n, int64_t in, int64_t out, int64_t group_size,
                       cudaStream_t s = 0) {
    b200_note(gsb_gemm_w4a16(x, qW, scales, bias, y, n, in, out, group_size, s));
}

// cuda/kernels.cuh:18-19, :282-283
inline void rmsnorm(const float* x, const float* w, float* out, int64_t n, int64_t d, float eps,
                    cudaStream_t s = 0) {
    b200_note(gsb_rmsnorm(x, w, out, n, d, eps, s));
}
inline void add_inplace(float* y, const float* x, int64_t n, cudaStream_t s = 0) {
    b200_note(gsb_add_inplace(y, x, n, s));
}
inline void silu_mul(const float* g, const float* u, float* out, int64_t n, cudaStream_t s = 0) {
    b200_note(gsb_silu_mul(g, u, out, n, s));
}

// ---- qgemm family, cuda/kernels.cuh:59-136 (GGML codecs report "unsupported") ----------
inline bool qtype_has_i8(uint32_t qtype) { return gsb_qtype_has_i8(qtype) != 0; }
inline void quantize_act_q8(const float* x, int64_t n, int64_t in, int8_t* xq, float* xs,
                            cudaStream_t s = 0) {
    b200_note(gsb_quantize_act_q8(x, n, in, xq, xs, s));
}
inline void gemm_q(uint32_t qtype, const float* x, const uint8_t* qW, const float* bias, float* y,
                   int64_t n, int64_t in, int64_t out, int64_t row_bytes, cudaStream_t s = 0) {
    b200_note(gsb_gemm_q(qtype, x, qW, bias, y, n, in, out, row_bytes, s));
}
inline void gemm_q_i8(uint32_t qtype, const int8_t* xq, const float* xs, const uint8_t* qW,
                      const float* bias, float* y, int64_t n, int64_t in, int64_t out,
                      int64_t row_bytes, cudaStream_t s = 0) {
    b200_note(gsb_gemm_q_i8(qtype, xq, xs, qW, bias, y, n, in, out, row_bytes, s));
}
inline void moe_expert_ffn_q(uint32_t gate_type, uint32_t up_type, uint32_t down_type, const float* x,
                             const int* topk_ids, const float* topk_w, const uint8_t* gate_q,
                             const uint8_t* up_q, const uint8_t* down_q, int n, int topk, int hidden,
                             int moe_inter, int E, int64_t gate_row_bytes, int64_t up_row_bytes,
                             int64_t down_row_bytes, float* h_act, float* dpart, float* out,
                             int* dispatch = nullptr, float* gu_part = nullptr, cudaStream_t s = 0) {
    b200_note(gsb_moe_expert_ffn_q(gate_type, up_type, down_type, x, topk_ids, topk_w, gate_q, up_q,
                                   down_q, n, topk, hidden, moe_inter, E, gate_row_bytes, up_row_bytes,
                                   down_row_bytes, h_act, dpart, out, dispatch, gu_part, s));
}
inline void moe_expert_ffn_q_i8(uint32_t gate_type, uint32_t up_type, uint32_t down_type,
                                const int8_t* xq, const float* xs, const int* topk_ids,
                                const float* topk_w, const uint8_t* gate_q, const uint8_t* up_q,
                                const uint8_t* down_q, int n, int topk, int hidden, int moe_inter, int E,
                                int64_t gate_row_bytes, int64_t up_row_bytes, int64_t down_row_bytes,
                                float* h_act, int8_t* hq, float* hs, float* dpart, float* out,
                                int* dispatch = nullptr, float* gu_part = nullptr, cudaStream_t s = 0) {
    b200_note(gsb_moe_expert_ffn_q_i8(gate_type, up_type, down_type, xq, xs, topk_ids, topk_w, gate_q,
                                      up_q, down_q, n, topk, hidden, moe_inter, E, gate_row_bytes,
                                      up_row_bytes, down_row_bytes, h_act, hq, hs, dpart, out, dispatch,
                                      gu_part, s));
}

}  // namespace cuda
}  // namespace glmserve

// gsb_moe_route_static: routing (router logits + top-k) for callers that must not allocate.
//
// The logits between the two kernels live in a fixed array that is part of the library
// image instead of in caller scratch.  See include/glmserve_b200.h for the contract.
#include <mutex>

#include "common.cuh"
#include "launchers.cuh"

namespace {

// 64 Ki floats = 256 KiB of device memory held by every GPU that loads the library, from
// load until the process exits.
constexpr int kStaticLogitsFloats = 64 * 1024;
static __device__ __align__(256) float g_route_logits[kStaticLogitsFloats];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_logits_ptr[kMaxDevices] = {};  // device address of g_route_logits, per device

// In host code `g_route_logits` is only a handle for the runtime, not a device address, so the
// address each GPU gave the array is looked up once per device (with that device current)
// and that pointer is what the kernels receive.
int scratch_for_current_device(float** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return GSB_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_logits_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_route_logits) != cudaSuccess || !p) return GSB_ERR_CUDA;
        g_logits_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_logits_ptr[dev];
    return GSB_OK;
}

}  // namespace

extern "C" {

int gsb_moe_route_static_max_floats(void) { return kStaticLogitsFloats; }

int gsb_moe_route_static(const void* x_bf16, const void* router_w_bf16, const float* e_bias, int n,
                         int hidden, int E, int topk, int norm_topk, float routed_scale,
                         int* topk_ids, float* topk_weights, void* stream) {
    if (n < 0 || hidden <= 0 || E <= 0 || topk <= 0) return GSB_ERR_INVALID_ARG;
    if (n == 0) return GSB_OK;
    if (!x_bf16 || !router_w_bf16 || !topk_ids || !topk_weights) return GSB_ERR_INVALID_ARG;
    if ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(router_w_bf16)) & 15)
        return GSB_ERR_INVALID_ARG;
    if (E > 1024 || topk > 32 || topk > E) return GSB_ERR_UNSUPPORTED;
    if ((long long)n * E > kStaticLogitsFloats) return GSB_ERR_TOO_LARGE;
    float* logits = nullptr;
    int st = scratch_for_current_device(&logits);
    if (st) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    // every logit the top-k reads is written by the first kernel, so nothing left in the
    // array by an earlier call can leak into this one and nothing needs clearing
    st = gsb::launch_router_logits(reinterpret_cast<const __nv_bfloat16*>(x_bf16),
                                   reinterpret_cast<const __nv_bfloat16*>(router_w_bf16), n, hidden, E,
                                   logits, nullptr, s);
    if (st) return st;
    return gsb::launch_router_topk(logits, e_bias, n, E, topk, norm_topk, routed_scale, topk_ids,
                                   topk_weights, s);
}

}  // extern "C"

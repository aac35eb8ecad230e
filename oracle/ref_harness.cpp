// Harness around the UNMODIFIED reference sources (test infrastructure only).
//
// The reference's CPU float32 MoE (GLM52Model::moe_mlp) is a private member and its
// helpers (linear_forward, rmsnorm_rows) are file-static, so this translation unit
// textually includes the reference's own src/model_glm52.cpp from where it lies
// (REF_ROOT, given by oracle/Makefile) and exposes a few extern "C" entry points that
// build a MoEMLP from int4 tensors - dequantised with the reference's own
// dequant_int4_to_f32 - and call the reference functions.  No reference source is
// copied into this repository; the built library lands in oracle/_ref/.
#define private public
#define protected public
#include "model.hpp"
#undef private
#undef protected
#include "tensor.hpp"
#include "src/model_glm52.cpp"

#include <chrono>
#include <cstdint>
#include <cstring>

using namespace glmserve;

namespace {
Linear make_linear(const uint8_t* q, const float* sc, int64_t out, int64_t in, int64_t group) {
    Linear L;
    L.out_features = out;
    L.in_features = in;
    L.group_size = group;
    L.w.resize((size_t)out * in);
    dequant_int4_to_f32(q, sc, out * in, group, L.w.data());
    return L;
}
}  // namespace

extern "C" {

__attribute__((visibility("default")))
void ref_dequant_int4(const uint8_t* packed, const float* scales, int64_t count, int64_t group,
                      float* out) {
    dequant_int4_to_f32(packed, scales, count, group, out);
}

__attribute__((visibility("default")))
void ref_rmsnorm_rows(const float* x, const float* w, float* out, int64_t n, int64_t dim,
                      float eps) {
    rmsnorm_rows(x, w, out, n, dim, eps);
}

__attribute__((visibility("default")))
void ref_linear_forward(const float* w, const float* x, float* y, int64_t n, int64_t in,
                        int64_t out) {
    Linear L;
    L.out_features = out;
    L.in_features = in;
    L.w.assign(w, w + (size_t)out * in);
    linear_forward(L, x, y, n);
}

// A reference MoE layer kept alive across calls: GLM52Model + MoEMLP with fp32 weights
// dequantised once (what the reference holds after load).
struct RefLayer {
    GLM52Model model;
    MoEMLP m;
    explicit RefLayer(const GLM52Config& cfg) : model(cfg) {}
};

// `active` (nullable, length E) marks the experts that get dequantised fp32 weights; the
// others stay empty, so a caller that knows the routing can keep GLM-scale memory bounded
// (an expert the router picks while empty makes linear_forward throw -> ref_moe_run
// returns a negative value).  Returns NULL on failure.
__attribute__((visibility("default")))
void* ref_moe_create(int H, int I, int Is, int E, int topk, int group, const float* router_w,
                     const float* e_bias, int norm_topk, double routed_scale,
                     const uint8_t* gate_q, const float* gate_sc, const uint8_t* up_q,
                     const float* up_sc, const uint8_t* down_q, const float* down_sc,
                     const uint8_t* sg_q, const float* sg_sc, const uint8_t* su_q,
                     const float* su_sc, const uint8_t* sd_q, const float* sd_sc,
                     const uint8_t* active) {
    try {
        GLM52Config cfg;
        cfg.hidden_size = H;
        cfg.n_routed_experts = E;
        cfg.num_experts_per_tok = topk;
        cfg.moe_intermediate_size = I;
        cfg.routed_scaling_factor = routed_scale;
        cfg.norm_topk_prob = norm_topk != 0;
        RefLayer* R = new RefLayer(cfg);
        MoEMLP& m = R->m;
        m.router.out_features = E;
        m.router.in_features = H;
        m.router.w.assign(router_w, router_w + (size_t)E * H);
        if (e_bias) m.e_bias.assign(e_bias, e_bias + E);
        m.experts.resize(E);
        const int64_t qh = (H + 1) / 2, gh = (H + group - 1) / group;
        const int64_t qi = (I + 1) / 2, gi = (I + group - 1) / group;
        for (int e = 0; e < E; ++e) {
            if (active && !active[e]) continue;
            m.experts[e].gate_proj = make_linear(gate_q + (size_t)e * I * qh, gate_sc + (size_t)e * I * gh, I, H, group);
            m.experts[e].up_proj = make_linear(up_q + (size_t)e * I * qh, up_sc + (size_t)e * I * gh, I, H, group);
            m.experts[e].down_proj = make_linear(down_q + (size_t)e * H * qi, down_sc + (size_t)e * H * gi, H, I, group);
        }
        if (sg_q) {
            m.has_shared = true;
            m.shared.gate_proj = make_linear(sg_q, sg_sc, Is, H, group);
            m.shared.up_proj = make_linear(su_q, su_sc, Is, H, group);
            m.shared.down_proj = make_linear(sd_q, sd_sc, H, Is, group);
        }
        return R;
    } catch (const std::exception&) {
        return nullptr;
    }
}

// GLM52Model::moe_mlp on n token rows; returns the seconds spent inside it (< 0: failure).
__attribute__((visibility("default")))
double ref_moe_run(void* handle, const float* x, int n, float* out) {
    RefLayer* R = static_cast<RefLayer*>(handle);
    if (!R) return -1.0;
    try {
        auto t0 = std::chrono::steady_clock::now();
        R->model.moe_mlp(R->m, x, out, n);
        auto t1 = std::chrono::steady_clock::now();
        return std::chrono::duration<double>(t1 - t0).count();
    } catch (const std::exception&) {
        return -1.0;
    }
}

__attribute__((visibility("default")))
void ref_moe_destroy(void* handle) { delete static_cast<RefLayer*>(handle); }

// One-shot convenience: create, run, destroy.
__attribute__((visibility("default")))
double ref_moe_mlp_w4(const float* x, int n, int H, int I, int Is, int E, int topk, int group,
                      const float* router_w, const float* e_bias, int norm_topk,
                      double routed_scale, const uint8_t* gate_q, const float* gate_sc,
                      const uint8_t* up_q, const float* up_sc, const uint8_t* down_q,
                      const float* down_sc, const uint8_t* sg_q, const float* sg_sc,
                      const uint8_t* su_q, const float* su_sc, const uint8_t* sd_q,
                      const float* sd_sc, const uint8_t* active, float* out) {
    void* h = ref_moe_create(H, I, Is, E, topk, group, router_w, e_bias, norm_topk, routed_scale,
                             gate_q, gate_sc, up_q, up_sc, down_q, down_sc, sg_q, sg_sc, su_q, su_sc,
                             sd_q, sd_sc, active);
    if (!h) return -1.0;
    const double secs = ref_moe_run(h, x, n, out);
    ref_moe_destroy(h);
    return secs;
}

}  // extern "C"

// Host-callable launch functions shared between translation units.
#pragma once
#include "common.cuh"

namespace gsb {

// ---- tile-stream ("prepacked") weight format ------------------------------------------
// A matrix set is experts x units x chunks.  A unit is 32 weight rows (gate/up: gate rows
// 16u..16u+15 then up rows 16u..16u+15; down: rows 32u..32u+31); a chunk covers 512 input
// columns of one unit: eight 1 KiB weight blocks (block b = kstep*2 + half_unit, kstep = 128
// columns) followed by 256 bytes of fp16 scales [kstep][half_unit][16 rows].  Inside a
// block, lane L = 4*g + t of a warp owns 16 bytes at [L*16] (row g) and at [512 + L*16]
// (row g+8): the 32 columns 32t..32t+31 of the kstep as four words; in each word the eight
// nibbles hold columns (k0,k2,k4,k6,k1,k3,k5,k7) so that masking with 0x000f000f /
// 0x00f000f0 yields fp16 pairs of adjacent columns.
constexpr int kChunkCols = 512;
constexpr int kChunkWeightBytes = 8192;
constexpr int kChunkBytes = 8448;
constexpr int kDecodeTokens = 8;  // token rows per work item of the decode kernels

// from_scores: `logits` already holds sigmoid scores
int launch_fixed_routing(int n, int topk, int* ids, float* w, cudaStream_t s);
int launch_router_topk(const float* logits, const float* e_bias, int n, int E, int topk,
                       int norm_topk, float routed_scale, int* ids, float* w, cudaStream_t s,
                       bool from_scores = false);
// scores (nullable): also store sigmoid(logit).  xp (nullable): also write the activations as fp16 rows
// (fragment order, or natural order when xp_natural).  hidden (nullable): the activations are
// bf16(rmsnorm(hidden, norm_w, eps)) instead of x.
int launch_router_logits(const __nv_bfloat16* x, const __nv_bfloat16* wr, int n, int H, int E,
                         float* logits, float* scores, cudaStream_t s, __half* xp = nullptr, int xp_natural = 0,
                         const float* hidden = nullptr, const float* norm_w = nullptr, float eps = 0.f);
// scratch: dispatch_scratch_bytes() of device memory, or null (then one block does everything)
int launch_dispatch(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                    int* sorted_token_ids, int* sorted_row, int* slot_pos, cudaStream_t s, int* scratch = nullptr);
size_t dispatch_scratch_bytes(int n, int topk, int E);

struct GenericExpertArgs {
    const void* x;
    const int* ids;
    const float* w;
    const void* gate;
    const void* gate_sc;
    const void* up;
    const void* up_sc;
    const void* down;
    const void* down_sc;
    const uint8_t* sg; const void* sg_sc; const uint8_t* su; const void* su_sc;
    const uint8_t* sd; const void* sd_sc;
    int n, topk, H, I, Is, E, group;
    float* out;
    const float* residual;   // nullable: out = residual + layer (out may be the residual itself)
};
int launch_generic_expert(const GenericExpertArgs& a, int xt, int st, bool w4, cudaStream_t s);
int launch_generic_gemm_w4(const float* x, const uint8_t* qW, const float* scales,
                           const float* bias, float* y, int64_t n, int64_t in, int64_t out,
                           int64_t group, cudaStream_t s);
int launch_silu_mul(const float* g, const float* u, float* out, int64_t n, cudaStream_t s);
int launch_add_inplace(float* y, const float* x, int64_t n, cudaStream_t s);
int launch_rmsnorm_f32(const float* x, const float* w, float* out, int64_t n, int64_t d, float eps,
                       cudaStream_t s);
int launch_rmsnorm_bf16(const float* x, const float* w, __nv_bfloat16* out, int64_t n, int64_t d,
                        float eps, cudaStream_t s);
int launch_quantize_act_q8(const float* x, int64_t n, int64_t in, int8_t* xq, float* xs,
                           cudaStream_t s);
int launch_f32_to_bf16(const float* x, __nv_bfloat16* y, int64_t n, cudaStream_t s);

// b == nullptr: one matrix [experts, rows, cols] in units of 32 rows; else two matrices
// a (gate) and b (up), each [experts, rows, cols], interleaved 16 + 16 rows per unit.
int launch_prepack(const uint8_t* a_q, const void* a_sc, const uint8_t* b_q, const void* b_sc,
                   int scales_f32, int experts, int rows, int cols, void* out, cudaStream_t s);

size_t decode_seg_bytes(int n, int topk, int E);
size_t decode_seg_bytes_raw(size_t slots, size_t n_shared, int E);

struct DecodeArgs {
    const __nv_bfloat16* x;
    int n, topk, H, I, Is, E;
    int Id, Isd;             // input dims of the down projections as packed (0 = I / Is): a tensor-parallel shard
                             // whose intermediate slice is narrower than a 512-column chunk carries zero-weight
                             // columns beyond I / Is; the matching columns of hbuf must be finite (zeroed by the caller)
    const void* gate_up_packed;
    const void* down_packed;
    const void* shared_gate_up_packed;
    const void* shared_down_packed;
    const int* expert_offsets;
    const int* sorted_tok;
    const int* slot_pos;
    const float* topk_w;
    int* segs;
    __half* xp;
    __half* hbuf;
    float* ybuf;
    int* status;
    float* out;
    const float* residual;   // nullable: out = residual + layer (out may be the residual itself)
    int sm_count;
    int force_smem_variant;  // 1: always use the shared-memory-activation variant (testing)
    cudaEvent_t ev_prep, ev_gate_up, ev_down;  // optional stage marks (null = none)
    // fused routing (decode_route_fusable): top-k, dispatch and the work lists run as one block
    // inside launch_decode_layer; the caller has run neither launch_router_topk nor launch_dispatch,
    // and expert_offsets / sorted_tok / slot_pos above are outputs as well
    int fused_route;
    const float* scores; const float* e_bias; int norm_topk; float routed_scale;
    int* ids; float* w_out; int* sorted_row;
    int xp_ready;            // 1: xp already holds the converted activations (logits launch did it)
};
int launch_decode_layer(const DecodeArgs& a, cudaStream_t s);
struct DecodeEpArgs {
    int H, I, Is, El;                   // El = experts resident on this GPU
    const void* gate_up_packed;
    const void* down_packed;
    const void* shared_gate_up_packed;
    const void* shared_down_packed;
    const int* recv_offsets;            // [El + 1] rows received per local expert (device)
    const __half* xbuf;                 // [recv_cap + n, H] fragment-order fp16: received rows, then this GPU's tokens
    int recv_cap, n;
    __half* hbuf;                       // [recv_cap + n, max(I, Is)]
    float* const* ydst;                 // [recv_cap + n] output row of every slot (fp32)
    int* segs;                          // decode_seg_bytes_raw(recv_cap, n, El)
    int* status;
    int sm_count;
};
int launch_decode_ep(const DecodeEpArgs& a, cudaStream_t s, int what = 3);   // what: 1 lists, 2 kernels, 3 both
int launch_combine_f32(const float* ybuf, const int* slot_pos, const float* topk_w, int n, int topk, int H, int P,
                       int has_shared, const float* residual, float* out, cudaStream_t s);
// bf16 rows -> fp16 rows in fragment order (natural = 0) or natural feature order (1)
int launch_xprep(const __nv_bfloat16* x, __half* xp, int64_t n, int H, int natural, cudaStream_t s);
int launch_xprep_f32(const float* x, __half* xp, int64_t n, int H, int natural, cudaStream_t s);
int launch_decode_dense(const void* packed, const __half* xf, int n, int K, int rows, float* y, int* segs,
                        const int* zero2, int* status, int sm_count, cudaStream_t s);
int launch_add_bias_rows(float* y, const float* bias, int64_t n, int64_t cols, cudaStream_t s);
// whether the single-block routing kernel covers this shape
inline bool decode_route_fusable(int n, int topk, int E) { return n <= 128 && E <= 256 && topk <= 32 && n * topk <= 4096; }

size_t prefill_tile_bytes(int n, int topk, int E);

struct PrefillArgs {
    const __nv_bfloat16* x;
    int n, topk, H, I, Is, E;
    int Id, Isd;    // as in DecodeArgs
    const void* gate_up_packed;
    const void* down_packed;
    const void* shared_gate_up_packed;
    const void* shared_down_packed;
    const int* expert_offsets;
    const int* sorted_tok;
    const int* slot_pos;
    const float* topk_w;
    int* tiles;     // token-tile list (prefill_tile_bytes), read by both GEMM kernels
    __half* xh;     // [n, H] fp16 activations in token order, natural feature order
    int xh_ready;   // 1: the router-logits launch already wrote xh
    __half* xs;     // [P + n, H] fp16 activations in expert order
    __half* hbuf;   // [P + n, max(I, Is)] fp16
    __half* ybuf;   // [P + n, H] fp16 per-slot output rows
    int* status;
    float* out;
    const float* residual;  // nullable: out = residual + layer (out may be the residual itself)
    int sm_count;
    cudaEvent_t ev_prep, ev_gate_up, ev_down;
};
int launch_prefill_layer(const PrefillArgs& a, cudaStream_t s);

// Expert-parallel pieces of the tcgen05 path (see comm.cu / ep.cu for the exchange).
struct PrefillEpArgs {
    const void* gate_up_packed;         // resident (local) experts
    const void* down_packed;
    const void* shared_gate_up_packed;
    const void* shared_down_packed;
    int H, I, Is, El;                   // El = experts resident on this GPU
    const int* recv_offsets;            // [El + 1] rows received per local expert (device)
    const __half* recv_x;               // [recv_cap, H] received activations (fp16)
    int recv_cap;
    __half* hbuf;                       // [recv_cap, I]
    __half* const* ydst;                // [recv_cap] where each received row's output goes
    int* tiles;                         // token-tile list over the received rows
    int e_begin, e_end;                 // resident experts this call covers (0, 0 = all El): the exchange can hand
                                        // the rows over in two waves, each with a tile list of its own
    int n;                              // this GPU's own tokens (shared expert)
    __half* xs_local;                   // [n, H] this GPU's tokens as fp16 in natural order, filled by the caller
    __half* hbuf_sh;                    // [n, Is]
    __half* y_shared;                   // [n, H]
    int* tiles_sh;                      // token-tile list of the shared expert over the local tokens
    int* status;
    int sm_count;
};
int launch_prefill_ep_shared(const PrefillEpArgs& a, cudaStream_t s);
int launch_prefill_ep_routed(const PrefillEpArgs& a, cudaStream_t s, int what = 3);   // what: 1 tile list, 2 kernels, 3 both
int launch_combine_h(const __half* ybuf, const int* slot_pos, const float* topk_w, int n, int topk, int H,
                     int P, int has_shared, const float* residual, float* out, cudaStream_t s);

}  // namespace gsb

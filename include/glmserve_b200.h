/*
 * glmserve_b200 - C ABI of the B200 (sm_100a) W4A16 MoE layer path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns an int
 * status (GSB_OK = 0) and never throws or aborts.  All data pointers are DEVICE pointers
 * unless a parameter says "host".  `stream` is a cudaStream_t passed as void* (NULL = the
 * legacy default stream, which is what the reference engine uses for every kernel).
 * Nothing here allocates device memory unless its comment says so: weights, activations
 * and scratch belong to the caller, as in the reference (src/model_gpu.cpp:578-645).
 *
 * Two families:
 *   1. "operator" entry points - the reference's own launch wrappers from
 *      cuda/kernels.cuh (namespace glmserve::cuda), same parameter lists and meaning;
 *      include/glmserve_cuda_shim.cuh re-creates those C++ names on top of them so that
 *      src/model_gpu.cpp of the reference compiles and links unchanged.
 *   2. "native" entry points - bf16 activations, fp16 scales, weights prepacked once into
 *      the tile-stream layout the sm_100a kernels read; one call runs the whole layer.
 */
#ifndef GLMSERVE_B200_H
#define GLMSERVE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GSB_API __attribute__((visibility("default")))

enum {
    GSB_OK = 0,
    GSB_ERR_INVALID_ARG = 1, /* null pointer, negative size, misaligned buffer, bad shape */
    GSB_ERR_UNSUPPORTED = 2, /* shape or format outside what the kernels implement */
    GSB_ERR_LAUNCH = 3,      /* cudaGetLastError() after the launch was not cudaSuccess */
    GSB_ERR_TIMEOUT = 4,     /* a bounded device-side wait gave up (status word set) */
    GSB_ERR_CUDA = 5,        /* another CUDA runtime call failed */
    GSB_ERR_WORKSPACE = 6,   /* caller scratch smaller than gsb_moe_workspace_bytes() */
    GSB_ERR_TOO_LARGE = 7    /* problem larger than a built-in fixed-size buffer */
};

/* Text for a status code (static storage). */
GSB_API const char* gsb_status_string(int status);
/* Library version and the architecture it was compiled for ("sm_100a"). */
GSB_API const char* gsb_build_info(void);

/* ------------------------------------------------------------------------------------
 * 1. Operator entry points (drop-in for cuda/kernels.cuh of the reference)
 * ---------------------------------------------------------------------------------- */

/* Replaces moe_router (cuda/kernels.cuh:243-245, cuda/moe_router.cu:17-79).
 * logits f32 [n,E]; e_bias f32 [E] or NULL; outputs topk_ids i32 [n,topk] in descending
 * order of (sigmoid(logit)+bias), ties to the smaller expert id, topk_weights f32 [n,topk]
 * = sigmoid scores, divided by their sum (in selection order) when norm_topk, times
 * routed_scale.  E <= 1024, topk <= 32, topk <= E.  The sigmoid is evaluated so that the
 * ids equal the CPU reference's (src/model_glm52.cpp:1113-1129) bit for bit. */
GSB_API int gsb_moe_router(const float* logits, const float* e_bias, int n, int E, int topk,
                           int norm_topk, float routed_scale, int* topk_ids,
                           float* topk_weights, void* stream);

/* Replaces moe_dispatch (cuda/kernels.cuh:249-250, cuda/moe_dispatch.cu:16-45): stable
 * counting sort of the flat slots i = t*topk + k by expert.  expert_offsets i32 [E+1],
 * sorted_token_ids / sorted_row i32 [n*topk].  Warp histograms + prefix scan; the order
 * inside an expert segment is increasing i (no atomics decide any position).
 * Ids outside [0,E) are a caller error; they are counted in no segment. */
GSB_API int gsb_moe_dispatch(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                             int* sorted_token_ids, int* sorted_row, void* stream);

/* The same dispatch with caller scratch (gsb_moe_dispatch_scratch_bytes bytes, 4-byte aligned):
 * above 8192 slots the work is spread over one block per 4096 slots (count, offsets, scatter
 * launches) instead of one block for everything - the reference's signature has no scratch
 * argument, so gsb_moe_dispatch cannot.  Same permutation, bit for bit.  scratch may be NULL. */
GSB_API size_t gsb_moe_dispatch_scratch_bytes(int n, int topk, int E);
GSB_API int gsb_moe_dispatch_ws(const int* topk_ids, int n, int topk, int E, int* expert_offsets,
                                int* sorted_token_ids, int* sorted_row, void* scratch,
                                size_t scratch_bytes, void* stream);

/* Replaces moe_expert_ffn_w4a16 (cuda/kernels.cuh:259-268, cuda/moe_expert.cu:132-244).
 * x f32 [n,hidden]; gate_q/up_q u8 [E,moe_inter,hidden/2], gate_sc/up_sc f32
 * [E,moe_inter,hidden/group]; down_q u8 [E,hidden,moe_inter/2], down_sc f32
 * [E,hidden,moe_inter/group]; out f32 [n,hidden] is OVERWRITTEN with
 * sum_k w[t,k] * down(silu(gate x) * up x), slots added in order k = 0..topk-1.
 * hidden, moe_inter and group must be multiples of 8, hidden and moe_inter multiples of group. */
GSB_API int gsb_moe_expert_ffn_w4a16(const float* x, const int* topk_ids,
                                     const float* topk_weights, const uint8_t* gate_q,
                                     const float* gate_sc, const uint8_t* up_q,
                                     const float* up_sc, const uint8_t* down_q,
                                     const float* down_sc, int n, int topk, int hidden,
                                     int moe_inter, int E, int group_size, float* out,
                                     void* stream);

/* Replaces moe_expert_ffn (cuda/kernels.cuh:254-257, cuda/moe_expert.cu:32-130): the same
 * with fp32 weights gate_w/up_w [E,moe_inter,hidden], down_w [E,hidden,moe_inter]. */
GSB_API int gsb_moe_expert_ffn(const float* x, const int* topk_ids, const float* topk_weights,
                               const float* gate_w, const float* up_w, const float* down_w,
                               int n, int topk, int hidden, int moe_inter, int E, float* out,
                               void* stream);

/* Replaces gemm_w4a16 (cuda/kernels.cuh:48-52, cuda/int4_gemm.cu:15-48):
 * y[n,out] = x[n,in] W[out,in]^T (+ bias), W = (nibble-8)*scales[out, in/group]. */
GSB_API int gsb_gemm_w4a16(const float* x, const uint8_t* qW, const float* scales,
                           const float* bias, float* y, int64_t n, int64_t in, int64_t out,
                           int64_t group_size, void* stream);

/* A fast path behind the two signatures above, for a caller that cannot change its call sites (the
 * reference's src/model_gpu.cpp:1460-1494, :441-445 passes the raw resident layout and fp32 activations on
 * every call).  After gsb_operator_cache_enable(max_weight_bytes) the first call that sees a set of weight
 * pointers repacks them ONCE into the tile stream - keyed on the pointers and shapes, so the weights must stay
 * where they are and unchanged - and that call and every later one runs the split-K / tcgen05 kernels
 * (group 128, hidden and moe_inter multiples of 512 for the expert FFN; group 128, in % 512 == 0,
 * out % 128 == 0, n <= 512 for gemm_w4a16); anything else, or a cache that is full, takes the direct-layout
 * kernels as before.  Activations are rounded from fp32 to fp16 for the tensor cores (the direct kernels
 * keep fp32).  This is the one place where the library allocates device memory by itself: packed copies
 * (the same size as the int4 originals) and a scratch area that grows to the largest batch seen.  0 switches
 * it off and frees everything (device-wide synchronise).  Off by default.  One device, host calls
 * serialised by a lock. */
GSB_API int gsb_operator_cache_enable(size_t max_weight_bytes);
GSB_API size_t gsb_operator_cache_bytes(void);

/* Replace silu_mul / add_inplace / rmsnorm (cuda/kernels.cuh:18-19, :282-283), the glue the
 * reference runs around the shared expert and the residual (src/model_gpu.cpp:1430,
 * :1486-1502).  rmsnorm sums squares in double like the CPU reference. */
GSB_API int gsb_silu_mul(const float* g, const float* u, float* out, int64_t n, void* stream);
GSB_API int gsb_add_inplace(float* y, const float* x, int64_t n, void* stream);
GSB_API int gsb_rmsnorm(const float* x, const float* w, float* out, int64_t n, int64_t d,
                        float eps, void* stream);

/* The GGML-block-quant ("qgemm") family of cuda/kernels.cuh:59-136.  The entry points and
 * their scratch contract exist so the reference's caller links; the GGML codecs are a
 * different weight format and every qtype reports GSB_ERR_UNSUPPORTED, except
 * gsb_quantize_act_q8 (cuda/qgemm.cu:569-587: per-32 absmax int8 activations), which is
 * format independent and implemented. */
GSB_API int gsb_qtype_has_i8(uint32_t qtype);
GSB_API int gsb_quantize_act_q8(const float* x, int64_t n, int64_t in, int8_t* xq, float* xs,
                                void* stream);
GSB_API int gsb_gemm_q(uint32_t qtype, const float* x, const uint8_t* qW, const float* bias,
                       float* y, int64_t n, int64_t in, int64_t out, int64_t row_bytes,
                       void* stream);
GSB_API int gsb_gemm_q_i8(uint32_t qtype, const int8_t* xq, const float* xs, const uint8_t* qW,
                          const float* bias, float* y, int64_t n, int64_t in, int64_t out,
                          int64_t row_bytes, void* stream);
GSB_API int gsb_moe_expert_ffn_q(uint32_t gate_type, uint32_t up_type, uint32_t down_type,
                                 const float* x, const int* topk_ids, const float* topk_w,
                                 const uint8_t* gate_q, const uint8_t* up_q,
                                 const uint8_t* down_q, int n, int topk, int hidden,
                                 int moe_inter, int E, int64_t gate_row_bytes,
                                 int64_t up_row_bytes, int64_t down_row_bytes, float* h_act,
                                 float* dpart, float* out, int* dispatch, float* gu_part,
                                 void* stream);
GSB_API int gsb_moe_expert_ffn_q_i8(uint32_t gate_type, uint32_t up_type, uint32_t down_type,
                                    const int8_t* xq, const float* xs, const int* topk_ids,
                                    const float* topk_w, const uint8_t* gate_q,
                                    const uint8_t* up_q, const uint8_t* down_q, int n,
                                    int topk, int hidden, int moe_inter, int E,
                                    int64_t gate_row_bytes, int64_t up_row_bytes,
                                    int64_t down_row_bytes, float* h_act, int8_t* hq,
                                    float* hs, float* dpart, float* out, int* dispatch,
                                    float* gu_part, void* stream);

/* ------------------------------------------------------------------------------------
 * 2. Native entry points
 * ---------------------------------------------------------------------------------- */

/* Size in bytes of one prepacked matrix set: `experts` matrices of [rows, cols] int4 with
 * one fp16 scale per 128 columns.  rows % 32 == 0 and cols % 512 == 0 are required
 * (returns 0 otherwise). */
GSB_API size_t gsb_prepack_bytes(int experts, int rows, int cols);

/* One-time repack of resident int4 weights (the layout src/model_gpu.cpp:948-1000 uploads)
 * into the tile stream the sm_100a kernels read.  Call where the reference concatenates the
 * experts at upload time.  scales_f32 != 0: scales are float32 (reference layout), else
 * fp16.  group must be 128.
 *   gate/up: matrices [experts, inter, hidden]; unit u holds gate rows 16u..16u+15 then up
 *            rows 16u..16u+15, so SwiGLU needs no second pass.  Output size
 *            gsb_prepack_bytes(experts, 2*inter, hidden).
 *   down:    matrices [experts, hidden, inter]; unit u holds rows 32u..32u+31.  Output size
 *            gsb_prepack_bytes(experts, hidden, inter). */
GSB_API int gsb_prepack_gate_up(const uint8_t* gate_q, const void* gate_sc, const uint8_t* up_q,
                                const void* up_sc, int scales_f32, int experts, int inter,
                                int hidden, int group, void* out, void* stream);
GSB_API int gsb_prepack_down(const uint8_t* down_q, const void* down_sc, int scales_f32,
                             int experts, int hidden, int inter, int group, void* out,
                             void* stream);

/* Static description of one MoE layer.  All pointers are device pointers owned by the
 * caller and must outlive the layer object.  Counterpart of the expert fields of DLayer
 * (src/model_gpu.cpp:499-524). */
typedef struct gsb_moe_config {
    int hidden;              /* H */
    int n_experts;           /* E routed experts resident on this GPU */
    int topk;                /* k */
    int moe_inter;           /* I (per-expert intermediate, already /tp under TP); tile kernels: multiple of 64 */
    int shared_inter;        /* Is, 0 = no shared expert */
    int group;               /* int4 group size along the input dim */
    int norm_topk;           /* normalise the top-k weights */
    float routed_scale;      /* routed_scaling_factor */
    const void* router_w;    /* bf16 [E_global, H] */
    const float* e_bias;     /* f32 [E_global] or NULL */
    /* raw resident layout (any shape the quantiser allows); scales fp16 */
    const uint8_t* gate_q;   /* [E, I, H/2] */
    const void* gate_sc;     /* fp16 [E, I, H/group] */
    const uint8_t* up_q;
    const void* up_sc;
    const uint8_t* down_q;   /* [E, H, I/2] */
    const void* down_sc;     /* fp16 [E, H, I/group] */
    const uint8_t* sg_q;     /* shared expert [Is, H/2] etc., NULL when shared_inter == 0 */
    const void* sg_sc;
    const uint8_t* su_q;
    const void* su_sc;
    const uint8_t* sd_q;     /* [H, Is/2] */
    const void* sd_sc;
    /* prepacked tile streams (gsb_prepack_*), or NULL: then only the direct-layout kernels
     * can run and shapes the fast kernels need report GSB_ERR_UNSUPPORTED in "fast" mode */
    const void* gate_up_packed;
    const void* down_packed;
    const void* shared_gate_up_packed;
    const void* shared_down_packed;
    /* expert parallelism (0 or 1 = off): n_experts stays the GLOBAL expert count E, the weight
     * pointers above hold the E / ep_size experts [ep_rank*E/ep_size, (ep_rank+1)*E/ep_size)
     * resident on this GPU; router_w / e_bias cover all E.  Such a layer runs through
     * gsb_moe_layer_forward_ep only. */
    int ep_size;
    int ep_rank;
    /* 1 = no router: every token goes to experts 0..topk-1 in that order with weight 1.0
     * (router_w may be NULL, norm_topk / routed_scale / e_bias are ignored).  A dense SwiGLU MLP
     * whose intermediate dim is cut into E = topk slices is exactly such a layer: the first
     * dense layers of the model (src/model_gpu.cpp:1432-1445) run through the same kernels. */
    int fixed_routing;
    /* Input dim of the packed down matrices when it is larger than moe_inter / shared_inter (0 = the same):
     * a tensor-parallel shard whose intermediate slice is narrower than the 512 columns a chunk of the tile
     * stream covers (e.g. 2048 / 8 = 256) packs its down matrices with zero weights (nibble 8) in the columns
     * beyond moe_inter; gate/up stay unpadded.  Multiples of 512. */
    int down_inter;
    int shared_down_inter;
} gsb_moe_config;

typedef struct gsb_moe_layer gsb_moe_layer; /* opaque, host memory only */

/* Creates the host-side plan (validates shapes, picks kernels by shape; allocates host
 * memory only).  No counterpart in the reference: its per-call wrappers re-derive
 * everything from arguments; a plan keeps the per-call host work to a few launches. */
GSB_API int gsb_moe_layer_create(const gsb_moe_config* cfg, gsb_moe_layer** out);
GSB_API void gsb_moe_layer_destroy(gsb_moe_layer* layer);

/* Scratch the caller must provide for n tokens (256-byte aligned device memory);
 * counterpart of Scratch::ensure (src/model_gpu.cpp:578-645). */
GSB_API size_t gsb_moe_workspace_bytes(const gsb_moe_layer* layer, int n_tokens);

/* Path selection for gsb_moe_layer_forward. */
enum {
    GSB_PATH_AUTO = 0,    /* by shape: direct-layout kernels for shapes the tile kernels do
                             not cover; else the split-K kernels below an average of 32 rows per
                             routed expert (n * topk < 32 * n_experts) and the tcgen05 grouped
                             GEMM from there on */
    GSB_PATH_DIRECT = 1,  /* direct-layout SIMT kernels (any shape) */
    GSB_PATH_DECODE = 2,  /* bandwidth-bound split-K tile-stream kernels */
    GSB_PATH_PREFILL = 3, /* tcgen05 grouped GEMM */
    GSB_PATH_DECODE_SMEM = 4 /* decode kernels, forcing the variant that keeps activations in shared
                                memory (the one used when an input dim is not a multiple of 2048) */
};

/* The whole layer, replacing the MoE branch of run_layer_step (src/model_gpu.cpp:1446-1495):
 * router GEMM -> router -> dispatch -> grouped gate/up + SwiGLU -> down -> shared expert ->
 * deterministic combine (slots in order, shared last).  x bf16 [n,H]; out f32 [n,H]
 * overwritten.  Optional outputs (NULL to skip): logits_out f32 [n,E], ids_out i32
 * [n,topk], weights_out f32 [n,topk].  Asynchronous on `stream`; no host sync. */
GSB_API int gsb_moe_layer_forward(gsb_moe_layer* layer, const void* x_bf16, int n, float* out,
                                  void* workspace, size_t workspace_bytes, int path,
                                  float* logits_out, int* ids_out, float* weights_out,
                                  void* stream);

/* Pre-norm + layer + residual, the MLP half of run_layer_step
 * (src/model_gpu.cpp:1430-1502): hidden f32 [n,H] <- hidden + moe(rmsnorm(hidden) as bf16).
 * norm_w f32 [H].  Scratch: gsb_moe_workspace_bytes() covers it. */
GSB_API int gsb_moe_block_layer_forward(gsb_moe_layer* layer, float* hidden,
                                        const float* norm_w, float eps, int n, void* workspace,
                                        size_t workspace_bytes, int path, int* ids_out,
                                        void* stream);

/* Stage entry points of the native path (what the reference's StageProf marks
 * "moe.router", "moe.experts", "moe.shared" separate; src/model_gpu.cpp:1451-1493). */
GSB_API int gsb_router_logits(const void* x_bf16, const void* router_w_bf16, int n, int hidden,
                              int E, float* logits, void* stream);

/* Stage profiler, the counterpart of the reference's StageProf (src/model_gpu.cpp:328-388):
 * cudaEventRecord at stage marks on the forward's stream.  Stages, in order:
 * "moe.router" (logits GEMM + top-k), "moe.dispatch" (permutation + activation staging),
 * "moe.gate_up" (gate/up GEMM + SwiGLU, routed and shared), "moe.down", "moe.combine".
 * enable() creates CUDA events for up to max_forwards forwards (0 = off; host resources
 * only); read() - after the caller synchronised - averages the stage times in ms over the
 * forwards recorded since the last read and starts over. */
#define GSB_N_STAGES 5
GSB_API int gsb_moe_layer_profile_enable(gsb_moe_layer* layer, int max_forwards);
GSB_API int gsb_moe_layer_profile_read(gsb_moe_layer* layer, float* stage_ms, int* n_forwards);

/* Diagnostic of the tcgen05 path: while device_buffer (2 x 1024 x 16 int64, device memory) is set, every
 * CTA of the gate/up kernel (first 1024 x 16) and of the down kernel (second) stores the SM cycles its
 * roles spent in bounded waits during the last forward: [0] producer loop total, [1] producer waiting
 * for a free int4 stage, [2] for a free activation stage, [3] MMA thread waiting for a free accumulator,
 * [4] for unpacked weights, [5] for an activation tile, [6] unpack warps waiting for int4 data, [7] for a
 * free slot of the weight ring, [8] MMA thread issuing tcgen05.mma / commit, [9] MMA thread total.  NULL switches it off (the default).  Host call, not thread safe. */
GSB_API int gsb_prefill_wait_profile(long long* device_buffer);

/* Routing without any allocation: x bf16 [n,hidden] and the bf16 router weight [E,hidden]
 * in, topk_ids i32 [n,topk] and topk_weights f32 [n,topk] out - the same result as
 * gsb_router_logits followed by gsb_moe_router, but the [n,E] logits in between are kept in
 * a fixed 256 KiB array inside the library instead of in a buffer the caller supplies.
 * This entry point has no counterpart in the reference.
 * It is meant for callers that cannot obtain device memory at the point of the call: an
 * engine that handed its whole memory budget to a weight/KV arena at start-up and has no
 * allocator left for per-call scratch, a plug-in running inside a host that forbids
 * cudaMalloc on its threads, or a latency-critical loop where an allocation's implicit
 * device synchronisation is not acceptable.  It calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 * Limits and rules:
 *   - n * E must not exceed gsb_moe_route_static_max_floats() (65536); larger problems
 *     return GSB_ERR_TOO_LARGE and launch nothing.  Other shape limits as gsb_moe_router.
 *   - every GPU that loads the library holds the 256 KiB array until the process exits.
 *   - the first call on each device looks up the array's device address (a host-side
 *     runtime query, done once per device with that device current); make that first call
 *     before starting any stream capture.
 *   - all calls on a device share the one array: the call overwrites every element it later
 *     reads, so stale contents are harmless, but two calls whose kernels can overlap on the
 *     GPU (different streams, no ordering between them) race on it.  Serialise them.
 *   - `stream` must belong to the device that is current at the call (the address looked up is that
 *     device's), and the cached address does not survive cudaDeviceReset or a re-created primary
 *     context: do not reset the device between calls. */
GSB_API int gsb_moe_route_static(const void* x_bf16, const void* router_w_bf16,
                                 const float* e_bias, int n, int hidden, int E, int topk,
                                 int norm_topk, float routed_scale, int* topk_ids,
                                 float* topk_weights, void* stream);
GSB_API int gsb_moe_route_static_max_floats(void);

/* ------------------------------------------------------------------------------------
 * 3. One 8-GPU box: peer memory over NVLink (one process per GPU)
 * ---------------------------------------------------------------------------------- */

/* A symmetric heap per rank, mapped into every peer with CUDA IPC; flags with sequence numbers
 * order the traffic; every device-side wait is bounded and reports GSB_ERR_TIMEOUT through
 * gsb_comm_status instead of hanging.  Replaces custom_ar_create / custom_ar_open /
 * custom_ar_run / custom_ar_destroy (cuda/custom_ar.h:26-43) and Communicator::all_reduce_sum
 * (include/nccl_comm.hpp:50-59, src/nccl_comm.cpp:283-350) for the MoE path.
 *   create: allocates (cudaMalloc) the local heap of heap_bytes (+ 1 MiB control area) and
 *           writes a gsb_comm_handle_bytes()-byte handle for the other ranks.
 *   open:   handles = world handles in rank order (entry [rank] ignored); all-or-none, like the
 *           reference: on failure destroy the communicator on EVERY rank.
 * Rules for every gsb_comm_* collective and for gsb_moe_layer_forward_ep: all ranks issue the same
 * calls in the same order, each rank on ONE stream of its own (staging areas and sequence numbers are
 * reused from call to call), on the device that was current at create; no device reset between calls;
 * nothing else may keep the GPUs so busy that a rank's kernel cannot start while its peers wait for it
 * (the waits are bounded, so that case ends in GSB_ERR_TIMEOUT, not in a hang). */
typedef struct gsb_comm gsb_comm;
GSB_API int gsb_comm_handle_bytes(void);
GSB_API int gsb_comm_create(int rank, int world, size_t heap_bytes, void* out_handle, gsb_comm** out);
GSB_API int gsb_comm_open(gsb_comm* comm, const void* handles);
/* Instead of open: maps every peer slot onto this rank's OWN heap, so a single process can exercise the
 * collectives' code paths without other GPUs - in particular the bounded waits: nothing ever posts the
 * peers' flags, so every wait runs out and reports GSB_ERR_TIMEOUT (tests). */
GSB_API int gsb_comm_open_loopback(gsb_comm* comm);
/* Budget of every device-side wait of this communicator in SM clock cycles (0 = the default, about two
 * seconds).  The reference's all-reduce spins without limit (cuda/custom_ar.cu:77-79). */
GSB_API int gsb_comm_set_wait_cycles(gsb_comm* comm, long long cycles);
GSB_API void gsb_comm_destroy(gsb_comm* comm);
GSB_API void* gsb_comm_heap(gsb_comm* comm);
GSB_API size_t gsb_comm_heap_bytes(gsb_comm* comm);
GSB_API int gsb_comm_rank(gsb_comm* comm);
GSB_API int gsb_comm_world(gsb_comm* comm);
/* After a stream synchronise: GSB_OK, GSB_ERR_TIMEOUT (a peer never posted) or
 * GSB_ERR_TOO_LARGE (more rows received than the receive capacity); clears the word. */
GSB_API int gsb_comm_status(gsb_comm* comm);
/* Device-side barrier over all ranks on `stream` (signal + bounded wait). */
GSB_API int gsb_comm_barrier(gsb_comm* comm, void* stream);

/* In-place sum of `count` floats over all ranks (count % 4 == 0, data 16-byte aligned, device
 * memory anywhere on this GPU).  Every element is summed in rank order 0..world-1, so the bits
 * do not depend on count, algorithm or grid: reducing rows one by one or as one batch gives the same
 * result (what all_reduce_sum_rows guarantees in the reference).  Both forms PUSH over NVLink (a rank
 * stores into its own slot on the peers, then a per-block flag; sums read local memory only): small
 * messages one-shot (every rank receives every vector), larger ones reduce-scatter + all-gather.
 * gsb_comm_allreduce_reserve(max_count) must be called once (same value on every rank): it
 * returns the bytes at the START of the heap that the all-reduce staging occupies. */
GSB_API size_t gsb_comm_allreduce_reserve(gsb_comm* comm, int64_t max_count);
/* The same byte count without a communicator, for sizing the heap before gsb_comm_create. */
GSB_API size_t gsb_comm_allreduce_reserve_bytes(int world, int64_t max_count);
GSB_API int gsb_comm_allreduce_sum(gsb_comm* comm, float* data, int64_t count, void* stream);
/* Algorithm switch: messages with count * world <= total_floats (and world * count <= 2 * max_count, the
 * room the staging has) take the one-shot form, larger ones reduce-scatter + all-gather.  0 restores the
 * default (2^20 * world / (world - 1): one-shot while a rank sends at most about 4 MB).  Same value on every rank; both orders of summation are rank 0..world-1 per element, so
 * the result does not depend on the choice. */
GSB_API int gsb_comm_allreduce_one_shot_limit(gsb_comm* comm, int64_t total_floats);
/* Decode-sized messages (count <= floats, at most 65536 = the default; 0 restores it, 1 switches the form off)
 * take a third form: every 16-byte word carries two floats and the call's sequence number twice, so the
 * receiver needs no flag round - one NVLink traversal.  Same rank-order sums, same bits.  Same value on every
 * rank. */
GSB_API int gsb_comm_allreduce_ll_limit(gsb_comm* comm, int64_t floats);
/* n back-to-back in-place sums from one host call (data ends as the n-fold sum): what a benchmark uses to see
 * the collective's device time instead of the host's per-call cost. */
GSB_API int gsb_comm_allreduce_sum_n(gsb_comm* comm, float* data, int64_t count, int n, void* stream);

/* Expert-parallel forward of one layer (cfg.ep_size = world): router and dispatch on this GPU's
 * n tokens, per-expert counts and buffer layouts exchanged, rows pushed over NVLink into the owners'
 * receive buffers (on a side stream, while the shared expert runs on the local tokens), grouped GEMMs
 * over the resident experts whose down-projection epilogue stores each output row straight to the
 * token's home GPU, then the deterministic combine.  No counterpart in the reference (it has no expert
 * parallelism).  path: GSB_PATH_PREFILL = tcgen05 kernels (results equal the single-GPU tcgen05 layer's
 * bit for bit), GSB_PATH_DECODE = split-K kernels (equal the single-GPU split-K layer's bit for bit),
 * GSB_PATH_AUTO = by recv_cap (split-K below 64 rows of capacity per resident expert).  All ranks must
 * pass the same path, or AUTO with the same recv_cap.
 *   heap_offset: byte offset into the comm heap (multiple of 1 KiB, after the all-reduce reserve) of
 *                gsb_moe_ep_heap_bytes() bytes for the receive and return buffers.  Ranks may use
 *                different offsets, n and recv_cap: each rank posts its own layout to its peers.
 *   recv_cap:    rows this GPU can receive; the sum of all ranks' n * topk can never overflow.  More
 *                rows than that: the excess is dropped, nothing is written out of bounds, and
 *                gsb_comm_status reports GSB_ERR_TOO_LARGE. */
GSB_API size_t gsb_moe_ep_heap_bytes(const gsb_moe_layer* layer, int n_tokens, int recv_cap);
GSB_API size_t gsb_moe_ep_workspace_bytes(const gsb_moe_layer* layer, int n_tokens, int recv_cap);
GSB_API int gsb_moe_layer_forward_ep(gsb_moe_layer* layer, gsb_comm* comm, const void* x_bf16, int n,
                                     float* out, void* workspace, size_t workspace_bytes,
                                     size_t heap_offset, int recv_cap, int path, int* ids_out, void* stream);
/* The same with the layer's pre-norm and residual add (gsb_moe_block_layer_forward over the box):
 * hidden f32 [n,H] <- hidden + moe(rmsnorm(hidden) as bf16); the norm rides the router-logits launch, the
 * residual the combine pass.  The result equals gsb_moe_block_layer_forward of the all-expert layer on one
 * GPU bit for bit (same kernel family). */
GSB_API int gsb_moe_block_layer_forward_ep(gsb_moe_layer* layer, gsb_comm* comm, float* hidden,
                                           const float* norm_w, float eps, int n, void* workspace,
                                           size_t workspace_bytes, size_t heap_offset, int recv_cap, int path,
                                           int* ids_out, void* stream);

/* Reads (and clears) the device status word of the last forward on this layer after the
 * caller synchronised the stream: GSB_OK, or the recorded code (GSB_ERR_TIMEOUT when a bounded
 * wait inside a kernel gave up).  Host call. */
GSB_API int gsb_moe_layer_status(gsb_moe_layer* layer, void* workspace);

#ifdef __cplusplus
}
#endif
#endif /* GLMSERVE_B200_H */

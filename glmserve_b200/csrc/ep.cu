// Expert-parallel forward of one MoE layer over the GPUs of one box (host orchestration).
// The exchange kernels live in comm.cu, the GEMMs in prefill_w4.cu (tcgen05) and decode_w4.cu (split-K).
#include "internal.cuh"

using namespace gsb;

namespace {

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// This rank's part of the symmetric heap.  Peers never compute an address in it from their own
// arguments: the offsets are posted with the expert counts (comm.cu).
//   xbuf  (recv_cap + n) fp16 rows: rows received from all ranks, then (split-K path) this GPU's own tokens
//   ybuf  (n * topk + n) rows of per-slot outputs, written by the experts' owners: fp16 (tcgen05 path) or
//         fp32 (split-K path); sized for fp32
struct EpHeap { size_t xbuf, ybuf, total; };
EpHeap ep_heap(const gsb_moe_config& c, int n, int recv_cap) {
    EpHeap h{};
    size_t off = 0;
    h.xbuf = off; off = align_up(off + ((size_t)recv_cap + n) * c.hidden * sizeof(__half), 1024);
    h.ybuf = off; off = align_up(off + ((size_t)n * c.topk + n) * c.hidden * sizeof(float), 1024);
    h.total = off;
    return h;
}

struct EpWs {
    int* status; float* logits; float* scores; int* ids; float* w; int* expert_offsets; int* sorted_tok;
    int* sorted_row; int* slot_pos; int* sorted_expert; int* disp_scratch; int* recv_offsets; int* send_base; void** ydst;
    int* plan; int* tiles; int* tiles2; int* tiles_sh; int* segs;
    __half* hbuf; __half* xs_local; __half* hbuf_sh;
    size_t total;
};
EpWs ep_carve(const gsb_moe_config& c, int n, int recv_cap, void* base) {
    EpWs ws{};
    const size_t P = (size_t)n * c.topk;
    const int El = c.n_experts / (c.ep_size > 0 ? c.ep_size : 1);
    const size_t imax = (size_t)(c.moe_inter > c.shared_inter ? c.moe_inter : c.shared_inter);
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off = align_up(off + bytes, 256);
        return base ? reinterpret_cast<char*>(base) + o : nullptr;
    };
    ws.status = reinterpret_cast<int*>(take(64 * sizeof(int)));
    ws.logits = reinterpret_cast<float*>(take((size_t)n * c.n_experts * sizeof(float)));
    ws.scores = reinterpret_cast<float*>(take((size_t)n * c.n_experts * sizeof(float)));
    ws.ids = reinterpret_cast<int*>(take(P * sizeof(int)));
    ws.w = reinterpret_cast<float*>(take(P * sizeof(float)));
    ws.expert_offsets = reinterpret_cast<int*>(take((size_t)(c.n_experts + 1) * sizeof(int)));
    ws.sorted_tok = reinterpret_cast<int*>(take(P * sizeof(int)));
    ws.sorted_row = reinterpret_cast<int*>(take(P * sizeof(int)));
    ws.slot_pos = reinterpret_cast<int*>(take(P * sizeof(int)));
    ws.sorted_expert = reinterpret_cast<int*>(take(P * sizeof(int)));
    ws.disp_scratch = reinterpret_cast<int*>(take(dispatch_scratch_bytes(n, c.topk, c.n_experts)));
    ws.recv_offsets = reinterpret_cast<int*>(take((size_t)(El + 1) * sizeof(int)));
    ws.send_base = reinterpret_cast<int*>(take((size_t)c.n_experts * sizeof(int)));
    ws.ydst = reinterpret_cast<void**>(take(((size_t)recv_cap + n) * sizeof(void*)));
    ws.plan = reinterpret_cast<int*>(take((4 + 4 * kMaxWorld) * sizeof(int)));
    ws.tiles = reinterpret_cast<int*>(take(prefill_tile_bytes(recv_cap / (c.topk > 0 ? c.topk : 1) + 1, c.topk, El)));
    ws.tiles2 = reinterpret_cast<int*>(take(prefill_tile_bytes(recv_cap / (c.topk > 0 ? c.topk : 1) + 1, c.topk, El)));
    ws.tiles_sh = reinterpret_cast<int*>(take(prefill_tile_bytes(n, 1, 1)));
    ws.segs = reinterpret_cast<int*>(take(decode_seg_bytes_raw((size_t)recv_cap, (size_t)n, El)));
    ws.hbuf = reinterpret_cast<__half*>(take(((size_t)recv_cap + n) * imax * sizeof(__half)));
    ws.xs_local = reinterpret_cast<__half*>(take((size_t)n * c.hidden * sizeof(__half)));
    ws.hbuf_sh = reinterpret_cast<__half*>(take((size_t)n * (c.shared_inter > 0 ? c.shared_inter : 1) * sizeof(__half)));
    ws.total = off;
    return ws;
}

// Output rows of the shared expert's slots (split-K path): this GPU's own row buffer.
__global__ void ep_shared_dst_kernel(void** ydst, float* y_shared, int n, int H) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) ydst[t] = y_shared + (size_t)t * H;
}

// Side stream and events of the expert-parallel forward (host resources, created on first use).
int ep_streams(gsb_moe_layer* L) {
    if (L->ep_side) return GSB_OK;
    if (cudaStreamCreateWithFlags(&L->ep_side, cudaStreamNonBlocking) != cudaSuccess) return GSB_ERR_CUDA;
    if (cudaEventCreateWithFlags(&L->ep_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&L->ep_join, cudaEventDisableTiming) != cudaSuccess)
        return GSB_ERR_CUDA;
    return GSB_OK;
}

}  // namespace

extern "C" {

size_t gsb_moe_ep_heap_bytes(const gsb_moe_layer* layer, int n_tokens, int recv_cap) {
    if (!layer || n_tokens < 0 || recv_cap < 0) return 0;
    return ep_heap(layer->cfg, n_tokens, recv_cap).total;
}

size_t gsb_moe_ep_workspace_bytes(const gsb_moe_layer* layer, int n_tokens, int recv_cap) {
    if (!layer || n_tokens < 0 || recv_cap < 0) return 0;
    return ep_carve(layer->cfg, n_tokens, recv_cap, nullptr).total;
}

}  // extern "C"

namespace {
// x (bf16 rows) or, when `hidden` is given, bf16(rmsnorm(hidden, norm_w, eps)) computed inside the
// router-logits launch; `residual` (nullable) rides the combine pass.
int forward_ep_impl(gsb_moe_layer* layer, gsb_comm* comm, const void* x_bf16, const float* hidden, const float* norm_w,
                    float eps, int n, float* out, const float* residual, void* workspace, size_t workspace_bytes,
                    size_t heap_offset, int recv_cap, int path, int* ids_out, void* stream) {
    if (!layer || !comm || n < 0 || recv_cap <= 0 || recv_cap >= (1 << 27)) return GSB_ERR_INVALID_ARG;
    const gsb_moe_config& c = layer->cfg;
    if (c.ep_size != comm->world || c.ep_rank != comm->rank || c.ep_size < 1) return GSB_ERR_INVALID_ARG;
    if (c.n_experts % c.ep_size || !layer->tiles_ok) return GSB_ERR_UNSUPPORTED;
    if (n > 0 && ((!x_bf16 && !hidden) || !out)) return GSB_ERR_INVALID_ARG;
    if (hidden && !norm_w) return GSB_ERR_INVALID_ARG;
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) || (heap_offset & 1023)) return GSB_ERR_INVALID_ARG;
    if (path != GSB_PATH_AUTO && path != GSB_PATH_DECODE && path != GSB_PATH_PREFILL) return GSB_ERR_INVALID_ARG;
    EpWs ws = ep_carve(c, n, recv_cap, workspace);
    if (workspace_bytes < ws.total) return GSB_ERR_WORKSPACE;
    const EpHeap hp = ep_heap(c, n, recv_cap);
    if (heap_offset + hp.total > comm->heap_bytes) return GSB_ERR_WORKSPACE;
    int st = ep_streams(layer);
    if (st) return st;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(x_bf16);
    const int E = c.n_experts, El = E / c.ep_size, P = n * c.topk;
    // Every rank must take the same path (the row formats differ), so AUTO decides on recv_cap, which the
    // ranks size alike, not on this rank's n: the split-K kernels below a capacity of 64 rows per resident
    // expert (an average of at most 32 at the usual two-fold head-room), the tcgen05 kernels from there on.
    if (path == GSB_PATH_AUTO) path = (int64_t)recv_cap >= 64LL * El ? GSB_PATH_PREFILL : GSB_PATH_DECODE;
    const bool decode = path == GSB_PATH_DECODE;
    uint8_t* heap = comm->local + kCtrlBytes + heap_offset;
    __half* xbuf = reinterpret_cast<__half*>(heap + hp.xbuf);
    void* ybuf = heap + hp.ybuf;

    __half* xh_local = decode ? xbuf + (size_t)recv_cap * c.hidden : ws.xs_local;
    cudaEvent_t* ev = nullptr;
    if (layer->prof_ev && layer->prof_used < layer->prof_sets)
        ev = layer->prof_ev + (size_t)(layer->prof_used++) * (GSB_N_STAGES + 1);
    auto mark = [&](int i) { if (ev) cudaEventRecord(ev[i], s); };
    mark(0);
    // decode-sized batches: top-k, dispatch and the posting of the counts ride one launch (inside comm_ep_plan)
    const bool fused_route = comm_ep_route_fusable(n, E);
    if (!fused_route && cudaMemsetAsync(ws.status, 0, 16, s) != cudaSuccess) return GSB_ERR_CUDA;
    if (n > 0) {
        // the logits launch leaves this rank's tokens behind as fp16 rows in the order the receiving kernels read
        // (fragment order behind the receive buffer for the split-K path, natural order for the tcgen05 path):
        // the push copies them as they lie, and the shared expert reads the same rows
        st = launch_router_logits(x, reinterpret_cast<const __nv_bfloat16*>(c.router_w), n, c.hidden, E, ws.logits, ws.scores, s,
                                  xh_local, decode ? 0 : 1, hidden, norm_w, eps);
        if (st) return st;
        if (!fused_route) {
            st = launch_router_topk(ws.scores, c.e_bias, n, E, c.topk, c.norm_topk, c.routed_scale, ws.ids, ws.w, s, true);
            if (st) return st;
        }
    }
    if (!fused_route) {
        st = launch_dispatch(ws.ids, n, c.topk, E, ws.expert_offsets, ws.sorted_tok, ws.sorted_row, ws.slot_pos, s,
                             ws.disp_scratch);
        if (st) return st;
    }
    // counts -> plan on the caller's stream; the push of this rank's rows and its signal on the side stream,
    // so that the shared expert (local tokens only) runs while rows travel in BOTH directions
    EpExchange ex{};
    ex.xh = xh_local; ex.expert_offsets = ws.expert_offsets; ex.sorted_tok = ws.sorted_tok; ex.P = P; ex.E = E; ex.H = c.hidden;
    ex.sorted_expert = ws.sorted_expert; ex.recv_offsets = ws.recv_offsets; ex.send_base = ws.send_base; ex.ydst = ws.ydst;
    ex.plan = ws.plan; ex.recv_off = heap_offset + hp.xbuf; ex.ybuf_off = heap_offset + hp.ybuf;
    ex.y_elem_bytes = decode ? (int)sizeof(float) : (int)sizeof(__half); ex.recv_cap = recv_cap;
    EpRouting rt{};
    rt.scores = ws.scores; rt.e_bias = c.e_bias; rt.n = n; rt.topk = c.topk; rt.norm_topk = c.norm_topk;
    rt.routed_scale = c.routed_scale; rt.ids = ws.ids; rt.w = ws.w; rt.expert_offsets = ws.expert_offsets;
    rt.sorted_tok = ws.sorted_tok; rt.sorted_row = ws.sorted_row; rt.slot_pos = ws.slot_pos; rt.status = ws.status;
    st = comm_ep_plan(comm, ex, s, fused_route ? &rt : nullptr);
    if (st) return st;
    if (n > 0 && ids_out && cudaMemcpyAsync(ids_out, ws.ids, (size_t)P * sizeof(int), cudaMemcpyDeviceToDevice, s) != cudaSuccess)
        return GSB_ERR_CUDA;
    if (cudaEventRecord(layer->ep_fork, s) != cudaSuccess || cudaStreamWaitEvent(layer->ep_side, layer->ep_fork, 0) != cudaSuccess)
        return GSB_ERR_CUDA;
    // tcgen05 path on four or more GPUs: the rows travel in two waves (first and second half of every owner's
    // experts) and the routed GEMMs of the first half run while the second half is still on the link - with more
    // ranks more of the rows are remote and the push outlasts the shared expert (8 GPUs: by 0.36 ms)
    const int waves = (!decode && comm->world >= 4 && El >= 2) ? 2 : 1;
    st = comm_ep_push(comm, ex, layer->ep_side, waves);
    if (st) return st;
    if (cudaEventRecord(layer->ep_join, layer->ep_side) != cudaSuccess) return GSB_ERR_CUDA;
    mark(1);

    if (decode) {
        // this GPU's own tokens behind the received rows (fragment order), for the shared expert
        if (n > 0 && c.shared_inter > 0) {
            ep_shared_dst_kernel<<<(n + 255) / 256, 256, 0, s>>>(ws.ydst + recv_cap, reinterpret_cast<float*>(ybuf) + (size_t)P * c.hidden, n, c.hidden);
        }
        DecodeEpArgs d{};
        d.H = c.hidden; d.I = c.moe_inter; d.Is = c.shared_inter; d.El = El;
        d.gate_up_packed = c.gate_up_packed; d.down_packed = c.down_packed;
        d.shared_gate_up_packed = c.shared_gate_up_packed; d.shared_down_packed = c.shared_down_packed;
        d.recv_offsets = ws.recv_offsets; d.xbuf = xbuf; d.recv_cap = recv_cap; d.n = c.shared_inter > 0 ? n : 0;
        d.hbuf = ws.hbuf; d.ydst = reinterpret_cast<float* const*>(ws.ydst); d.segs = ws.segs; d.status = ws.status;
        d.sm_count = layer->sm_count;
        st = launch_decode_ep(d, s, 1);      // the work lists need only the plan: built while the rows travel
        if (st) return st;
        mark(2);
        st = comm_launch_wait(comm, kChDispatch, s);
        if (st) return st;
        mark(3);
        st = launch_decode_ep(d, s, 2);
        if (st) return st;
    } else {
        PrefillEpArgs a{};
        a.gate_up_packed = c.gate_up_packed; a.down_packed = c.down_packed;
        a.shared_gate_up_packed = c.shared_gate_up_packed; a.shared_down_packed = c.shared_down_packed;
        a.H = c.hidden; a.I = c.moe_inter; a.Is = c.shared_inter; a.El = El;
        a.recv_offsets = ws.recv_offsets; a.recv_x = xbuf; a.recv_cap = recv_cap; a.hbuf = ws.hbuf;
        a.ydst = reinterpret_cast<__half* const*>(ws.ydst); a.tiles = ws.tiles;
        a.n = n; a.xs_local = ws.xs_local; a.hbuf_sh = ws.hbuf_sh;
        a.y_shared = reinterpret_cast<__half*>(ybuf) + (size_t)P * c.hidden;
        a.tiles_sh = ws.tiles_sh; a.status = ws.status;
        // the push keeps a few SMs to itself: the shared expert's persistent CTAs take the others, or the
        // CTAs without an SM would start their tiles only when the push is over
        a.sm_count = layer->sm_count - comm_ep_push_sms(P, comm->world);
        if (n > 0) { st = launch_prefill_ep_shared(a, s); if (st) return st; }
        PrefillEpArgs a0 = a, a1 = a;
        if (waves == 2) { a0.e_begin = 0; a0.e_end = (El + 1) / 2; a1.e_begin = (El + 1) / 2; a1.e_end = El; a1.tiles = ws.tiles2; }
        st = launch_prefill_ep_routed(a0, s, 1);   // the tile lists need only the plan
        if (st) return st;
        if (waves == 2) { st = launch_prefill_ep_routed(a1, s, 1); if (st) return st; }
        mark(2);
        st = comm_launch_wait(comm, kChDispatch, s, waves - 1);   // the first (or only) wave of every peer has landed
        if (st) return st;
        mark(3);
        if (waves == 2) {
            st = launch_prefill_ep_routed(a0, s, 2);               // beside this rank's own second wave: not on its SMs
            if (st) return st;
            st = comm_launch_wait(comm, kChDispatch, s);
            if (st) return st;
        }
        // the rest takes every SM: this rank's own push has to be off them first (it normally is by the time
        // every peer's rows have arrived)
        if (cudaStreamWaitEvent(s, layer->ep_join, 0) != cudaSuccess) return GSB_ERR_CUDA;
        PrefillEpArgs& al = waves == 2 ? a1 : a0;
        al.sm_count = layer->sm_count;
        st = launch_prefill_ep_routed(al, s, 2);
        if (st) return st;
    }
    mark(4);
    // this rank's pushes are part of the call: the caller's stream does not run past them
    if (cudaStreamWaitEvent(s, layer->ep_join, 0) != cudaSuccess) return GSB_ERR_CUDA;
    ++comm->seq[kChCombine];
    st = comm_launch_signal_wait(comm, kChCombine, s);
    if (st) return st;
    if (decode)
        st = launch_combine_f32(reinterpret_cast<const float*>(ybuf), ws.slot_pos, ws.w, n, c.topk, c.hidden, P,
                                c.shared_inter > 0 ? 1 : 0, residual, out, s);
    else
        st = launch_combine_h(reinterpret_cast<const __half*>(ybuf), ws.slot_pos, ws.w, n, c.topk, c.hidden, P,
                              c.shared_inter > 0 ? 1 : 0, residual, out, s);
    mark(5);
    return st;
}
}  // namespace

extern "C" {

int gsb_moe_layer_forward_ep(gsb_moe_layer* layer, gsb_comm* comm, const void* x_bf16, int n, float* out,
                             void* workspace, size_t workspace_bytes, size_t heap_offset, int recv_cap,
                             int path, int* ids_out, void* stream) {
    if (n > 0 && !x_bf16) return GSB_ERR_INVALID_ARG;
    return forward_ep_impl(layer, comm, x_bf16, nullptr, nullptr, 0.f, n, out, nullptr, workspace, workspace_bytes,
                           heap_offset, recv_cap, path, ids_out, stream);
}

int gsb_moe_block_layer_forward_ep(gsb_moe_layer* layer, gsb_comm* comm, float* hidden, const float* norm_w, float eps,
                                   int n, void* workspace, size_t workspace_bytes, size_t heap_offset, int recv_cap,
                                   int path, int* ids_out, void* stream) {
    if (n > 0 && (!hidden || !norm_w)) return GSB_ERR_INVALID_ARG;
    return forward_ep_impl(layer, comm, nullptr, hidden, norm_w, eps, n, hidden, hidden, workspace, workspace_bytes,
                           heap_offset, recv_cap, path, ids_out, stream);
}

}  // extern "C"

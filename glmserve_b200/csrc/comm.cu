// Intra-node communication over NVLink peer memory: one process per GPU, a symmetric heap per
// rank mapped into every peer through CUDA IPC, flags with sequence numbers for ordering.
//
// Replaces, for the MoE path, the reference's one-shot CUDA-IPC all-reduce
// (cuda/custom_ar.cu:49-93, cuda/custom_ar.h:26-43) and supplies what the reference does not
// have: the expert-parallel token exchange.  Differences from the reference's kernel: data is
// PULLED from the peers' staging areas (one staging copy per rank instead of world slots),
// large messages take a two-shot reduce-scatter + all-gather, flags use release/acquire at
// system scope, and every wait is bounded (about a second of SM clocks) and reports
// GSB_ERR_TIMEOUT through a status word instead of spinning forever
// (cuda/custom_ar.cu:77-79 spins without limit).
// Sums are taken in rank order 0..world-1 for every element, independent of the message
// size or grid, so a row reduces to the same bits whether it travels alone or in a batch
// (the property the reference's all_reduce_sum_rows exists for, include/nccl_comm.hpp:53-59).
#include <new>

#include "internal.cuh"

namespace gsb {

__device__ __forceinline__ void st_release_sys(int* p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Bounded wait until *p >= seq (sequence numbers only grow).  Returns false on timeout.
__device__ __forceinline__ bool wait_flag(const int* p, int seq, int* status) {
    if (ld_acquire_sys(p) - seq >= 0) return true;
    const long long start = clock64();
    while (ld_acquire_sys(p) - seq < 0) {
        if (clock64() - start > kCommWaitCycles) {
            atomicCAS(status, 0, GSB_ERR_TIMEOUT);
            return false;
        }
    }
    return true;
}
__device__ __forceinline__ int* ctrl_of(const CommPeers& pr, int r) { return reinterpret_cast<int*>(pr.base[r]); }

// Posts `seq` on channel ch to every peer (after all of this grid's earlier writes).
__global__ void signal_kernel(CommPeers pr, int rank, int world, int ch, int seq) {
    __threadfence_system();
    if (threadIdx.x < world && threadIdx.x != rank)
        st_release_sys(ctrl_of(pr, threadIdx.x) + kFlagBase + ch * kMaxWorld + rank, seq);
}
// Waits until every peer posted `seq` on channel ch.
__global__ void wait_kernel(CommPeers pr, int rank, int world, int ch, int seq) {
    int* ctrl = ctrl_of(pr, rank);
    if (threadIdx.x < world && threadIdx.x != rank)
        wait_flag(ctrl + kFlagBase + ch * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord);
}

// ---- all-reduce ---------------------------------------------------------------------------
// Phase 1: copy `data` into the local staging area, then (last block) post the flag.
// Phase 2: wait for every peer's flag.
// Phase 3 (one-shot): out[i] = sum over ranks in rank order of staging_r[i], read over NVLink.
// Two-shot: phase 3 reduces only this rank's slice into a second staging area, posts a second
// flag, and phase 4 gathers every owner's reduced slice.
// Element i of every rank's staging, added in rank order.  The loads of up to eight ranks are issued
// before the first add: a loop that adds as it loads waits one NVLink round trip per rank.
__device__ __forceinline__ float4 sum_over_ranks(const CommPeers& pr, int world, size_t stage_off, int64_t i) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < world; r0 += 8) {
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (r0 + j < world) v[j] = reinterpret_cast<const float4*>(pr.base[r0 + j] + stage_off)[i];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (r0 + j < world) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
    }
    return acc;
}

__global__ void __launch_bounds__(512)
allreduce_kernel(CommPeers pr, int rank, int world, float* __restrict__ data, int64_t count4,
                 size_t stage_off, size_t stage2_off, int seq, int two_shot) {
    int* ctrl = ctrl_of(pr, rank);
    __shared__ int last_block, ok;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    float4* stage = reinterpret_cast<float4*>(pr.base[rank] + stage_off);
    const float4* src = reinterpret_cast<const float4*>(data);
    for (int64_t i = i0; i < count4; i += stride) stage[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        last_block = atomicAdd(ctrl + kArriveCounter, 1) == (int)gridDim.x - 1;
        ok = 1;
    }
    __syncthreads();
    if (last_block && threadIdx.x < world) {
        if (threadIdx.x == 0) ctrl[kArriveCounter] = 0;
        if (threadIdx.x != rank)
            st_release_sys(ctrl_of(pr, threadIdx.x) + kFlagBase + kChAllReduce * kMaxWorld + rank, seq);
    }
    if (threadIdx.x < world && threadIdx.x != rank)
        if (!wait_flag(ctrl + kFlagBase + kChAllReduce * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord)) ok = 0;
    __syncthreads();
    if (!ok) return;
    float4* out = reinterpret_cast<float4*>(data);
    if (!two_shot) {
        for (int64_t i = i0; i < count4; i += stride) out[i] = sum_over_ranks(pr, world, stage_off, i);
        return;
    }
    // two-shot: this rank owns slice [lo, hi)
    const int64_t per = (count4 + world - 1) / world;
    const int64_t lo = min(count4, per * rank), hi = min(count4, lo + per);
    float4* stage2 = reinterpret_cast<float4*>(pr.base[rank] + stage2_off);
    for (int64_t i = lo + i0; i < hi; i += stride) {
        const float4 acc = sum_over_ranks(pr, world, stage_off, i);
        stage2[i] = acc;
        out[i] = acc;
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) last_block = atomicAdd(ctrl + kArriveCounter + 1, 1) == (int)gridDim.x - 1;
    __syncthreads();
    if (last_block && threadIdx.x < world) {
        if (threadIdx.x == 0) ctrl[kArriveCounter + 1] = 0;
        if (threadIdx.x != rank)
            st_release_sys(ctrl_of(pr, threadIdx.x) + kFlagBase + kChAllReduce2 * kMaxWorld + rank, seq);
    }
    if (threadIdx.x < world && threadIdx.x != rank)
        if (!wait_flag(ctrl + kFlagBase + kChAllReduce2 * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord)) ok = 0;
    __syncthreads();
    if (!ok) return;
    for (int r = 0; r < world; ++r) {
        if (r == rank) continue;
        const int64_t rlo = min(count4, per * r), rhi = min(count4, rlo + per);
        const float4* rs = reinterpret_cast<const float4*>(pr.base[r] + stage2_off);
        for (int64_t i = rlo + i0; i < rhi; i += stride) out[i] = rs[i];
    }
}

// ---- expert-parallel exchange ---------------------------------------------------------------
// Counts: rank posts its per-expert row counts (from its local dispatch offsets) to every peer.
__global__ void ep_post_counts_kernel(CommPeers pr, int rank, int world, const int* __restrict__ expert_offsets,
                                      int E, int seq) {
    for (int p = 0; p < world; ++p) {
        int* dst = ctrl_of(pr, p) + kCntBase + rank * kMaxExperts;
        for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = expert_offsets[e + 1] - expert_offsets[e];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank)
        st_release_sys(ctrl_of(pr, threadIdx.x) + kFlagBase + kChCounts * kMaxWorld + rank, seq);
}

// After every rank's counts arrived: the layout of the rows this rank RECEIVES (local expert
// major, then source rank, then the source's order) and where the rows it SENDS land.
//   recv_offsets[El + 1]      first received row of each local expert (El = E / world)
//   send_base[E]              row index on the owner's receive buffer of this rank's first row for expert e
//   ydst[row]                 for each received row: where its output row goes (peer ybuf row pointer)
// One block; E <= 1024.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(CommPeers pr, int rank, int world, int E, int seq, int* __restrict__ recv_offsets,
               int* __restrict__ send_base, float** __restrict__ ydst, size_t ybuf_off, int H, int y_elem_bytes,
               int recv_cap, int* __restrict__ recv_total) {
    int* ctrl = ctrl_of(pr, rank);
    __shared__ int tot_s[kMaxExperts];             // rows of expert e over all sources
    __shared__ int base_s[kMaxExperts];            // first receive row of expert e on its owner
    __shared__ int spos_s[kMaxWorld][kMaxExperts]; // position of expert e's rows in source s's sorted order
    if (threadIdx.x < world && threadIdx.x != rank)
        wait_flag(ctrl + kFlagBase + kChCounts * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord);
    __syncthreads();
    const int* cnt = ctrl + kCntBase;              // [src][e]
    const int El = E / world;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0;
        for (int s = 0; s < world; ++s) t += cnt[s * kMaxExperts + e];
        tot_s[e] = t;
    }
    if (threadIdx.x < world) {                     // one thread per source: running prefix over experts
        int run = 0;
        for (int e = 0; e < E; ++e) { spos_s[threadIdx.x][e] = run; run += cnt[threadIdx.x * kMaxExperts + e]; }
    }
    __syncthreads();
    if (threadIdx.x < world) {                     // one thread per owner: running prefix over its experts
        int run = 0;
        for (int e = threadIdx.x * El; e < (threadIdx.x + 1) * El; ++e) { base_s[e] = run; run += tot_s[e]; }
        if (threadIdx.x == rank) {
            recv_offsets[El] = run;
            *recv_total = run;
            if (run > recv_cap) atomicCAS(ctrl + kStatusWord, 0, GSB_ERR_TOO_LARGE);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int before = 0;
        for (int s = 0; s < rank; ++s) before += cnt[s * kMaxExperts + e];
        send_base[e] = base_s[e] + before;
        if (e / El == rank) recv_offsets[e - rank * El] = base_s[e];
    }
    // output destinations of the rows this rank will compute: one warp per (local expert, source)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    for (int job = warp; job < El * world; job += nwarp) {
        const int el = job / world, sidx = job - el * world;
        const int e = rank * El + el;
        int row = base_s[e];
        for (int s2 = 0; s2 < sidx; ++s2) row += cnt[s2 * kMaxExperts + e];
        const int c = cnt[sidx * kMaxExperts + e];
        const int src_pos = spos_s[sidx][e];
        for (int i = lane; i < c; i += 32)
            if (row + i < recv_cap)
                ydst[row + i] = reinterpret_cast<float*>(pr.base[sidx] + ybuf_off + (size_t)(src_pos + i) * H * y_elem_bytes);
    }
}

// Dispatch: every local (token, slot) row, in sorted order, is stored as fp16 into the owner's
// receive buffer over NVLink (16-byte stores); one block per row.
__global__ void __launch_bounds__(256)
ep_dispatch_push_kernel(CommPeers pr, int world, int E, const __nv_bfloat16* __restrict__ x,
                        const int* __restrict__ expert_offsets, const int* __restrict__ sorted_tok,
                        const int* __restrict__ send_base, const int* __restrict__ sorted_expert, int H,
                        size_t recv_off, int recv_cap) {
    const int r = blockIdx.x;
    const int e = sorted_expert[r];
    const int owner = e / (E / world);
    const int dst_row = send_base[e] + (r - expert_offsets[e]);
    if (dst_row >= recv_cap) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)sorted_tok[r] * H);
    uint4* dst = reinterpret_cast<uint4*>(pr.base[owner] + recv_off + (size_t)dst_row * H * 2);
    for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
        const uint4 in = __ldg(src + v);
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&in);
        uint4 o;
        uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 f = __bfloat1622float2(bp[q]);
            f.x = fminf(fmaxf(f.x, -65504.f), 65504.f);
            f.y = fminf(fmaxf(f.y, -65504.f), 65504.f);
            const __half2 hh = __floats2half2_rn(f.x, f.y);
            op[q] = *reinterpret_cast<const uint32_t*>(&hh);
        }
        dst[v] = o;
    }
}

// expert id of every sorted row (inverse of the offsets), for the push kernel
__global__ void rows_to_expert_kernel(const int* __restrict__ expert_offsets, int E, int* __restrict__ sorted_expert) {
    const int e = blockIdx.x;
    for (int r = expert_offsets[e] + threadIdx.x; r < expert_offsets[e + 1]; r += blockDim.x) sorted_expert[r] = e;
}

int comm_launch_signal(gsb_comm* c, int ch, cudaStream_t s) {
    signal_kernel<<<1, 32, 0, s>>>(c->peers, c->rank, c->world, ch, (int)c->seq[ch]);
    return launch_status();
}
int comm_launch_wait(gsb_comm* c, int ch, cudaStream_t s) {
    wait_kernel<<<1, 32, 0, s>>>(c->peers, c->rank, c->world, ch, (int)c->seq[ch]);
    return launch_status();
}

// Count exchange, plan, dispatch push and its signal - everything up to (not including) the wait
// for the peers' rows.  The caller waits on kChDispatch before reading its receive buffer.
int comm_ep_exchange(gsb_comm* c, const __nv_bfloat16* x, const int* expert_offsets, const int* sorted_tok,
                     int P, int E, int H, int* sorted_expert, int* recv_offsets, int* send_base, void** ydst,
                     size_t ybuf_off, int y_elem_bytes, size_t recv_off, int recv_cap, int* recv_total,
                     cudaStream_t s) {
    if (E > kMaxExperts || E % c->world) return GSB_ERR_UNSUPPORTED;
    rows_to_expert_kernel<<<E, 128, 0, s>>>(expert_offsets, E, sorted_expert);
    const int seq_c = (int)++c->seq[kChCounts];
    ep_post_counts_kernel<<<1, 256, 0, s>>>(c->peers, c->rank, c->world, expert_offsets, E, seq_c);
    ep_plan_kernel<<<1, 1024, 0, s>>>(c->peers, c->rank, c->world, E, seq_c, recv_offsets, send_base,
                                      reinterpret_cast<float**>(ydst), kCtrlBytes + ybuf_off, H, y_elem_bytes,
                                      recv_cap, recv_total);
    if (P > 0)
        ep_dispatch_push_kernel<<<P, 256, 0, s>>>(c->peers, c->world, E, x, expert_offsets, sorted_tok, send_base,
                                                  sorted_expert, H, kCtrlBytes + recv_off, recv_cap);
    ++c->seq[kChDispatch];
    return comm_launch_signal(c, kChDispatch, s);
}

}  // namespace gsb

using namespace gsb;

extern "C" {

int gsb_comm_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

int gsb_comm_create(int rank, int world, size_t heap_bytes, void* out_handle, gsb_comm** out) {
    if (!out || !out_handle || rank < 0 || world < 1 || rank >= world) return GSB_ERR_INVALID_ARG;
    if (world > kMaxWorld) return GSB_ERR_UNSUPPORTED;
    gsb_comm* c = new (std::nothrow) gsb_comm();
    if (!c) return GSB_ERR_CUDA;
    c->rank = rank; c->world = world;
    c->heap_bytes = (heap_bytes + 255) / 256 * 256;
    if (cudaMalloc(reinterpret_cast<void**>(&c->local), kCtrlBytes + c->heap_bytes) != cudaSuccess) { delete c; return GSB_ERR_CUDA; }
    if (cudaMemset(c->local, 0, kCtrlBytes) != cudaSuccess) { cudaFree(c->local); delete c; return GSB_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, c->local) != cudaSuccess) { cudaFree(c->local); delete c; return GSB_ERR_CUDA; }
    memcpy(out_handle, &h, sizeof(h));
    c->peers.base[rank] = c->local;
    *out = c;
    return GSB_OK;
}

int gsb_comm_open(gsb_comm* c, const void* handles) {
    if (!c || !handles) return GSB_ERR_INVALID_ARG;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles) + (size_t)r * sizeof(h), sizeof(h));
        void* p = nullptr;
        if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return GSB_ERR_CUDA;
        c->peers.base[r] = static_cast<uint8_t*>(p);
        c->opened[r] = true;
    }
    return GSB_OK;
}

void gsb_comm_destroy(gsb_comm* c) {
    if (!c) return;
    for (int r = 0; r < c->world; ++r)
        if (c->opened[r]) cudaIpcCloseMemHandle(c->peers.base[r]);
    if (c->local) cudaFree(c->local);
    delete c;
}

void* gsb_comm_heap(gsb_comm* c) { return c ? c->local + kCtrlBytes : nullptr; }
size_t gsb_comm_heap_bytes(gsb_comm* c) { return c ? c->heap_bytes : 0; }
int gsb_comm_rank(gsb_comm* c) { return c ? c->rank : -1; }
int gsb_comm_world(gsb_comm* c) { return c ? c->world : 0; }

int gsb_comm_status(gsb_comm* c) {
    if (!c) return GSB_ERR_INVALID_ARG;
    int st = 0;
    if (cudaMemcpy(&st, c->local, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return GSB_ERR_CUDA;
    if (st) cudaMemset(c->local, 0, sizeof(int));
    return st;
}

int gsb_comm_barrier(gsb_comm* c, void* stream) {
    if (!c) return GSB_ERR_INVALID_ARG;
    if (c->world == 1) return GSB_OK;
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    ++c->seq[kChBarrier];
    int st = comm_launch_signal(c, kChBarrier, s);
    if (st) return st;
    return comm_launch_wait(c, kChBarrier, s);
}

// The first `2 * 2 * stage_floats` floats of the heap are the all-reduce staging (two parities,
// two areas); callers that also use the heap for expert parallelism place their buffers after
// gsb_comm_allreduce_reserve() bytes.
size_t gsb_comm_allreduce_reserve(gsb_comm* c, int64_t max_count) {
    if (!c || max_count < 0) return 0;
    const size_t fl = ((size_t)max_count + 3) / 4 * 4;
    c->ar_stage_floats = fl;
    return 4 * fl * sizeof(float);
}

int gsb_comm_allreduce_one_shot_limit(gsb_comm* c, int64_t total_floats) {
    if (!c || total_floats < 0) return GSB_ERR_INVALID_ARG;
    c->ar_one_shot_limit = total_floats ? total_floats : (int64_t)(1 << 21);
    return GSB_OK;
}

int gsb_comm_allreduce_sum(gsb_comm* c, float* data, int64_t count, void* stream) {
    if (!c || count < 0 || (count > 0 && !data)) return GSB_ERR_INVALID_ARG;
    if (c->world == 1 || count == 0) return GSB_OK;
    if (count % 4 || (reinterpret_cast<uintptr_t>(data) & 15)) return GSB_ERR_INVALID_ARG;
    if ((size_t)count > c->ar_stage_floats) return GSB_ERR_TOO_LARGE;
    if (4 * c->ar_stage_floats * sizeof(float) > c->heap_bytes) return GSB_ERR_WORKSPACE;
    const unsigned seq = ++c->seq[kChAllReduce];
    c->seq[kChAllReduce2] = seq;
    const int parity = seq & 1;
    const size_t stage_off = kCtrlBytes + (size_t)parity * 2 * c->ar_stage_floats * sizeof(float);
    const size_t stage2_off = stage_off + c->ar_stage_floats * sizeof(float);
    const int64_t count4 = count / 4;
    const int two_shot = count * c->world > c->ar_one_shot_limit ? 1 : 0;
    int sms = 148;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int64_t blocks = (count4 + 511) / 512;
    if (blocks > sms) blocks = sms;   // every block must be resident: they wait on one another's flags
    allreduce_kernel<<<(unsigned)blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
        c->peers, c->rank, c->world, data, count4, stage_off, stage2_off, (int)seq, two_shot);
    return launch_status();
}

}  // extern "C"

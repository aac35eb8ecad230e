// Intra-node communication over NVLink peer memory: one process per GPU, a symmetric heap per
// rank mapped into every peer through CUDA IPC, flags with sequence numbers for ordering.
//
// Replaces, for the MoE path, the reference's one-shot CUDA-IPC all-reduce
// (cuda/custom_ar.cu:49-93, cuda/custom_ar.h:26-43) and supplies what the reference does not
// have: the expert-parallel token exchange.  Like the reference's kernel the all-reduce PUSHES:
// a rank stores its data straight into a slot of its own on every peer, then a flag, and each
// rank sums slots that sit in its own memory - one NVLink traversal on the critical path.
// Unlike it, flags are per thread block (block b of a rank waits only for block b of its
// peers, which wrote the same element range: no grid-wide arrival counter), large messages take
// a two-shot reduce-scatter + all-gather (also pushed), flags use release/acquire at system
// scope, and every wait is bounded (gsb_comm_set_wait_cycles, about two seconds of SM clocks by
// default) and reports GSB_ERR_TIMEOUT through a status word instead of spinning forever
// (cuda/custom_ar.cu:77-79 spins without limit).
// Sums are taken in rank order 0..world-1 for every element, independent of the message
// size, the algorithm or the grid, so a row reduces to the same bits whether it travels alone or
// in a batch (the property the reference's all_reduce_sum_rows exists for,
// include/nccl_comm.hpp:53-59).
#include <new>

#include "internal.cuh"
#include "route_device.cuh"

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
__device__ __forceinline__ bool wait_flag(const int* p, int seq, int* status, long long limit) {
    if (ld_acquire_sys(p) - seq >= 0) return true;
    const long long start = clock64();
    while (ld_acquire_sys(p) - seq < 0) {
        if (clock64() - start > limit) {
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
// Waits until every peer posted `seq` on channel ch (a timeout is recorded in the status word; what
// runs afterwards must be safe on stale data, see ep_plan_kernel).
__global__ void wait_kernel(CommPeers pr, int rank, int world, int ch, int seq, long long limit) {
    int* ctrl = ctrl_of(pr, rank);
    if (threadIdx.x < world && threadIdx.x != rank)
        wait_flag(ctrl + kFlagBase + ch * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord, limit);
}

__global__ void signal_wait_kernel(CommPeers pr, int rank, int world, int ch, int seq, long long limit) {
    __threadfence_system();
    int* ctrl = ctrl_of(pr, rank);
    if (threadIdx.x < world && threadIdx.x != rank) {
        st_release_sys(ctrl_of(pr, threadIdx.x) + kFlagBase + ch * kMaxWorld + rank, seq);
        wait_flag(ctrl + kFlagBase + ch * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord, limit);
    }
}

// ---- all-reduce ---------------------------------------------------------------------------
// Staging of one parity: two areas of `area` floats.
//   one-shot  slot[src] = area 0 + src * count floats (both areas together; needs world * count <= 2 * area).
//             Block b owns elements [b * chunk, (b + 1) * chunk): it stores them into its slot on every peer,
//             posts flag(0, rank, b) to every peer, waits for flag(0, s, b) of every peer s, then sums the
//             slots (its own contribution straight from `data`) in rank order into `data`.
//   two-shot  rank j owns slice j of `per` elements.  Area 0 holds world scatter slots of `per` elements,
//             area 1 the gathered result.  Block b takes sub-range b of EVERY slice: it pushes its part of
//             slice j to rank j, flags, waits, sums its part of the own slice in rank order, pushes the sums
//             to every peer's gather area, flags (phase 1), waits, and copies the other slices' sums home.
// Every rank launches the same grid for the same count, so "block b" means the same elements everywhere.
struct ArArgs {
    CommPeers pr;
    int rank, world;
    float* data;
    int64_t count4;          // float4 elements
    size_t stage_off;        // byte offset (from the heap base pointer) of this parity's staging
    size_t area_bytes;       // bytes of one area
    int seq;
    int two_shot;
    long long wait_cycles;
};

__device__ __forceinline__ int* blk_flag(const CommPeers& pr, int owner, int phase, int src) {
    return ctrl_of(pr, owner) + kBlkFlagBase + (phase * kMaxWorld + src) * kMaxArBlocks + (int)blockIdx.x;
}

// All peers' block-b flags of `phase`: post ours, then wait for theirs.  Returns false on a timeout (all threads).
__device__ __forceinline__ bool ar_exchange_flags(const ArArgs& a, int phase, int* ok_s) {
    if (threadIdx.x == 0) *ok_s = 1;
    // The block's stores are ordered before the flags by the barrier plus the release of the flag store
    // itself (release is cumulative over what the storing thread observed through the barrier): one
    // release per peer, not a system-wide fence by every thread.
    __syncthreads();
    if (threadIdx.x < a.world && threadIdx.x != a.rank) {
        st_release_sys(blk_flag(a.pr, threadIdx.x, phase, a.rank), a.seq);
        if (!wait_flag(blk_flag(a.pr, a.rank, phase, threadIdx.x), a.seq, ctrl_of(a.pr, a.rank) + kStatusWord, a.wait_cycles))
            *ok_s = 0;
    }
    __syncthreads();
    return *ok_s != 0;
}

__device__ __forceinline__ float4 ld_cg4(const float4* p) { return __ldcg(p); }

__global__ void __launch_bounds__(256)
allreduce_kernel(const ArArgs a) {
    __shared__ int ok_s;
    const int B = (int)gridDim.x, b = (int)blockIdx.x;
    float4* data = reinterpret_cast<float4*>(a.data);
    // Every loop below first asks for all the values a thread will need in one go and only then stores or adds:
    // written as load-store pairs, the stores (which may alias the loads for all the compiler knows) keep
    // the next load from being issued, and a pass becomes a chain of memory round trips.
    if (!a.two_shot) {
        constexpr int U = 4;
        const int64_t chunk = (a.count4 + B - 1) / B;
        const int64_t lo = min(a.count4, chunk * b), hi = min(a.count4, lo + chunk);
        const size_t slot_bytes = (size_t)a.count4 * sizeof(float4);
        for (int64_t i0 = lo + threadIdx.x; i0 < hi; i0 += (int64_t)U * blockDim.x) {
            float4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i0 + u * (int64_t)blockDim.x < hi) v[u] = data[i0 + u * (int64_t)blockDim.x];
            for (int p = 0; p < a.world; ++p) {
                if (p == a.rank) continue;
                float4* dst = reinterpret_cast<float4*>(a.pr.base[p] + a.stage_off + a.rank * slot_bytes);
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (i0 + u * (int64_t)blockDim.x < hi) dst[i0 + u * (int64_t)blockDim.x] = v[u];
            }
        }
        if (!ar_exchange_flags(a, 0, &ok_s)) return;
        const uint8_t* mine = a.pr.base[a.rank] + a.stage_off;
        for (int64_t i0 = lo + threadIdx.x; i0 < hi; i0 += 2 * (int64_t)blockDim.x) {
            float4 v[2][kMaxWorld];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int64_t i = i0 + u * (int64_t)blockDim.x;
#pragma unroll
                for (int r = 0; r < kMaxWorld; ++r)
                    if (i < hi && r < a.world)
                        v[u][r] = r == a.rank ? data[i] : ld_cg4(reinterpret_cast<const float4*>(mine + r * slot_bytes) + i);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int64_t i = i0 + u * (int64_t)blockDim.x;
                if (i >= hi) continue;
                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int r = 0; r < kMaxWorld; ++r)
                    if (r < a.world) { acc.x += v[u][r].x; acc.y += v[u][r].y; acc.z += v[u][r].z; acc.w += v[u][r].w; }
                data[i] = acc;
            }
        }
        return;
    }
    const int64_t per = (a.count4 + a.world - 1) / a.world;   // slice length
    const int64_t sub = (per + B - 1) / B;                     // this block's part of a slice
    const size_t slot_bytes = (size_t)per * sizeof(float4);
    // scatter: my part of slice j goes to rank j's slot for me
    for (int64_t k = threadIdx.x; k < sub; k += blockDim.x) {
        float4 v[kMaxWorld];
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j) {
            if (j >= a.world || j == a.rank) continue;
            const int64_t slo = min(a.count4, per * j), shi = min(a.count4, slo + per);
            const int64_t i = slo + sub * b + k;
            if (i < shi) v[j] = data[i];
        }
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j) {
            if (j >= a.world || j == a.rank) continue;
            const int64_t slo = min(a.count4, per * j), shi = min(a.count4, slo + per);
            const int64_t i = slo + sub * b + k;
            if (i < shi) reinterpret_cast<float4*>(a.pr.base[j] + a.stage_off + a.rank * slot_bytes)[i - slo] = v[j];
        }
    }
    if (!ar_exchange_flags(a, 0, &ok_s)) return;
    {   // reduce my part of my slice in rank order, write it home and into every peer's gather area
        const int64_t slo = min(a.count4, per * a.rank), shi = min(a.count4, slo + per);
        const int64_t lo = min(shi, slo + sub * b), hi = min(shi, lo + sub);
        const uint8_t* mine = a.pr.base[a.rank] + a.stage_off;
        for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            float4 v[kMaxWorld];
#pragma unroll
            for (int r = 0; r < kMaxWorld; ++r)
                if (r < a.world) v[r] = r == a.rank ? data[i] : ld_cg4(reinterpret_cast<const float4*>(mine + r * slot_bytes) + (i - slo));
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < kMaxWorld; ++r)
                if (r < a.world) { acc.x += v[r].x; acc.y += v[r].y; acc.z += v[r].z; acc.w += v[r].w; }
            data[i] = acc;
            for (int p = 0; p < a.world; ++p)
                if (p != a.rank) reinterpret_cast<float4*>(a.pr.base[p] + a.stage_off + a.area_bytes)[i] = acc;
        }
    }
    if (!ar_exchange_flags(a, 1, &ok_s)) return;
    const float4* gathered = reinterpret_cast<const float4*>(a.pr.base[a.rank] + a.stage_off + a.area_bytes);
    for (int64_t k = threadIdx.x; k < sub; k += blockDim.x) {
        float4 v[kMaxWorld];
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j) {
            if (j >= a.world || j == a.rank) continue;
            const int64_t slo = min(a.count4, per * j), shi = min(a.count4, slo + per);
            const int64_t i = slo + sub * b + k;
            if (i < shi) v[j] = ld_cg4(gathered + i);
        }
#pragma unroll
        for (int j = 0; j < kMaxWorld; ++j) {
            if (j >= a.world || j == a.rank) continue;
            const int64_t slo = min(a.count4, per * j), shi = min(a.count4, slo + per);
            const int64_t i = slo + sub * b + k;
            if (i < shi) data[i] = v[j];
        }
    }
}

// Flag-in-data form for decode-sized messages: a 16-byte word carries two floats and the call's sequence number
// twice, {x, seq, y, seq} - each 8-byte half validates itself, so the word may cross the link as one store or as
// two.  A rank stores its words into its slot on every peer and then polls the peers' slots in its own memory
// until both sequence numbers match: no fence, no separate flag, one NVLink traversal (the exchange of flags
// costs the other forms ~4.7 us a round).  Slots alternate between two parities: a rank can be one call ahead of
// a peer, never two, because a call needs every peer's words of the same call.  Sum order: rank 0..world-1 per
// element with the own contribution from `data`, as in the other forms - the same bits.
__global__ void __launch_bounds__(256)
allreduce_ll_kernel(const ArArgs a) {
    const int64_t nw = a.count4 * 2;
    const uint32_t seq = (uint32_t)a.seq;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const float2* in = reinterpret_cast<const float2*>(a.data);
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < nw; w += stride) {
        const float2 v = in[w];
        const uint32_t x = __float_as_uint(v.x), y = __float_as_uint(v.y);
        for (int p = 0; p < a.world; ++p) {
            if (p == a.rank) continue;
            uint8_t* dst = a.pr.base[p] + a.stage_off + (size_t)a.rank * a.area_bytes + (size_t)w * 16;
            asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(x), "r"(seq), "r"(y), "r"(seq) : "memory");
        }
    }
    const uint8_t* mine = a.pr.base[a.rank] + a.stage_off;
    const long long start = clock64();
    for (int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; w < nw; w += stride) {
        uint4 got[kMaxWorld];
        uint32_t pending = 0;
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r)
            if (r < a.world && r != a.rank) pending |= 1u << r;
        while (pending) {
#pragma unroll
            for (int r = 0; r < kMaxWorld; ++r) {
                if (!(pending >> r & 1u)) continue;
                const uint8_t* src = mine + (size_t)r * a.area_bytes + (size_t)w * 16;
                asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                             : "=r"(got[r].x), "=r"(got[r].y), "=r"(got[r].z), "=r"(got[r].w) : "l"(src) : "memory");
            }
#pragma unroll
            for (int r = 0; r < kMaxWorld; ++r)
                if ((pending >> r & 1u) && got[r].y == seq && got[r].w == seq) pending &= ~(1u << r);
            if (pending && clock64() - start > a.wait_cycles) {
                atomicCAS(ctrl_of(a.pr, a.rank) + kStatusWord, 0, GSB_ERR_TIMEOUT);
                return;
            }
        }
        const float2 own = in[w];
        float2 acc = make_float2(0.f, 0.f);
#pragma unroll
        for (int r = 0; r < kMaxWorld; ++r) {
            if (r >= a.world) continue;
            acc.x += r == a.rank ? own.x : __uint_as_float(got[r].x);
            acc.y += r == a.rank ? own.y : __uint_as_float(got[r].z);
        }
        reinterpret_cast<float2*>(a.data)[w] = acc;
    }
}

// ---- expert-parallel exchange ---------------------------------------------------------------
// Counts: rank posts its per-expert row counts (from its local dispatch offsets) and the layout of its
// own buffers {receive buffer offset, receive capacity, per-slot row buffer offset} to every peer, so a
// peer never derives an address on this rank from its own arguments.
__device__ __forceinline__ void ep_post_counts_block(const CommPeers& pr, int rank, int world,
                                                     const int* __restrict__ expert_offsets, int E, int seq,
                                                     int recv_off_kib, int recv_cap, int ybuf_off_kib) {
    for (int p = 0; p < world; ++p) {
        int* dst = ctrl_of(pr, p) + kCntBase + rank * kMaxExperts;
        for (int e = threadIdx.x; e < E; e += blockDim.x) dst[e] = expert_offsets[e + 1] - expert_offsets[e];
        if (threadIdx.x == 0) {
            int* m = ctrl_of(pr, p) + kMetaBase + rank * 8;
            m[0] = recv_off_kib; m[1] = recv_cap; m[2] = ybuf_off_kib;
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank)
        st_release_sys(ctrl_of(pr, threadIdx.x) + kFlagBase + kChCounts * kMaxWorld + rank, seq);
}
__global__ void ep_post_counts_kernel(CommPeers pr, int rank, int world, const int* __restrict__ expert_offsets,
                                      int E, int seq, int recv_off_kib, int recv_cap, int ybuf_off_kib) {
    ep_post_counts_block(pr, rank, world, expert_offsets, E, seq, recv_off_kib, recv_cap, ybuf_off_kib);
}

// Small decode batches (at most kRouteTokens tokens): top-k selection, dispatch and the posting of the counts
// in ONE launch of one block - three launches and a memset less ahead of the exchange.  Each step is the
// stand-alone kernel's body, so ids, weights and permutation are the same bits.
constexpr int kRouteTokens = 32;    // one token per warp: a single block is slower than the separate launches beyond that
                                    // (128 tokens per GPU: route + plan 98 us fused, 80 us as three launches)
__global__ void __launch_bounds__(kDispWarps * 32)
ep_route_post_kernel(CommPeers pr, int rank, int world, const float* __restrict__ scores,
                     const float* __restrict__ e_bias, int n, int E, int topk, int norm_topk, float routed_scale,
                     int* __restrict__ ids, float* __restrict__ w, int* __restrict__ expert_offsets,
                     int* __restrict__ sorted_tok, int* __restrict__ sorted_row, int* __restrict__ slot_pos,
                     int* __restrict__ status, int seq, int recv_off_kib, int recv_cap, int ybuf_off_kib) {
    extern __shared__ int route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x < 4) status[threadIdx.x] = 0;
    for (int t = warp; t < n; t += kDispWarps) {
        if (E <= 256) topk_token<8, true>(scores + (size_t)t * E, e_bias, E, topk, norm_topk, routed_scale, lane,
                                          ids + (size_t)t * topk, w + (size_t)t * topk);
        else topk_token<32, true>(scores + (size_t)t * E, e_bias, E, topk, norm_topk, routed_scale, lane,
                                  ids + (size_t)t * topk, w + (size_t)t * topk);
    }
    __syncthreads();   // the block's own global writes (ids) are visible to it from here
    dispatch_block(ids, n * topk, topk, E, expert_offsets, sorted_tok, sorted_row, slot_pos, route_smem);
    __syncthreads();
    ep_post_counts_block(pr, rank, world, expert_offsets, E, seq, recv_off_kib, recv_cap, ybuf_off_kib);
}

constexpr int kDestShift = 27;   // row_dest = wave << 30 | owner << 27 | row (receive capacities stay below 2^27 rows)
constexpr int kDestWaveBit = 30; // wave 1 = the second half of the owner's resident experts

// After every rank's counts arrived: the layout of the rows this rank RECEIVES (local expert
// major, then source rank, then the source's order) and where the rows it SENDS land.
//   recv_offsets[El + 1]      first received row of each local expert (El = E / world), clamped to recv_cap
//   send_base[E]              row index on the owner's receive buffer of this rank's first row for expert e
//   ydst[row]                 for each received row: where its output row goes (the source's row buffer)
//   row_dest[P]               for each sorted row this rank sends: owner rank and row of the owner's receive
//                             buffer packed into one int (-1: the owner has no room for it)
//   plan[0] = 1 when every peer's counts arrived (0: nothing is pushed and nothing is computed),
//   plan[1] = rows received, plan[4 + 4r ..] = rank r's posted {receive offset KiB, capacity, row buffer KiB}
// More rows than recv_cap: GSB_ERR_TOO_LARGE is recorded, the offsets are clamped so that no tile, row of
// the intermediate buffer or ydst entry lies beyond recv_cap, and the senders drop the rows that do not fit.
// One block; E <= 1024.
__global__ void __launch_bounds__(1024)
ep_plan_kernel(CommPeers pr, int rank, int world, int E, int seq, int* __restrict__ recv_offsets,
               int* __restrict__ send_base, void** __restrict__ ydst, int H, int y_elem_bytes,
               int recv_cap, int own_ybuf_kib, int* __restrict__ plan, long long wait_cycles,
               const int* __restrict__ expert_offsets, int* __restrict__ row_dest) {
    int* ctrl = ctrl_of(pr, rank);
    __shared__ int tot_s[kMaxExperts];             // rows of expert e over all sources
    __shared__ int base_s[kMaxExperts];            // first receive row of expert e on its owner
    __shared__ int spos_s[kMaxWorld][kMaxExperts]; // position of expert e's rows in source s's sorted order
    __shared__ int ok_s;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != rank)
        if (!wait_flag(ctrl + kFlagBase + kChCounts * kMaxWorld + threadIdx.x, seq, ctrl + kStatusWord, wait_cycles)) ok_s = 0;
    __syncthreads();
    const int El = E / world;
    if (!ok_s) {   // a peer never posted: plan nothing (stale counts must not steer any address)
        for (int e = threadIdx.x; e < E; e += blockDim.x) send_base[e] = 0;
        for (int e = threadIdx.x; e <= El; e += blockDim.x) recv_offsets[e] = 0;
        if (threadIdx.x == 0) { plan[0] = 0; plan[1] = 0; }
        return;
    }
    const int* cnt = ctrl + kCntBase;              // [src][e]
    const int* meta = ctrl + kMetaBase;            // [src][8]
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int t = 0;
        for (int s = 0; s < world; ++s) t += cnt[s * kMaxExperts + e];
        tot_s[e] = t;
    }
    if (threadIdx.x < world) {                     // one thread per source: running prefix over experts
        int run = 0;
        for (int e = 0; e < E; ++e) { spos_s[threadIdx.x][e] = run; run += cnt[threadIdx.x * kMaxExperts + e]; }
        plan[4 + 4 * threadIdx.x + 0] = threadIdx.x == rank ? 0 : meta[threadIdx.x * 8 + 0];
        plan[4 + 4 * threadIdx.x + 1] = threadIdx.x == rank ? recv_cap : meta[threadIdx.x * 8 + 1];
        plan[4 + 4 * threadIdx.x + 2] = threadIdx.x == rank ? own_ybuf_kib : meta[threadIdx.x * 8 + 2];
    }
    __syncthreads();
    if (threadIdx.x < world) {                     // one thread per owner: running prefix over its experts
        int run = 0;
        for (int e = threadIdx.x * El; e < (threadIdx.x + 1) * El; ++e) { base_s[e] = run; run += tot_s[e]; }
        if (threadIdx.x == rank) {
            recv_offsets[El] = min(run, recv_cap);
            plan[0] = 1; plan[1] = min(run, recv_cap);
            if (run > recv_cap) atomicCAS(ctrl + kStatusWord, 0, GSB_ERR_TOO_LARGE);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int before = 0;
        for (int s = 0; s < rank; ++s) before += cnt[s * kMaxExperts + e];
        send_base[e] = base_s[e] + before;
        tot_s[e] = base_s[e] + before;             // (the totals are used up) kept for the row loop below
        if (e / El == rank) recv_offsets[e - rank * El] = min(base_s[e], recv_cap);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarp = blockDim.x >> 5;
    // where every sorted row this rank sends goes: one warp per expert
    for (int e = warp; e < E; e += nwarp) {
        const int owner = e / El, base = tot_s[e], beg = expert_offsets[e], end = expert_offsets[e + 1];
        const int cap = owner == rank ? recv_cap : meta[owner * 8 + 1];
        for (int r = beg + lane; r < end; r += 32) {
            const int dst_row = base + (r - beg);
            row_dest[r] = dst_row < cap ? ((((e - owner * El) >= (El + 1) / 2 ? 1 : 0) << kDestWaveBit) | (owner << kDestShift) | dst_row) : -1;
        }
    }
    // output destinations of the rows this rank will compute: one warp per (local expert, source)
    for (int job = warp; job < El * world; job += nwarp) {
        const int el = job / world, sidx = job - el * world;
        const int e = rank * El + el;
        int row = base_s[e];
        for (int s2 = 0; s2 < sidx; ++s2) row += cnt[s2 * kMaxExperts + e];
        const int c = cnt[sidx * kMaxExperts + e];
        const int src_pos = spos_s[sidx][e];
        // the source's own row buffer, at the offset the source posted (this rank's own: its argument)
        const size_t yoff = kCtrlBytes + ((size_t)(sidx == rank ? own_ybuf_kib : meta[sidx * 8 + 2]) << 10);
        for (int i = lane; i < c; i += 32)
            if (row + i < recv_cap)
                ydst[row + i] = pr.base[sidx] + yoff + (size_t)(src_pos + i) * H * y_elem_bytes;
    }
}

// Dispatch: every local (token, slot) row, in sorted order, is stored as fp16 into the owner's
// receive buffer over NVLink (16-byte stores), at the offset and within the capacity the OWNER
// posted.  frag_order: the decode kernels' fragment order instead of natural order.
// The push owns a FEW WHOLE SMs (kPushBlocks blocks whose staging buffers take most of an SM's shared memory,
// so no GEMM CTA can sit beside them) and the shared expert's GEMMs, launched right after on the caller's
// stream, take the others (comm_ep_push_sms).  The rows are pushed as they lie in `xh` (fp16, already in the
// order the receiving kernels want), so the copy unit does all of it: one lane per warp runs a two-buffer
// pipeline of bulk copies, global -> shared (completion on an mbarrier) and shared -> the owner's memory,
// the load of one piece in flight while the previous piece is stored.  192 KiB are in flight per SM.
// Measured on 2 and 4 GPUs with 4096 tokens each (400 MB of rows per GPU): as one block per row with 16-byte
// stores the push filled every SM first and the GEMMs waited for it (4 GPUs: shared-expert phase 1.13 ms =
// push 0.5 + GEMMs 0.62); as one small block per SM, sized to fit beside a GEMM CTA, it was no better
// (1.14 ms); on 16 SMs of its own it took 0.6 ms by itself, however the bytes were moved: an SM copies
// ~47 GB/s, and half (2 GPUs) or a quarter (4) of the rows stay on the GPU and take SM time all the same.
constexpr int kPushWarps = 32, kPushThreads = kPushWarps * 32;
constexpr int kPushChunk = 3072;                                  // bytes per staged piece
constexpr int kPushSmem = kPushWarps * 2 * kPushChunk + kPushWarps * 2 * 8;
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__global__ void __launch_bounds__(kPushThreads, 1)
ep_dispatch_push_kernel(CommPeers pr, int rank, int world, const __half* __restrict__ xh,
                        const int* __restrict__ sorted_tok, const int* __restrict__ row_dest, int H, int P,
                        const int* __restrict__ plan, size_t own_recv_off, long long wait_cycles, int wave) {
    extern __shared__ __align__(128) uint8_t push_smem[];
    if (!plan[0] || (threadIdx.x & 31)) return;                  // one lane per warp drives the copy unit
    const int warp = threadIdx.x >> 5;
    uint8_t* stage = push_smem + (size_t)warp * 2 * kPushChunk;
    uint64_t* bars = reinterpret_cast<uint64_t*>(push_smem + (size_t)kPushWarps * 2 * kPushChunk) + warp * 2;
    mbar_init(&bars[0], 1); mbar_init(&bars[1], 1);
    fence_barrier_init();
    const int warps = (int)gridDim.x * kPushWarps;
    const int row_bytes = H * 2;
    // cursor over the pieces this warp sends: positions k, k + warps, ... of a row order that deals the sorted
    // rows out over `world` equal runs (k -> (k % world) * (P / world) + k / world; the last P % world rows
    // as they are), each row cut into pieces of kPushChunk bytes.  In sorted order all warps would send the
    // rows of one owner after those of another - the local rows (SM-bound) in one phase, the remote rows
    // (link-bound) in the next, 0.15 + 0.3 ms instead of the larger of the two.
    int k = (int)blockIdx.x * kPushWarps + warp;
    const int run = P / world, dealt = run * world;
    int off = 0;
    const uint8_t* src_row = nullptr;
    uint8_t* dst_row = nullptr;
    auto seek = [&]() -> bool {                                   // first position at or after k whose row is sent
        for (; k < P; k += warps) {
            const int r = k < dealt ? (k % world) * run + k / world : k;
            const int dest = row_dest[r];
            if (dest < 0) continue;                               // beyond what the owner can receive
            if (wave >= 0 && ((dest >> kDestWaveBit) & 1) != wave) continue;   // the other wave's launch sends it
            const int owner = (dest >> kDestShift) & 7;
            const size_t recv_off = owner == rank ? own_recv_off : ((size_t)plan[4 + 4 * owner + 0] << 10);
            src_row = reinterpret_cast<const uint8_t*>(xh) + (size_t)sorted_tok[r] * row_bytes;
            dst_row = pr.base[owner] + kCtrlBytes + recv_off + (size_t)(dest & ((1 << kDestShift) - 1)) * row_bytes;
            off = 0;
            return true;
        }
        return false;
    };
    uint8_t* dstp[2];
    uint32_t nbytes[2], ph[2] = {0u, 0u};
    auto load = [&](int b) {                                      // the piece under the cursor into buffer b; cursor on
        const uint32_t len = (uint32_t)min(kPushChunk, row_bytes - off);
        dstp[b] = dst_row + off; nbytes[b] = len;
        mbar_arrive_expect_tx(&bars[b], len);
        bulk_g2s(stage + b * kPushChunk, src_row + off, len, &bars[b]);
        off += (int)len;
        if (off >= row_bytes) { k += warps; return seek(); }
        return true;
    };
    if (!seek()) return;
    bool more = load(0);
    for (int i = 0;; ++i) {
        const int b = i & 1;
        const bool had_more = more;
        if (had_more) {
            // buffer b ^ 1 was last read by the store of piece i - 1, the only store that can be pending here
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            more = load(b ^ 1);
        }
        if (!mbar_wait(&bars[b], ph[b], wait_cycles)) {           // a local copy that never lands: give up, say so
            atomicCAS(ctrl_of(pr, rank) + kStatusWord, 0, GSB_ERR_TIMEOUT);
            break;
        }
        ph[b] ^= 1u;
        bulk_s2g(dstp[b], stage + b * kPushChunk, nbytes[b]);
        if (!had_more) break;
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // every piece this lane sent has been written
}

int comm_launch_signal(gsb_comm* c, int ch, cudaStream_t s) {
    signal_kernel<<<1, 32, 0, s>>>(c->peers, c->rank, c->world, ch, (int)c->seq[ch]);
    return launch_status();
}
// signal and wait in one launch (the return exchange: nothing lies between the two)
int comm_launch_signal_wait(gsb_comm* c, int ch, cudaStream_t s) {
    signal_wait_kernel<<<1, 32, 0, s>>>(c->peers, c->rank, c->world, ch, (int)c->seq[ch], c->wait_cycles);
    return launch_status();
}
// back = 0: the channel's newest sequence number; 1: the one before it (the first of two waves)
int comm_launch_wait(gsb_comm* c, int ch, cudaStream_t s, int back) {
    wait_kernel<<<1, 32, 0, s>>>(c->peers, c->rank, c->world, ch, (int)c->seq[ch] - back, c->wait_cycles);
    return launch_status();
}

// Count exchange and plan: everything that decides where rows go.
int comm_ep_plan(gsb_comm* c, const EpExchange& e, cudaStream_t s, const EpRouting* r) {
    if (e.E > kMaxExperts || e.E % c->world) return GSB_ERR_UNSUPPORTED;
    if ((e.recv_off & 1023) || (e.ybuf_off & 1023) || (e.recv_off >> 10) > 0x7fffffff || (e.ybuf_off >> 10) > 0x7fffffff)
        return GSB_ERR_INVALID_ARG;
    const int seq_c = (int)++c->seq[kChCounts];
    if (r) {   // routing not done yet: top-k + dispatch + counts in one launch (comm_ep_route_fusable)
        const size_t smem = (size_t)(kDispWarps * e.E + 1024) * sizeof(int);
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(ep_route_post_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return GSB_ERR_CUDA;
        ep_route_post_kernel<<<1, kDispWarps * 32, smem, s>>>(c->peers, c->rank, c->world, r->scores, r->e_bias, r->n, e.E,
                                                              r->topk, r->norm_topk, r->routed_scale, r->ids, r->w,
                                                              r->expert_offsets, r->sorted_tok, r->sorted_row, r->slot_pos,
                                                              r->status, seq_c, (int)(e.recv_off >> 10), e.recv_cap,
                                                              (int)(e.ybuf_off >> 10));
    } else {
        ep_post_counts_kernel<<<1, 256, 0, s>>>(c->peers, c->rank, c->world, e.expert_offsets, e.E, seq_c,
                                                (int)(e.recv_off >> 10), e.recv_cap, (int)(e.ybuf_off >> 10));
    }
    ep_plan_kernel<<<1, 1024, 0, s>>>(c->peers, c->rank, c->world, e.E, seq_c, e.recv_offsets, e.send_base, e.ydst,
                                      e.H, e.y_elem_bytes, e.recv_cap, (int)(e.ybuf_off >> 10), e.plan, c->wait_cycles,
                                      e.expert_offsets, e.sorted_expert);
    return launch_status();
}
bool comm_ep_route_fusable(int n, int E) { return n > 0 && n <= kRouteTokens && E <= 1024; }

// SMs the push of P rows keeps to itself while it runs (a warp per row in flight).  An SM copies ~47 GB/s
// (measured, plain stores and bulk copies alike, local or remote), NVLink takes ~670 GB/s per sender, and
// (world - 1) / world of the rows are remote: with more ranks the link bounds the push and fewer SMs keep up
// with it; with two ranks half the rows stay local and it pays to give the copy more SMs.
int comm_ep_push_sms(int P, int world) {
    const int blocks = world <= 2 ? 28 : (world <= 4 ? 20 : 16);
    const int want = (P + kPushWarps - 1) / kPushWarps;
    return want < blocks ? want : blocks;
}

int comm_ep_push(gsb_comm* c, const EpExchange& e, cudaStream_t s, int waves) {
    if (e.P > 0 &&
        cudaFuncSetAttribute(ep_dispatch_push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPushSmem) != cudaSuccess)
        return GSB_ERR_CUDA;
    for (int wv = 0; wv < (waves == 2 ? 2 : 1); ++wv) {
        if (e.P > 0)
            ep_dispatch_push_kernel<<<comm_ep_push_sms(e.P, c->world), kPushThreads, kPushSmem, s>>>(
                c->peers, c->rank, c->world, e.xh, e.sorted_tok, e.sorted_expert, e.H, e.P, e.plan, e.recv_off, c->wait_cycles,
                waves == 2 ? wv : -1);
        ++c->seq[kChDispatch];
        const int st = comm_launch_signal(c, kChDispatch, s);
        if (st) return st;
    }
    return GSB_OK;
}

}  // namespace gsb

using namespace gsb;

extern "C" {

// One-shot while a rank sends at most ~4 MB ((world - 1) copies of the message): measured for 64 x 6144 floats,
// device time one-shot / two-shot: 2 ranks 14.0 / 18.7 us, 4 ranks 21.1 / 21.1, 8 ranks 38.6 / 23.3.
static int64_t default_one_shot_limit(int world) {
    return ((int64_t)1 << 20) * world / (world > 1 ? world - 1 : 1);
}

int gsb_comm_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

int gsb_comm_create(int rank, int world, size_t heap_bytes, void* out_handle, gsb_comm** out) {
    if (!out || !out_handle || rank < 0 || world < 1 || rank >= world) return GSB_ERR_INVALID_ARG;
    if (world > kMaxWorld) return GSB_ERR_UNSUPPORTED;
    gsb_comm* c = new (std::nothrow) gsb_comm();
    if (!c) return GSB_ERR_CUDA;
    c->rank = rank; c->world = world;
    c->ar_one_shot_limit = default_one_shot_limit(world);
    c->heap_bytes = (heap_bytes + 255) / 256 * 256;
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    c->sm_count = sms > 0 ? sms : 148;
    if (cudaMalloc(reinterpret_cast<void**>(&c->local), kCtrlBytes + c->heap_bytes) != cudaSuccess) { delete c; return GSB_ERR_CUDA; }
    // all of it zero before any peer can reach it: the flag-in-data all-reduce takes a word for valid when its
    // sequence numbers match, and those start at 1
    if (cudaMemset(c->local, 0, kCtrlBytes + c->heap_bytes) != cudaSuccess) { cudaFree(c->local); delete c; return GSB_ERR_CUDA; }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, c->local) != cudaSuccess) { cudaFree(c->local); delete c; return GSB_ERR_CUDA; }
    memcpy(out_handle, &h, sizeof(h));
    c->peers.base[rank] = c->local;
    *out = c;
    return GSB_OK;
}

int gsb_comm_open(gsb_comm* c, const void* handles) {
    if (!c || !handles || c->loopback) return GSB_ERR_INVALID_ARG;
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

int gsb_comm_open_loopback(gsb_comm* c) {
    if (!c) return GSB_ERR_INVALID_ARG;
    for (int r = 0; r < c->world; ++r)
        if (c->opened[r]) return GSB_ERR_INVALID_ARG;
    for (int r = 0; r < c->world; ++r) c->peers.base[r] = c->local;
    c->loopback = true;
    return GSB_OK;
}

int gsb_comm_set_wait_cycles(gsb_comm* c, long long cycles) {
    if (!c || cycles < 0) return GSB_ERR_INVALID_ARG;
    c->wait_cycles = cycles ? cycles : kCommWaitCycles;
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
    return comm_launch_signal_wait(c, kChBarrier, s);
}

// The first bytes of the heap are the all-reduce staging: two parities of two areas of
// (max_count + kArPad) floats; callers that also use the heap for expert parallelism place their
// buffers after gsb_comm_allreduce_reserve() bytes.
// staging of the two flag forms, then the flag-in-data area: two parities of world slots of 16-byte words
size_t gsb_comm_allreduce_reserve_bytes(int world, int64_t max_count) {
    if (world < 1 || max_count < 0) return 0;
    const size_t fl = ((size_t)max_count + 3) / 4 * 4;
    const size_t ll_words = (fl < (size_t)kArLLFloats ? fl : (size_t)kArLLFloats) / 2;
    return 4 * (fl + kArPad) * sizeof(float) + 2 * (size_t)world * ll_words * 16;
}

size_t gsb_comm_allreduce_reserve(gsb_comm* c, int64_t max_count) {
    if (!c || max_count < 0) return 0;
    const size_t fl = ((size_t)max_count + 3) / 4 * 4;
    c->ar_stage_floats = fl;
    c->ar_ll_words = (fl < (size_t)kArLLFloats ? fl : (size_t)kArLLFloats) / 2;
    return gsb_comm_allreduce_reserve_bytes(c->world, max_count);
}

int gsb_comm_allreduce_ll_limit(gsb_comm* c, int64_t floats) {
    if (!c || floats < 0) return GSB_ERR_INVALID_ARG;
    c->ar_ll_limit = floats ? floats : (int64_t)kArLLFloats;
    return GSB_OK;
}

int gsb_comm_allreduce_one_shot_limit(gsb_comm* c, int64_t total_floats) {
    if (!c || total_floats < 0) return GSB_ERR_INVALID_ARG;
    c->ar_one_shot_limit = total_floats ? total_floats : default_one_shot_limit(c->world);
    return GSB_OK;
}

int gsb_comm_allreduce_sum(gsb_comm* c, float* data, int64_t count, void* stream) {
    if (!c || count < 0 || (count > 0 && !data)) return GSB_ERR_INVALID_ARG;
    if (c->world == 1 || count == 0) return GSB_OK;
    if (count % 4 || (reinterpret_cast<uintptr_t>(data) & 15)) return GSB_ERR_INVALID_ARG;
    if ((size_t)count > c->ar_stage_floats) return GSB_ERR_TOO_LARGE;
    const size_t area = c->ar_stage_floats + kArPad;
    const size_t ll_bytes = 2 * (size_t)c->world * c->ar_ll_words * 16;
    if (4 * area * sizeof(float) + ll_bytes > c->heap_bytes) return GSB_ERR_WORKSPACE;
    ArArgs a{};
    a.pr = c->peers; a.rank = c->rank; a.world = c->world; a.data = data; a.count4 = count / 4;
    if (count <= c->ar_ll_limit && (size_t)count / 2 <= c->ar_ll_words) {
        const unsigned lseq = ++c->ar_ll_seq;
        a.area_bytes = c->ar_ll_words * 16;                                   // one source's slot
        a.stage_off = kCtrlBytes + 4 * area * sizeof(float) + (size_t)(lseq & 1u) * c->world * a.area_bytes;
        a.seq = (int)lseq; a.wait_cycles = c->wait_cycles;
        int64_t lb = (a.count4 * 2 + 255) / 256;
        if (lb > c->sm_count) lb = c->sm_count;
        allreduce_ll_kernel<<<(unsigned)lb, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
        return launch_status();
    }
    const unsigned seq = ++c->seq[kChAllReduce];
    a.area_bytes = area * sizeof(float);
    a.stage_off = kCtrlBytes + (size_t)(seq & 1u) * 2 * a.area_bytes;
    a.seq = (int)seq; a.wait_cycles = c->wait_cycles;
    // one-shot while it is allowed and the world slots of `count` floats fit the two areas
    a.two_shot = (count * c->world > c->ar_one_shot_limit || (size_t)count * c->world > 2 * c->ar_stage_floats) ? 1 : 0;
    int64_t blocks = (a.count4 + 255) / 256;
    if (a.two_shot) blocks = ((a.count4 + c->world - 1) / c->world + 255) / 256 * 1;   // one 256-thread pass over a slice part
    if (a.two_shot) blocks = blocks * 2;                                                // two parts per slice pass: more stores in flight
    const int64_t cap = c->sm_count < kMaxArBlocks ? c->sm_count : kMaxArBlocks;       // every block resident: blocks wait on peers
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    allreduce_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(a);
    return launch_status();
}

int gsb_comm_allreduce_sum_n(gsb_comm* c, float* data, int64_t count, int n, void* stream) {
    for (int i = 0; i < n; ++i) {
        const int st = gsb_comm_allreduce_sum(c, data, count, stream);
        if (st) return st;
    }
    return GSB_OK;
}

}  // extern "C"

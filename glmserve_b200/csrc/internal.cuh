// Private definitions shared by the translation units of the library (not installed).
#pragma once
#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

constexpr int kMaxWorld = 8;
constexpr int kArLLFloats = 65536;   // largest all-reduce message of the flag-in-data form (256 KiB)
constexpr size_t kCtrlBytes = 1 << 20;          // control area at the start of the heap
constexpr long long kCommWaitCycles = 4000000000LL;

// Control area layout (ints): every flag is written by exactly one peer.
//   [kFlagBase + ch*kMaxWorld + src]   sequence flag of channel ch from rank src
//   [kCntBase + src*kMaxExperts + e]   expert counts posted by rank src (expert parallel)
enum { kChAllReduce = 0, kChAllReduce2 = 1, kChCounts = 2, kChDispatch = 3, kChCombine = 4, kChBarrier = 5, kNumCh = 8 };
constexpr int kFlagBase = 64;
constexpr int kMaxExperts = 1024;
constexpr int kCntBase = 1024;
constexpr int kStatusWord = 0;                  // ctrl[0]: sticky GSB_ERR_TIMEOUT
//   [kMetaBase + src*8 + i]            expert-parallel layout posted by rank src: {receive buffer offset and
//                                      per-slot row buffer offset in KiB from the heap start, receive capacity}
//   [kBlkFlagBase + (phase*kMaxWorld + src)*kMaxArBlocks + b]   all-reduce: block b of rank src finished `phase`
constexpr int kMetaBase = 12288;
constexpr int kMaxArBlocks = 256;
constexpr int kBlkFlagBase = 16384;
static_assert(kCntBase + kMaxWorld * kMaxExperts <= kMetaBase && kMetaBase + kMaxWorld * 8 <= kBlkFlagBase &&
              (kBlkFlagBase + 2 * kMaxWorld * kMaxArBlocks) * sizeof(int) <= kCtrlBytes, "control area layout");
constexpr size_t kArPad = 64;                   // floats of slack per staging area (slices are rounded up)

struct CommPeers { uint8_t* base[kMaxWorld]; };

}  // namespace gsb

struct gsb_comm {
    int rank = 0, world = 1;
    size_t heap_bytes = 0;                      // payload bytes after the control area
    uint8_t* local = nullptr;
    gsb::CommPeers peers{};
    bool opened[gsb::kMaxWorld] = {};
    unsigned seq[gsb::kNumCh] = {};
    size_t ar_stage_floats = 0;                 // largest message the all-reduce staging was reserved for
    int64_t ar_one_shot_limit = 1 << 18;        // count * world up to which the one-shot form is used
    size_t ar_ll_words = 0;                     // 16-byte words per source and parity of the flag-in-data area (0: none)
    int64_t ar_ll_limit = gsb::kArLLFloats;     // messages up to this many floats take the flag-in-data form
    unsigned ar_ll_seq = 0;
    long long wait_cycles = gsb::kCommWaitCycles;  // budget of every device-side wait (SM clocks)
    bool loopback = false;                      // every peer slot maps this rank's own heap (single-process tests)
    int sm_count = 148;
};


struct gsb_moe_layer {
    gsb_moe_config cfg;
    bool tiles_ok;       // shapes fit the tile-stream kernels and prepacked weights are given
    int sm_count;
    // stage profiler (counterpart of StageProf, src/model_gpu.cpp:328-388 of the reference)
    cudaEvent_t* prof_ev = nullptr;   // [prof_sets][GSB_N_STAGES + 1]
    int prof_sets = 0;
    int prof_used = 0;
    // expert-parallel forward: a side stream for the dispatch push, fork/join events (created on first use)
    cudaStream_t ep_side = nullptr;
    cudaEvent_t ep_fork = nullptr, ep_join = nullptr;
};

namespace gsb {
int comm_launch_signal(gsb_comm* c, int ch, cudaStream_t s);
int comm_launch_wait(gsb_comm* c, int ch, cudaStream_t s, int back = 0);
int comm_launch_signal_wait(gsb_comm* c, int ch, cudaStream_t s);
struct EpExchange {
    const __half* xh;              // this rank's tokens [n, H] as fp16, in the feature order the receiving kernels
                                   // read (natural for the tcgen05 path, fragment order for the split-K path)
    const int* expert_offsets;     // local dispatch [E + 1]
    const int* sorted_tok;         // [P]
    int P, E, H;
    int* sorted_expert;            // scratch [P]: destination (owner, row) of every sorted row
    int* recv_offsets;             // out [El + 1]
    int* send_base;                // out [E]
    void** ydst;                   // out [recv_cap]
    int* plan;                     // out [4 + 4 * kMaxWorld]: {ok, rows received, 0, 0} then every rank's layout
                                   // {receive offset KiB, capacity, row buffer offset KiB, 0}
    size_t recv_off, ybuf_off;     // byte offsets from the heap start (multiples of 1 KiB) of this rank's buffers
    int y_elem_bytes;              // element size of the per-slot output rows (2 = fp16, 4 = fp32)
    int recv_cap;
};
// Routing inputs and outputs for the fused form of comm_ep_plan (decode-sized batches): sigmoid scores in,
// ids / weights / dispatch permutation out, status words zeroed.
struct EpRouting {
    const float* scores; const float* e_bias;
    int n, topk, norm_topk; float routed_scale;
    int* ids; float* w; int* expert_offsets; int* sorted_tok; int* sorted_row; int* slot_pos; int* status;
};
int comm_ep_plan(gsb_comm* c, const EpExchange& e, cudaStream_t s, const EpRouting* routing = nullptr);
bool comm_ep_route_fusable(int n, int E);
// waves = 2: the rows for the first half of every owner's experts, a signal, then the rest and a second signal
int comm_ep_push(gsb_comm* c, const EpExchange& e, cudaStream_t s, int waves = 1);
int comm_ep_push_sms(int P, int world);   // SMs that push occupies by itself while it runs
}  // namespace gsb

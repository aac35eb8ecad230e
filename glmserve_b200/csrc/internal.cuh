// Private definitions shared by the translation units of the library (not installed).
#pragma once
#include "common.cuh"
#include "launchers.cuh"

namespace gsb {

constexpr int kMaxWorld = 8;
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
constexpr int kArriveCounter = 8;               // ctrl[8..]: block arrival counters (local use)

struct CommPeers { uint8_t* base[kMaxWorld]; };

}  // namespace gsb

struct gsb_comm {
    int rank = 0, world = 1;
    size_t heap_bytes = 0;                      // payload bytes after the control area
    uint8_t* local = nullptr;
    gsb::CommPeers peers{};
    bool opened[gsb::kMaxWorld] = {};
    unsigned seq[gsb::kNumCh] = {};
    size_t ar_stage_floats = 0;                 // capacity of the all-reduce staging (per parity)
    int64_t ar_one_shot_limit = 1 << 21;        // count * world up to which every rank pulls everything
};


struct gsb_moe_layer {
    gsb_moe_config cfg;
    bool tiles_ok;       // shapes fit the tile-stream kernels and prepacked weights are given
    int sm_count;
    // stage profiler (counterpart of StageProf, src/model_gpu.cpp:328-388 of the reference)
    cudaEvent_t* prof_ev = nullptr;   // [prof_sets][GSB_N_STAGES + 1]
    int prof_sets = 0;
    int prof_used = 0;
};

namespace gsb {
int comm_launch_signal(gsb_comm* c, int ch, cudaStream_t s);
int comm_launch_wait(gsb_comm* c, int ch, cudaStream_t s);
int comm_ep_exchange(gsb_comm* c, const __nv_bfloat16* x, const int* expert_offsets, const int* sorted_tok,
                     int P, int E, int H, int* sorted_expert, int* recv_offsets, int* send_base, void** ydst,
                     size_t ybuf_off, int y_elem_bytes, size_t recv_off, int recv_cap, int* recv_total,
                     cudaStream_t s);
}  // namespace gsb

// Host-side work decomposition shared by the decode kernels.
#pragma once

#include <algorithm>
#include <vector>

#include "common.cuh"

namespace pkv {

// Segments whose descriptors travel inside the kernel parameter block of one launch.
constexpr int kMaxInlineSegs = 24;

// Device-visible image of a pkv_segment_t plus its share of the split-K work list.
struct SegDev {
    const uint8_t* kp;
    const __half* ks;
    const __half* km;
    const uint8_t* vp;
    const __half* vs;
    const __half* vm;
    long long S;
    long long head_stride;
    long long split_len;  // tokens per work item
    long long k_pitch;    // bytes between channel rows of kp (KIVI layout)
    long long km_pitch;   // elements between rows of ks / km (KIVI layout)
    int kind, kbits, vbits, kgs, vgs;
    int work_begin;  // index of the segment's first work item
    int n_splits;    // work items of this segment
    int key_tma;     // 1 + index of this segment's key tensor maps in the launch parameters, 0 = none
    int fresh;       // the kernel launched just before may have written the segment: read it only after the
                     // stream dependency is resolved
    int slot_tokens, slot_valid;  // KIVI: only the first slot_valid tokens of every slot_tokens count (0 = all)
    long long v_head_tokens;      // KIVI: token rows between KV heads of the value arrays
    const int* len_dev;           // optional: min(S, *len_dev) tokens count, read at run time; S is the capacity
};

// Segments are routed to one of two kernels: the tensor-core kernel (`fast`, split_len counts
// tiles) or the layout-generic kernel (`generic`, split_len counts tokens).  Work items are
// numbered fast first, generic after; work_begin is relative to the start of each list.
struct DecodePlan {
    std::vector<SegDev> fast;
    std::vector<int> fast_index;  // position of each `fast` entry in the caller's segment array
    std::vector<SegDev> generic;
    int fast_work = 0;
    int generic_work = 0;
    int total_work() const { return fast_work + generic_work; }
};

// Where the split-K launches of one call left their partials: pm, pl [n][Hq], pacc [n][Hq][hd].
struct SplitKParts {
    size_t n;
    float* pm;
    float* pl;
    float* pacc;
};

int run_splitk(const void* q, const pkv_segment_t* segs, int n_segs, int num_q_heads, int num_kv_heads,
               int head_dim, float sm_scale, int sm_count, void* workspace, size_t workspace_bytes,
               cudaStream_t stream, SplitKParts* parts);

DecodePlan plan_decode(const pkv_segment_t* segs, int n_segs, int Hq, int Hkv, int hd, int sm_count);

}  // namespace pkv

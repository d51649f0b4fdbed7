// Sequence-sharded decode: split-K over this GPU's shard, then ONE kernel that merges the local partials,
// pushes the result into every peer's memory over NVLink, waits for the peers' pushes and merges those.
//
// The reference is single-GPU; the algebra is its split merge (attention_triton.py:257-266, 300-307) applied
// across GPUs.  Each rank owns an exchange buffer in its own memory that the peers map through CUDA IPC:
//
//   inbox  [2][world][Hq][hd + 2] x {float value, uint32 epoch}   one row per (parity, source rank, head):
//                                                                 acc[hd], m, l
//   epoch  [Hq]  uint32   calls completed by this rank, per head
//   status [1]   uint32   1 after a wait ran out
//
// Every element travels as ONE 8-byte store that carries its own epoch, so no flag, fence or second round trip
// is needed: a reader polls the element itself until the epoch matches (8-byte stores arrive whole).
// CTA h of rank r: merge the local split-K partials of head h; store row h of slot [e & 1][r] into every
// rank's inbox (plain remote stores); poll its OWN inbox rows [e & 1][*][h] (bounded: after `spin_limit` polls
// the status word is set, the output row is NaN and the kernel returns); merge the `world` rows; write
// out[h].  Nothing is ever read from a peer.  Epochs live in device memory so that a CUDA graph replays
// correctly.  Two parities suffice: a rank can be at most one call ahead of another, because call e + 1
// cannot finish before every rank has pushed e + 1, which each does only after it has finished reading call e.
#include <string.h>

#include <vector>

#include "common.cuh"
#include "decode_plan.h"
#include "merge.cuh"

namespace pkv {
namespace {

constexpr int kMaxWorld = 16;
constexpr size_t kHandleBytes = 64;
static_assert(sizeof(cudaIpcMemHandle_t) == kHandleBytes, "CUDA IPC handle size");

struct ExchangeLayout {
    size_t slot_words;  // Hq * (hd + 2) elements of 8 bytes per (parity, source rank)
    size_t off_epoch, off_status, bytes;
};

ExchangeLayout layout_of(int world, int Hq, int hd) {
    ExchangeLayout L;
    L.slot_words = (size_t)Hq * (hd + 2);
    L.off_epoch = 2 * (size_t)world * L.slot_words * sizeof(uint2);
    L.off_status = L.off_epoch + (size_t)Hq * sizeof(uint32_t);
    L.bytes = (L.off_status + sizeof(uint32_t) + 255) & ~(size_t)255;
    return L;
}

struct ExchangeArgs {
    char* peer[kMaxWorld];  // exchange buffers of all ranks as mapped here; peer[rank] is the local one
    int world, rank, Hq, hd;
    size_t slot_words, off_epoch, off_status;
    unsigned spin_limit;  // most polling passes of one wait
    unsigned wait_us;     // most microseconds of one wait
};

// One element = one aligned 8-byte word {value, epoch}, moved by ONE 64-bit access: single-copy atomic, so a
// reader sees either the old pair or the new pair, never a new epoch with an old value.
__device__ __forceinline__ void st_word(uint2* p, float v, uint32_t e) {
    const unsigned long long w = ((unsigned long long)e << 32) | __float_as_uint(v);
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2((unsigned)w, (unsigned)(w >> 32));
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__global__ void __launch_bounds__(kMergeThreads)
merge_exchange_kernel(const float* __restrict__ pm, const float* __restrict__ pl, const float* __restrict__ pacc,
                      int n_parts, const __grid_constant__ ExchangeArgs x, __half* __restrict__ out) {
    const int h = blockIdx.x, tid = threadIdx.x;
    const int Hq = x.Hq, hd = x.hd;
    cudaGridDependencySynchronize();  // the split-K kernel of this call
    cudaTriggerProgrammaticLaunchCompletion();
    char* local = x.peer[x.rank];
    uint32_t* status = reinterpret_cast<uint32_t*>(local + x.off_status);
    // A wait that ran out once means the ranks are out of step for good: every later call returns at once
    // (NaN rows, no push, no wait) instead of spending its whole budget again.
    if (*reinterpret_cast<volatile uint32_t*>(status) != 0u) {
        if (tid < hd) out[(size_t)h * hd + tid] = __float2half_rn(nanf(""));
        return;
    }
    uint32_t* epoch = reinterpret_cast<uint32_t*>(local + x.off_epoch);
    const uint32_t e = epoch[h] + 1;
    const size_t par = e & 1u;

    // 1. this rank's partial of head h: A in threads tid < hd, (M, L) in every thread
    float M, L, A;
    merge_reduce<false>(pm, pl, pacc, n_parts, (size_t)Hq, (size_t)Hq * hd, hd, h, M, L, A);

    // 2. push row h of slot [par][rank] into every rank's inbox
    const size_t row = ((par * x.world + x.rank) * Hq + h) * (size_t)(hd + 2);
    for (int r = 0; r < x.world; ++r) {
        uint2* dst = reinterpret_cast<uint2*>(x.peer[r]) + row;
        if (tid < hd) st_word(dst + tid, A, e);
        if (tid < 2) st_word(dst + hd + tid, tid == 0 ? M : L, e);
    }

    // 3. collect row h of every rank from the local inbox.  The three words a thread needs from a rank (m, l and
    //    its own dim of acc) are polled together, four ranks per pass: one round of independent loads per pass
    //    instead of one round trip per word.  The wait is bounded twice: by a number of passes and by the clock.
    const uint2* in = reinterpret_cast<const uint2*>(local) + (par * x.world * Hq + h) * (size_t)(hd + 2);
    const size_t rank_stride = (size_t)Hq * (hd + 2);
    float mr[kMaxWorld], lr[kMaxWorld], ar[kMaxWorld];
    const bool has_dim = tid < hd;
    unsigned pending = x.world >= 32 ? 0xffffffffu : ((1u << x.world) - 1u);
    unsigned polls = 0;
    bool ok = true;
    const unsigned long long deadline = global_ns() + (unsigned long long)x.wait_us * 1000ull;
    while (pending) {
#pragma unroll 1
        for (int r0 = 0; r0 < x.world; r0 += 4) {
            uint2 wm[4], wl[4], wa[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = r0 + k;
                wm[k] = wl[k] = wa[k] = make_uint2(0u, e);
                if (r < x.world && (pending >> r & 1u)) {
                    const uint2* src = in + r * rank_stride;
                    wm[k] = ld_word(src + hd);
                    wl[k] = ld_word(src + hd + 1);
                    if (has_dim) wa[k] = ld_word(src + tid);
                }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = r0 + k;
                if (r < x.world && (pending >> r & 1u) && wm[k].y == e && wl[k].y == e && wa[k].y == e) {
                    mr[r] = __uint_as_float(wm[k].x);
                    lr[r] = __uint_as_float(wl[k].x);
                    ar[r] = __uint_as_float(wa[k].x);
                    pending &= ~(1u << r);
                }
            }
        }
        if (pending) {
            if (++polls >= x.spin_limit || ((polls & 15u) == 0u && global_ns() > deadline)) {
                ok = false;
                break;
            }
            if (polls > 32) __nanosleep(polls < 512 ? 32 : 256);
        }
    }
    // a thread that gave up makes the whole CTA give up: the row is either complete or NaN
    ok = __syncthreads_and(ok);
    if (ok) {
        // merge in rank order (products and sums rounded separately, as the split merge does, so that both give
        // the same bits)
        float mx = -INFINITY;
#pragma unroll 1
        for (int r = 0; r < x.world; ++r) mx = fmaxf(mx, mr[r]);
        float acc = 0.f, den = 0.f;
#pragma unroll 1
        for (int r = 0; r < x.world; ++r) {
            const float w = expf(mr[r] - mx);  // -inf -> 0
            acc = __fadd_rn(acc, __fmul_rn(w, ar[r]));
            den = __fadd_rn(den, __fmul_rn(w, lr[r]));
        }
        if (tid < hd) out[(size_t)h * hd + tid] = __float2half_rn(acc / den);
    } else {
        if (tid == 0) atomicOr(status, 1u);
        if (tid < hd) out[(size_t)h * hd + tid] = __float2half_rn(nanf(""));
    }
    __syncthreads();  // nobody still reads epoch[h]
    if (tid == 0) epoch[h] = e;
}

}  // namespace
}  // namespace pkv

using namespace pkv;

struct pkv_exchange {
    int world, rank, Hq, hd, device;
    ExchangeLayout layout;
    char* local;
    char* peer[kMaxWorld];
    bool connected;
    unsigned spin_limit;
    unsigned wait_us;
};

extern "C" {

int pkv_exchange_create(int world, int rank, int num_q_heads, int head_dim, pkv_exchange_t** ex, void* handle_out) {
    if (!ex || !handle_out) return PKV_E_NULL;
    if (world <= 0 || rank < 0 || rank >= world || num_q_heads <= 0 || head_dim <= 0 || head_dim % 4) return PKV_E_SHAPE;
    if (world > kMaxWorld || head_dim > 256) return PKV_E_LIMIT;
    pkv_exchange* e = new pkv_exchange();
    e->world = world;
    e->rank = rank;
    e->Hq = num_q_heads;
    e->hd = head_dim;
    e->layout = layout_of(world, num_q_heads, head_dim);
    e->connected = false;
    e->spin_limit = 1u << 21;
    e->wait_us = 250000;  // a rank that is a quarter of a second late is out of step, not slow
    for (int r = 0; r < kMaxWorld; ++r) e->peer[r] = nullptr;
    cudaError_t err = cudaGetDevice(&e->device);
    if (err == cudaSuccess) err = cudaMalloc(reinterpret_cast<void**>(&e->local), e->layout.bytes);
    if (err == cudaSuccess) err = cudaMemset(e->local, 0, e->layout.bytes);
    cudaIpcMemHandle_t h;
    if (err == cudaSuccess) err = cudaIpcGetMemHandle(&h, e->local);
    if (err != cudaSuccess) {
        delete e;
        return cuda_fail(err);
    }
    memcpy(handle_out, &h, kHandleBytes);
    e->peer[rank] = e->local;
    *ex = e;
    return PKV_OK;
}

int pkv_exchange_connect(pkv_exchange_t* ex, const void* handles) {
    if (!ex || !handles) return PKV_E_NULL;
    if (ex->connected) return PKV_E_SHAPE;
    for (int r = 0; r < ex->world; ++r) {
        if (r == ex->rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(handles) + (size_t)r * kHandleBytes, kHandleBytes);
        void* p = nullptr;
        PKV_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
        ex->peer[r] = static_cast<char*>(p);
    }
    ex->connected = true;
    return PKV_OK;
}

int pkv_exchange_connect_loopback(pkv_exchange_t* ex) {
    if (!ex) return PKV_E_NULL;
    if (ex->connected) return PKV_E_SHAPE;
    for (int r = 0; r < ex->world; ++r) ex->peer[r] = ex->local;
    ex->connected = true;
    return PKV_OK;
}

int pkv_exchange_set_spin_limit(pkv_exchange_t* ex, unsigned polls) {
    if (!ex) return PKV_E_NULL;
    if (polls == 0) return PKV_E_SHAPE;
    ex->spin_limit = polls;
    return PKV_OK;
}

int pkv_exchange_set_wait_us(pkv_exchange_t* ex, unsigned microseconds) {
    if (!ex) return PKV_E_NULL;
    if (microseconds == 0) return PKV_E_SHAPE;
    ex->wait_us = microseconds;
    return PKV_OK;
}

int pkv_exchange_status(pkv_exchange_t* ex, int* timed_out) {
    if (!ex || !timed_out) return PKV_E_NULL;
    uint32_t v = 0;
    PKV_CUDA_TRY(cudaMemcpy(&v, ex->local + ex->layout.off_status, sizeof(v), cudaMemcpyDeviceToHost));
    *timed_out = (int)v;
    return PKV_OK;
}

int pkv_exchange_destroy(pkv_exchange_t* ex) {
    if (!ex) return PKV_E_NULL;
    cudaError_t first = cudaSuccess;
    for (int r = 0; r < ex->world; ++r) {
        if (ex->peer[r] && ex->peer[r] != ex->local) {
            const cudaError_t err = cudaIpcCloseMemHandle(ex->peer[r]);
            if (first == cudaSuccess) first = err;
        }
    }
    const cudaError_t err = cudaFree(ex->local);
    if (first == cudaSuccess) first = err;
    delete ex;
    return first == cudaSuccess ? PKV_OK : cuda_fail(first);
}

int pkv_decode_attention_sharded(const void* q, const pkv_segment_t* segs, int n_segs, int num_q_heads,
                                 int num_kv_heads, int head_dim, float sm_scale, int sm_count, void* workspace,
                                 size_t workspace_bytes, pkv_exchange_t* ex, void* out, pkv_stream_t stream) {
    if (!ex || !out) return PKV_E_NULL;
    if (!ex->connected || ex->Hq != num_q_heads || ex->hd != head_dim) return PKV_E_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    SplitKParts parts = {0, nullptr, nullptr, nullptr};
    if (n_segs > 0) {
        const int rc = run_splitk(q, segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_scale, sm_count,
                                  workspace, workspace_bytes, s, &parts);
        if (rc != PKV_OK) return rc;
    }
    ExchangeArgs x;
    for (int r = 0; r < kMaxWorld; ++r) x.peer[r] = ex->peer[r];
    x.world = ex->world;
    x.rank = ex->rank;
    x.Hq = num_q_heads;
    x.hd = head_dim;
    x.slot_words = ex->layout.slot_words;
    x.off_epoch = ex->layout.off_epoch;
    x.off_status = ex->layout.off_status;
    x.spin_limit = ex->spin_limit;
    x.wait_us = ex->wait_us;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)num_q_heads);
    cfg.blockDim = dim3(kMergeThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* cpm = parts.pm;
    const float* cpl = parts.pl;
    const float* cpacc = parts.pacc;
    PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_exchange_kernel, cpm, cpl, cpacc, (int)parts.n, x,
                                    static_cast<__half*>(out)));
    return PKV_OK;
}

}  // extern "C"

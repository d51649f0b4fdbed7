// Three-tier split-K decode attention: host planning, the layout-generic kernel, the merge.
//
// One launch covers every segment of a layer (prompt, prompt extensions, every frozen cold
// segment, the float16 hot buffer): a CTA owns (work item, KV head), where a work item is a
// token range of one segment.  All query heads of the GQA group are served from one read of
// the KV bytes; dequantisation happens in registers and nothing dense is written back.
// Each CTA emits an un-normalised flash partial (m, l, acc) and the merge kernel combines them
// (attention_triton.py:257-266 and :300-307 of the reference define the same algebra).
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "decode_plan.h"
#include "decode_mma.cuh"

namespace pkv {
namespace {

constexpr int GMAX = 8;        // query heads served per CTA pass
constexpr int kThreads = 128;  // threads per CTA of the generic kernel
constexpr int kChunk = 128;    // tokens per inner step (= kThreads)
constexpr int kMaxDimsPerThread = 2;  // head_dim <= 256

struct DecodeArgs {
    const __half* q;
    float* pm;
    float* pl;
    float* pacc;
    int Hq, Hkv, hd, G;
    float sm_scale;
    int n_segs;
    int work_offset;  // global index of this launch's first work item
    SegDev segs[kMaxInlineSegs];
};

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(kThreads)
decode_generic_kernel(const __grid_constant__ DecodeArgs a) {
    extern __shared__ float smem[];
    const int hd = a.hd;
    float* q_s = smem;                    // [GMAX][hd], pre-multiplied by sm_scale
    float* p_s = q_s + GMAX * hd;         // [GMAX][kChunk]
    float* alpha_s = p_s + GMAX * kChunk; // [GMAX]
    float* m_s = alpha_s + GMAX;
    float* l_s = m_s + GMAX;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int w = blockIdx.x, kvh = blockIdx.y, hc = blockIdx.z;

    int si = 0;
    while (si + 1 < a.n_segs && w >= a.segs[si + 1].work_begin) ++si;
    const SegDev& sg = a.segs[si];
    const long long t0 = (long long)(w - sg.work_begin) * sg.split_len;
    const long long t1 = min(sg.S, t0 + sg.split_len);

    const int h0 = kvh * a.G + hc * GMAX;
    const int nh = min(GMAX, a.G - hc * GMAX);
    for (int i = tid; i < GMAX * hd; i += kThreads) {
        const int h = i / hd, d = i % hd;
        q_s[i] = h < nh ? __half2float(a.q[(size_t)(h0 + h) * hd + d]) * a.sm_scale : 0.f;
    }
    if (tid < GMAX) {
        m_s[tid] = -INFINITY;
        l_s[tid] = 0.f;
    }
    float acc[GMAX][kMaxDimsPerThread];
#pragma unroll
    for (int h = 0; h < GMAX; ++h)
#pragma unroll
        for (int k = 0; k < kMaxDimsPerThread; ++k) acc[h][k] = 0.f;
    __syncthreads();

    const int kvpb = 8 / sg.kbits, vvpb = 8 / sg.vbits;
    const long long S = sg.S;

    for (long long c0 = t0; c0 < t1; c0 += kChunk) {
        // ---- phase 1: one token per thread, scores for all heads of the group
        const long long n = c0 + tid;
        float dot[GMAX];
#pragma unroll
        for (int h = 0; h < GMAX; ++h) dot[h] = 0.f;
        if (n < t1) {
            if (sg.kind == PKV_SEG_KIVI) {
                const long long nbK = ceil_div(S, kvpb), ngK = ceil_div(S, sg.kgs);
                const uint8_t* kp = sg.kp + (size_t)kvh * hd * nbK + n / kvpb;
                const __half* ks = sg.ks + (size_t)kvh * hd * ngK + n / sg.kgs;
                const __half* km = sg.km + (size_t)kvh * hd * ngK + n / sg.kgs;
                const unsigned pos = (unsigned)(n % kvpb);
                for (int d = 0; d < hd; ++d) {
                    const float c = (float)extract_code_rt(kp[(size_t)d * nbK], pos, sg.kbits);
                    const float kv = fmaf(c, __half2float(ks[(size_t)d * ngK]), __half2float(km[(size_t)d * ngK]));
#pragma unroll
                    for (int h = 0; h < GMAX; ++h) dot[h] = fmaf(q_s[h * hd + d], kv, dot[h]);
                }
            } else if (sg.kind == PKV_SEG_PER_TOKEN) {
                const long long nbK = ceil_div(hd, kvpb), ngK = ceil_div(hd, sg.kgs);
                const uint8_t* kp = sg.kp + ((size_t)kvh * S + n) * nbK;
                const __half* ks = sg.ks + ((size_t)kvh * S + n) * ngK;
                const __half* km = sg.km + ((size_t)kvh * S + n) * ngK;
                for (int d = 0; d < hd; ++d) {
                    const float c = (float)extract_code_rt(kp[d / kvpb], (unsigned)(d % kvpb), sg.kbits);
                    const float kv = fmaf(c, __half2float(ks[d / sg.kgs]), __half2float(km[d / sg.kgs]));
#pragma unroll
                    for (int h = 0; h < GMAX; ++h) dot[h] = fmaf(q_s[h * hd + d], kv, dot[h]);
                }
            } else {
                const __half* kr = reinterpret_cast<const __half*>(sg.kp) + (size_t)kvh * sg.head_stride + (size_t)n * hd;
                for (int d = 0; d < hd; ++d) {
                    const float kv = __half2float(kr[d]);
#pragma unroll
                    for (int h = 0; h < GMAX; ++h) dot[h] = fmaf(q_s[h * hd + d], kv, dot[h]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < GMAX; ++h) p_s[h * kChunk + tid] = n < t1 ? dot[h] : -INFINITY;
        __syncthreads();

        // ---- phase 2: online softmax bookkeeping, one warp per head
        for (int h = wid; h < nh; h += kThreads / 32) {
            float v[kChunk / 32];
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < kChunk / 32; ++i) {
                v[i] = p_s[h * kChunk + lane + 32 * i];
                mx = fmaxf(mx, v[i]);
            }
            mx = warp_max(mx);
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < kChunk / 32; ++i) {
                const float p = expf(v[i] - m_new);  // -inf -> 0
                p_s[h * kChunk + lane + 32 * i] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = expf(m_old - m_new);  // first chunk: exp(-inf) = 0
                alpha_s[h] = alpha;
                m_s[h] = m_new;
                l_s[h] = l_s[h] * alpha + sum;
            }
        }
        __syncthreads();

        // ---- phase 3: one head_dim column per thread, acc += p * v
        const int nvalid = (int)min((long long)kChunk, t1 - c0);
#pragma unroll
        for (int k = 0; k < kMaxDimsPerThread; ++k) {
            const int d = tid + k * kThreads;
            if (d < hd) {
#pragma unroll
                for (int h = 0; h < GMAX; ++h) acc[h][k] *= alpha_s[h];
                if (sg.kind == PKV_SEG_FP16) {
                    const __half* vr = reinterpret_cast<const __half*>(sg.vp) + (size_t)kvh * sg.head_stride + (size_t)c0 * hd + d;
                    for (int i = 0; i < nvalid; ++i) {
                        const float vv = __half2float(vr[(size_t)i * hd]);
#pragma unroll
                        for (int h = 0; h < GMAX; ++h) acc[h][k] = fmaf(p_s[h * kChunk + i], vv, acc[h][k]);
                    }
                } else {
                    const long long nbV = ceil_div(hd, vvpb), ngV = ceil_div(hd, sg.vgs);
                    const uint8_t* vp = sg.vp + ((size_t)kvh * S + c0) * nbV + d / vvpb;
                    const __half* vs = sg.vs + ((size_t)kvh * S + c0) * ngV + d / sg.vgs;
                    const __half* vm = sg.vm + ((size_t)kvh * S + c0) * ngV + d / sg.vgs;
                    const unsigned pos = (unsigned)(d % vvpb);
                    for (int i = 0; i < nvalid; ++i) {
                        const float c = (float)extract_code_rt(vp[(size_t)i * nbV], pos, sg.vbits);
                        const float vv = fmaf(c, __half2float(vs[(size_t)i * ngV]), __half2float(vm[(size_t)i * ngV]));
#pragma unroll
                        for (int h = 0; h < GMAX; ++h) acc[h][k] = fmaf(p_s[h * kChunk + i], vv, acc[h][k]);
                    }
                }
            }
        }
        __syncthreads();
    }

    const size_t widx = (size_t)(a.work_offset + w);
    if (tid < nh) {
        a.pm[widx * a.Hq + h0 + tid] = m_s[tid];
        a.pl[widx * a.Hq + h0 + tid] = l_s[tid];
    }
#pragma unroll
    for (int k = 0; k < kMaxDimsPerThread; ++k) {
        const int d = tid + k * kThreads;
        if (d < hd) {
#pragma unroll
            for (int h = 0; h < GMAX; ++h)
                if (h < nh) a.pacc[(widx * a.Hq + h0 + h) * hd + d] = acc[h][k];
        }
    }
}

// Log-sum-exp merge of n_parts partials, one query head per CTA of 256 threads.
// Warp w owns parts p = w (mod 8) and lane owns four consecutive dims (float4; head_dim <= 256 means
// up to two float4 per lane), so every load of a thread is independent of the others and of the
// weights: they are all issued before the first use, one memory round trip for the whole merge.
constexpr int kMergeThreads = 256;
constexpr int kMergeMaxInflight = 6;  // parts per thread held in registers at once

__global__ void __launch_bounds__(kMergeThreads)
merge_partials_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                      const float* __restrict__ pacc, int n_parts, int Hq, int hd,
                      __half* __restrict__ out, float* __restrict__ m_out,
                      float* __restrict__ l_out, float* __restrict__ acc_out) {
    __shared__ float red_m[8];
    __shared__ float red_l[8];
    __shared__ __align__(16) float red_acc[8][256];
    const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    // When launched as a programmatic dependent of the split-K kernel this grid may already be resident while
    // that kernel finishes; wait here for its results (a no-op for an ordinary launch).
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();  // the next kernel of the stream may start its own prologue
    const int nvec = hd >> 2;  // float4 per row (hd % 4 == 0 is checked on the host)
    const bool v0 = lane < nvec, v1 = lane + 32 < nvec;

    // Every load of a batch (acc rows, m, l of up to 8 * kMergeMaxInflight parts) is issued before anything
    // is reduced, so a typical merge (a few dozen parts) is one memory round trip.  Batches are combined
    // with a running maximum, like the online softmax itself.
    float run_m = -INFINITY;  // block-wide running max (identical in every thread)
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    float ls = 0.f;
    for (int base = 0; base < n_parts; base += 8 * kMergeMaxInflight) {
        float4 r0[kMergeMaxInflight], r1[kMergeMaxInflight];
        float wm[kMergeMaxInflight], wl[kMergeMaxInflight];
        float mx = -INFINITY;
#pragma unroll
        for (int u = 0; u < kMergeMaxInflight; ++u) {
            const int p = base + wid + 8 * u;
            r0[u] = r1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            wm[u] = -INFINITY;
            wl[u] = 0.f;
            if (p < n_parts) {
                const float4* row = reinterpret_cast<const float4*>(pacc + ((size_t)p * Hq + h) * hd);
                if (v0) r0[u] = __ldg(row + lane);
                if (v1) r1[u] = __ldg(row + lane + 32);
                wm[u] = __ldg(pm + (size_t)p * Hq + h);
                wl[u] = __ldg(pl + (size_t)p * Hq + h);
            }
        }
#pragma unroll
        for (int u = 0; u < kMergeMaxInflight; ++u) mx = fmaxf(mx, wm[u]);
        __syncthreads();  // red_m is free again
        if (lane == 0) red_m[wid] = mx;
        __syncthreads();
        mx = run_m;
#pragma unroll
        for (int w = 0; w < 8; ++w) mx = fmaxf(mx, red_m[w]);
        const float rescale = expf(run_m - mx);  // first batch: exp(-inf) = 0 on zero accumulators
        run_m = mx;
        ls *= rescale;
        a0.x *= rescale; a0.y *= rescale; a0.z *= rescale; a0.w *= rescale;
        a1.x *= rescale; a1.y *= rescale; a1.z *= rescale; a1.w *= rescale;
#pragma unroll
        for (int u = 0; u < kMergeMaxInflight; ++u) {
            const float wgt = expf(wm[u] - mx);  // -inf -> 0
            ls = fmaf(wgt, wl[u], ls);
            a0.x = fmaf(wgt, r0[u].x, a0.x); a0.y = fmaf(wgt, r0[u].y, a0.y);
            a0.z = fmaf(wgt, r0[u].z, a0.z); a0.w = fmaf(wgt, r0[u].w, a0.w);
            a1.x = fmaf(wgt, r1[u].x, a1.x); a1.y = fmaf(wgt, r1[u].y, a1.y);
            a1.z = fmaf(wgt, r1[u].z, a1.z); a1.w = fmaf(wgt, r1[u].w, a1.w);
        }
    }
    const float mx = run_m;
    if (v0) *reinterpret_cast<float4*>(&red_acc[wid][4 * lane]) = a0;
    if (v1) *reinterpret_cast<float4*>(&red_acc[wid][4 * (lane + 32)]) = a1;
    if (lane == 0) red_l[wid] = ls;  // every lane of a warp holds the same sum
    __syncthreads();
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) L += red_l[w];
    if (tid < hd) {
        float A = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) A += red_acc[w][tid];
        if (out) out[(size_t)h * hd + tid] = __float2half_rn(A / L);
        if (acc_out) acc_out[(size_t)h * hd + tid] = A;
    }
    if (tid == 0) {
        if (m_out) m_out[h] = mx;
        if (l_out) l_out[h] = L;
    }
}

int check_segments(const pkv_segment_t* segs, int n_segs, int Hq, int Hkv, int hd) {
    if (!segs) return PKV_E_NULL;
    if (n_segs <= 0 || n_segs > PKV_MAX_SEGMENTS) return PKV_E_LIMIT;
    if (Hq <= 0 || Hkv <= 0 || hd <= 0 || Hq % Hkv) return PKV_E_SHAPE;
    if (hd > kThreads * kMaxDimsPerThread) return PKV_E_LIMIT;
    if (hd % 4) return PKV_E_LAYOUT;
    for (int i = 0; i < n_segs; ++i) {
        const pkv_segment_t& s = segs[i];
        if (s.seq_len <= 0) return PKV_E_SHAPE;
        if (!s.k_packed || !s.v_packed) return PKV_E_NULL;
        if (s.kind == PKV_SEG_FP16) {
            if (s.head_stride < s.seq_len * hd) return PKV_E_SHAPE;
            continue;
        }
        if (s.kind != PKV_SEG_KIVI && s.kind != PKV_SEG_PER_TOKEN) return PKV_E_LAYOUT;
        if (!valid_bits(s.k_bits) || !valid_bits(s.v_bits)) return PKV_E_BITS;
        if (s.k_group <= 0 || s.v_group <= 0) return PKV_E_LAYOUT;
        if (!s.k_scale || !s.k_mins || !s.v_scale || !s.v_mins) return PKV_E_NULL;
    }
    return PKV_OK;
}

}  // namespace

// bytes-proportional cost of streaming a segment
static double seg_cost(const pkv_segment_t& s) {
    return (double)s.seq_len * (s.kind == PKV_SEG_FP16 ? 16 : s.k_bits);
}

DecodePlan plan_decode(const pkv_segment_t* segs, int n_segs, int Hq, int Hkv, int hd, int sm_count) {
    DecodePlan plan;
    const int G = Hq / Hkv;
    const int head_chunks = (G + GMAX - 1) / GMAX;
    sm_count = std::max(sm_count, 1);
    long long generic_tokens = 0;
    double fast_cost = 0.0;
    std::vector<char> is_fast(n_segs);
    for (int i = 0; i < n_segs; ++i) {
        is_fast[i] = mma::eligible(segs[i], Hq, Hkv, hd);
        if (is_fast[i]) fast_cost += seg_cost(segs[i]);
        else generic_tokens += segs[i].seq_len;
    }
    // generic kernel: about four CTAs per SM over its share of the layer
    const long long target = std::max<long long>(1, (4LL * sm_count) / ((long long)Hkv * head_chunks));
    // tensor-core kernel: one CTA per SM (it owns the SM's shared memory), one wave
    const double fast_ctas_per_head = std::max(1.0, (double)sm_count * mma::CTAS_PER_SM / Hkv);
    for (int i = 0; i < n_segs; ++i) {
        const pkv_segment_t& s = segs[i];
        SegDev d;
        d.kp = static_cast<const uint8_t*>(s.k_packed);
        d.ks = static_cast<const __half*>(s.k_scale);
        d.km = static_cast<const __half*>(s.k_mins);
        d.vp = static_cast<const uint8_t*>(s.v_packed);
        d.vs = static_cast<const __half*>(s.v_scale);
        d.vm = static_cast<const __half*>(s.v_mins);
        d.S = s.seq_len;
        d.head_stride = s.head_stride;
        d.kind = s.kind;
        d.kbits = s.kind == PKV_SEG_FP16 ? 8 : s.k_bits;
        d.vbits = s.kind == PKV_SEG_FP16 ? 8 : s.v_bits;
        d.kgs = s.kind == PKV_SEG_FP16 ? 1 : s.k_group;
        d.vgs = s.kind == PKV_SEG_FP16 ? 1 : s.v_group;
        if (is_fast[i]) {
            const long long tiles = mma::tiles_of(s);
            long long ctas;
            if (s.num_splits > 0) {
                ctas = std::min<long long>(tiles, s.num_splits);
            } else {
                ctas = (long long)(fast_ctas_per_head * seg_cost(s) / fast_cost);
                ctas = std::max<long long>(1, std::min(ctas, tiles));
            }
            d.split_len = ceil_div(tiles, ctas);
            // a CTA range that starts on a multiple of four tiles keeps the key scale rows 16-byte aligned
            if (s.kind != PKV_SEG_FP16 && s.num_splits <= 0 && d.split_len > 4) d.split_len = (d.split_len + 3) / 4 * 4;
            d.n_splits = (int)ceil_div(tiles, d.split_len);
            d.work_begin = plan.fast_work;
            plan.fast_work += d.n_splits;
            plan.fast.push_back(d);
        } else {
            if (s.num_splits > 0) {
                // plan_kivi_decode's manual convention (launch_config.py:58-60 of the reference)
                d.split_len = ceil_div(s.seq_len, std::min<long long>(s.seq_len, s.num_splits));
            } else {
                long long share = (target * s.seq_len + generic_tokens / 2) / generic_tokens;
                share = std::max<long long>(1, share);
                d.split_len = ceil_div(ceil_div(s.seq_len, share), kChunk) * kChunk;
            }
            d.n_splits = (int)ceil_div(s.seq_len, d.split_len);
            d.work_begin = plan.generic_work;
            plan.generic_work += d.n_splits;
            plan.generic.push_back(d);
        }
    }
    return plan;
}

}  // namespace pkv

using namespace pkv;

extern "C" {

int pkv_decode_workspace_bytes(const pkv_segment_t* segs, int n_segs, int num_q_heads, int num_kv_heads,
                               int head_dim, int sm_count, size_t* bytes) {
    if (!bytes) return PKV_E_NULL;
    const int rc = check_segments(segs, n_segs, num_q_heads, num_kv_heads, head_dim);
    if (rc != PKV_OK) return rc;
    const DecodePlan plan = plan_decode(segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_count);
    *bytes = (size_t)plan.total_work() * num_q_heads * (head_dim + 2) * sizeof(float);
    return PKV_OK;
}

int pkv_decode_attention(const void* q, const pkv_segment_t* segs, int n_segs, int num_q_heads,
                         int num_kv_heads, int head_dim, float sm_scale, int sm_count, void* workspace,
                         size_t workspace_bytes, void* out, float* m, float* l, float* acc,
                         pkv_stream_t stream) {
    const int rc = check_segments(segs, n_segs, num_q_heads, num_kv_heads, head_dim);
    if (rc != PKV_OK) return rc;
    if (!q || !workspace) return PKV_E_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const DecodePlan plan = plan_decode(segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_count);
    const size_t W = (size_t)plan.total_work();
    const size_t need = W * num_q_heads * (head_dim + 2) * sizeof(float);
    if (workspace_bytes < need) return PKV_E_WORKSPACE;
    // acc rows first: they are read as float4 and must start on 16 bytes
    float* pacc = reinterpret_cast<float*>(static_cast<char*>(workspace));
    float* pm = pacc + W * num_q_heads * head_dim;
    float* pl = pm + W * num_q_heads;
    // one tensor-core launch and nothing else: its last CTAs do the merge themselves
    static const bool carve = getenv("PKV_NO_CARVEOUT") == nullptr;
    static thread_local bool carved = false;
    if (carve && !carved) {
        // keep the SM's shared-memory split where the tensor-core kernel wants it, so alternating kernels do not
        // force a reconfiguration between launches
        cudaFuncSetAttribute(merge_partials_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(decode_generic_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        carved = true;
    }
    const int G = num_q_heads / num_kv_heads;

    // tensor-core kernel over the aligned KIVI segments
    for (size_t first = 0; first < plan.fast.size(); first += kMaxInlineSegs) {
        const int cnt = (int)std::min<size_t>(kMaxInlineSegs, plan.fast.size() - first);
        mma::MmaArgs a;
        a.q = static_cast<const __half*>(q);
        a.pm = pm;
        a.pl = pl;
        a.pacc = pacc;
        a.Hq = num_q_heads;
        a.Hkv = num_kv_heads;
        a.G = G;
        a.sm_scale = sm_scale;
        a.n_segs = cnt;
        a.work_offset = plan.fast[first].work_begin;
        int launch_work = 0;
        for (int i = 0; i < cnt; ++i) {
            a.segs[i] = plan.fast[first + i];
            a.segs[i].work_begin -= a.work_offset;
            launch_work += a.segs[i].n_splits;
        }
        static const int dbg2 = getenv("PKV_DEBUG_SKIP") ? atoi(getenv("PKV_DEBUG_SKIP")) : 0;
        if (dbg2 & 2) continue;
        const int rc2 = mma::launch(a, launch_work, num_kv_heads, s);
        if (rc2 != PKV_OK) return rc2;
    }
    // layout-generic kernel over everything else (float16 hot tier, per-token layout, ragged shapes)
    const size_t smem = sizeof(float) * ((size_t)GMAX * head_dim + (size_t)GMAX * kChunk + 3 * GMAX);
    for (size_t first = 0; first < plan.generic.size(); first += kMaxInlineSegs) {
        const int cnt = (int)std::min<size_t>(kMaxInlineSegs, plan.generic.size() - first);
        DecodeArgs a;
        a.q = static_cast<const __half*>(q);
        a.pm = pm;
        a.pl = pl;
        a.pacc = pacc;
        a.Hq = num_q_heads;
        a.Hkv = num_kv_heads;
        a.hd = head_dim;
        a.G = G;
        a.sm_scale = sm_scale;
        a.n_segs = cnt;
        a.work_offset = plan.fast_work + plan.generic[first].work_begin;
        int launch_work = 0;
        for (int i = 0; i < cnt; ++i) {
            a.segs[i] = plan.generic[first + i];
            a.segs[i].work_begin -= plan.generic[first].work_begin;
            launch_work += a.segs[i].n_splits;
        }
        dim3 grid((unsigned)launch_work, (unsigned)num_kv_heads, (unsigned)((G + GMAX - 1) / GMAX));
        decode_generic_kernel<<<grid, kThreads, smem, s>>>(a);
        PKV_LAUNCH_CHECK();
    }
    static const int dbg = getenv("PKV_DEBUG_SKIP") ? atoi(getenv("PKV_DEBUG_SKIP")) : 0;
    if (dbg & 1) return PKV_OK;
    {
        // programmatic dependent launch: the merge grid is scheduled while the split-K kernel drains, which hides
        // its launch latency; cudaGridDependencySynchronize() inside orders the data
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)num_q_heads);
        cfg.blockDim = dim3(kMergeThreads);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = s;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        const float* cpm = pm;
        const float* cpl = pl;
        const float* cpacc = pacc;
        PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partials_kernel, cpm, cpl, cpacc, (int)W, num_q_heads, head_dim,
                                        static_cast<__half*>(out), m, l, acc));
    }
    return PKV_OK;
}

int pkv_merge_partials(const float* m, const float* l, const float* acc, int n_parts, int num_q_heads,
                       int head_dim, void* out, float* m_out, float* l_out, float* acc_out,
                       pkv_stream_t stream) {
    if (!m || !l || !acc) return PKV_E_NULL;
    if (n_parts <= 0 || num_q_heads <= 0 || head_dim <= 0) return PKV_E_SHAPE;
    if (head_dim > 256) return PKV_E_LIMIT;
    if (head_dim % 4 || (reinterpret_cast<uintptr_t>(acc) & 15u)) return PKV_E_LAYOUT;
    merge_partials_kernel<<<num_q_heads, kMergeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        m, l, acc, n_parts, num_q_heads, head_dim, static_cast<__half*>(out), m_out, l_out, acc_out);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot provide scratch: a serving plugin that is handed a fixed memory
// budget at load time and is forbidden to touch the allocator on the request path, or code that runs
// while a stream is being captured, where cudaMalloc is illegal.  For them the split-K partials live
// in a fixed array inside the library image.  Every GPU that loads the library carries the array
// until the process exits, so it is kept modest.
//
// The array's name is only a host-side handle: the device address is looked up once per device with
// cudaGetSymbolAddress (with that device current) on the first call made on that device, which
// should therefore happen before any stream capture begins.  All calls on a device share the array
// and it keeps the previous call's partials; nothing in it has to start at zero, because each call
// overwrites every entry it later reads.  Two calls whose kernels overlap on the GPU race on it.
namespace {
__device__ __align__(256) unsigned char g_static_scratch[PKV_STATIC_SCRATCH_BYTES];
constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};
}  // namespace

extern "C" int pkv_decode_attention_static(const void* q, const pkv_segment_t* segs, int n_segs,
                                           int num_q_heads, int num_kv_heads, int head_dim, float sm_scale,
                                           int sm_count, void* out, float* m, float* l, float* acc,
                                           pkv_stream_t stream) {
    size_t need = 0;
    const int rc = pkv_decode_workspace_bytes(segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_count, &need);
    if (rc != PKV_OK) return rc;
    if (need > (size_t)PKV_STATIC_SCRATCH_BYTES) return PKV_E_LIMIT;
    int dev = 0;
    PKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return PKV_E_LIMIT;
    void* ptr = g_static_scratch_addr[dev];
    if (ptr == nullptr) {
        PKV_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_static_scratch_addr[dev] = ptr;  // racing first calls store the same value
    }
    return pkv_decode_attention(q, segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_scale, sm_count, ptr,
                                (size_t)PKV_STATIC_SCRATCH_BYTES, out, m, l, acc, stream);
}

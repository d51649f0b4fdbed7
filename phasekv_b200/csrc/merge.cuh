// Log-sum-exp merge of split-K partials, shared by the single-sequence and the batched decode entry points.
#pragma once

#include "common.cuh"

namespace pkv {

// Log-sum-exp merge of n_parts partials, one query head per CTA.
// Warp w owns parts p = w (mod kMergeWarps) and lane owns four consecutive dims (float4; head_dim <= 256 means
// up to two float4 per lane), so every load of a thread is independent of the others and of the
// weights: they are all issued before the first use, one memory round trip for the whole merge.
constexpr int kMergeThreads = 256;
constexpr int kMergeWarps = kMergeThreads / 32;
constexpr int kMergeMaxInflight = 6;  // parts per thread held in registers at once

// pm, pl, pacc point at the first of the n_parts partials ([Hq] and [Hq][hd] each); consecutive partials are
// ml_stride floats apart in pm and pl and acc_stride floats apart in pacc (Hq and Hq * hd when the arrays are
// dense).  out, m_out, l_out, acc_out point at the result rows of this query head's sequence.
// COHERENT: the partials may have been written by another GPU while this kernel runs; read them through L2
// (ld.cg) instead of the non-coherent path.
//
// merge_reduce leaves the merged (M, L) in every thread and A[tid] in threads tid < hd; no partials at all give
// the neutral element (-inf, 0, 0).  It uses static shared memory: put a __syncthreads() between two calls.
template <bool COHERENT = false>
__device__ __forceinline__ void merge_reduce(const float* __restrict__ pm, const float* __restrict__ pl,
                                             const float* __restrict__ pacc, int n_parts, size_t ml_stride,
                                             size_t acc_stride, int hd, int h, float& M_out, float& L_out,
                                             float& A_out) {
    __shared__ float red_m[kMergeWarps];
    __shared__ float red_l[kMergeWarps];
    __shared__ __align__(16) float red_acc[kMergeWarps][256];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int nvec = hd >> 2;  // float4 per row (hd % 4 == 0 is checked on the host)
    const bool v0 = lane < nvec, v1 = lane + 32 < nvec;

    // Every load of a batch (acc rows, m, l of up to kMergeWarps * kMergeMaxInflight parts) is issued before anything
    // is reduced, so a typical merge (a few dozen parts) is one memory round trip.  Batches are combined
    // with a running maximum, like the online softmax itself.
    float run_m = -INFINITY;  // block-wide running max (identical in every thread)
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    float ls = 0.f;
    for (int base = 0; base < n_parts; base += kMergeWarps * kMergeMaxInflight) {
        float4 r0[kMergeMaxInflight], r1[kMergeMaxInflight];
        float wm[kMergeMaxInflight], wl[kMergeMaxInflight];
        float mx = -INFINITY;
#pragma unroll
        for (int u = 0; u < kMergeMaxInflight; ++u) {
            const int p = base + wid + kMergeWarps * u;
            r0[u] = r1[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            wm[u] = -INFINITY;
            wl[u] = 0.f;
            if (p < n_parts) {
                const float4* row = reinterpret_cast<const float4*>(pacc + (size_t)p * acc_stride + (size_t)h * hd);
                if (v0) r0[u] = COHERENT ? __ldcg(row + lane) : __ldg(row + lane);
                if (v1) r1[u] = COHERENT ? __ldcg(row + lane + 32) : __ldg(row + lane + 32);
                wm[u] = COHERENT ? __ldcg(pm + (size_t)p * ml_stride + h) : __ldg(pm + (size_t)p * ml_stride + h);
                wl[u] = COHERENT ? __ldcg(pl + (size_t)p * ml_stride + h) : __ldg(pl + (size_t)p * ml_stride + h);
            }
        }
#pragma unroll
        for (int u = 0; u < kMergeMaxInflight; ++u) mx = fmaxf(mx, wm[u]);
        __syncthreads();  // red_m is free again
        if (lane == 0) red_m[wid] = mx;
        __syncthreads();
        mx = run_m;
#pragma unroll
        for (int w = 0; w < kMergeWarps; ++w) mx = fmaxf(mx, red_m[w]);
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
    for (int w = 0; w < kMergeWarps; ++w) L += red_l[w];
    float A = 0.f;
    if (tid < hd) {
#pragma unroll
        for (int w = 0; w < kMergeWarps; ++w) A += red_acc[w][tid];
    }
    M_out = mx;
    L_out = L;
    A_out = A;
}

template <bool COHERENT = false>
__device__ __forceinline__ void merge_parts(const float* __restrict__ pm, const float* __restrict__ pl,
                                            const float* __restrict__ pacc, int n_parts, size_t ml_stride,
                                            size_t acc_stride, int hd, int h,
                                            __half* __restrict__ out, float* __restrict__ m_out,
                                            float* __restrict__ l_out, float* __restrict__ acc_out) {
    float mx, L, A;
    merge_reduce<COHERENT>(pm, pl, pacc, n_parts, ml_stride, acc_stride, hd, h, mx, L, A);
    const int tid = threadIdx.x;
    if (tid < hd) {
        if (out) out[(size_t)h * hd + tid] = __float2half_rn(A / L);
        if (acc_out) acc_out[(size_t)h * hd + tid] = A;
    }
    if (tid == 0) {
        if (m_out) m_out[h] = mx;
        if (l_out) l_out[h] = L;
    }
}

}  // namespace pkv

// Stage-A operators on a dense float16 / bfloat16 KV cache: the reference evaluates accuracy by quantising
// and immediately dequantising cache slices in place ("fake quantisation", quant.py:34-79), choosing the
// tokens to keep from value norms (hetero_cache.py:98-113, 157-167) and compacting the cache per head
// (hetero_cache.py:120-154).  Each of those torch pipelines is one launch here.
//
// Fake quantisation differs from the packed path in two ways that both matter bit for bit: scale and zero stay
// float32 (the packed path stores them as float16), and any width from 1 to 15 bits is allowed.
#include <cuda_bf16.h>

#include "common.cuh"

namespace pkv {
namespace {

constexpr int kStageThreads = 256;

template <class T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <class T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }

// One thread owns one group: it reads the group (min / max), then reads it again and writes the grid values,
// so the operation is safe in place.  Threads are adjacent along `inner` (coalesced when the axis is not the
// last dimension); for inner == 1 adjacent threads own adjacent groups of one row.
template <class T>
__global__ void __launch_bounds__(kStageThreads)
fake_quant_kernel(const T* x, T* out,  /* out may equal x */ int64_t outer, int64_t A, int64_t inner,
                  int64_t outer_stride, int64_t gs, int64_t n_groups, float qmax) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= outer * n_groups * inner) return;
    const int64_t j = tid % inner;
    const int64_t g = (tid / inner) % n_groups;
    const int64_t o = tid / (inner * n_groups);
    const int64_t a0 = g * gs, a1 = min(A, a0 + gs);
    const T* xp = x + o * outer_stride + j;
    T* op = out + o * outer_stride + j;
    float lo = to_f32(xp[a0 * inner]), hi = lo;
    for (int64_t a = a0 + 1; a < a1; ++a) {
        const float v = to_f32(xp[a * inner]);
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
    const float sc = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
    for (int64_t a = a0; a < a1; ++a) {
        float q = rintf(__fdiv_rn(__fsub_rn(to_f32(xp[a * inner]), lo), sc));
        q = fminf(fmaxf(q, 0.f), qmax);
        op[a * inner] = from_f32<T>(__fadd_rn(__fmul_rn(q, sc), lo));  // two roundings, as q * scale + min in torch
    }
}

// L2 norm over head_dim of tokens [0, n) of each row (row = one (batch, KV head)); one warp per token.
template <class T>
__global__ void __launch_bounds__(kStageThreads)
value_norm_kernel(const T* __restrict__ v, int64_t rows, int64_t row_stride, int64_t n, int hd,
                  float* __restrict__ out) {
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= rows * n) return;
    const int64_t row = w / n, t = w % n;
    const T* p = v + row * row_stride + t * hd;
    float s = 0.f;
    for (int d = lane; d < hd; d += 32) {
        const float f = to_f32(p[d]);
        s = fmaf(f, f, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[w] = sqrtf(s);
}

// Positions of the `keep` largest entries of every row of signal [rows, n], ties towards the lower position,
// written in ascending position order.  Rank counting: n^2 comparisons per row, meant for a lazy batch of a
// few hundred tokens.
constexpr int kTopkMax = 4096;
__global__ void __launch_bounds__(kStageThreads)
topk_rows_kernel(const float* __restrict__ signal, int64_t n, int64_t keep, long long* __restrict__ indices) {
    __shared__ float s[kTopkMax];
    __shared__ int warp_tot[kStageThreads / 32];
    __shared__ int running;
    const int64_t row = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    for (int64_t i = tid; i < n; i += kStageThreads) s[i] = signal[row * n + i];
    if (tid == 0) running = 0;
    __syncthreads();
    for (int64_t base = 0; base < n; base += kStageThreads) {
        const int64_t t = base + tid;
        int flag = 0;
        if (t < n) {
            // a total order (NaN largest, as torch.topk has it): exactly `keep` entries rank below keep
            const unsigned mine = order_key(s[t]);
            int rank = 0;
            for (int64_t k = 0; k < n; ++k) {
                const unsigned o = order_key(s[k]);
                rank += (o > mine) || (o == mine && k < t);
            }
            flag = rank < keep;
        }
        const unsigned ballot = __ballot_sync(0xffffffffu, flag);
        if (lane == 0) warp_tot[wid] = __popc(ballot);
        __syncthreads();
        int offset = running;
        for (int w = 0; w < wid; ++w) offset += warp_tot[w];
        const int pos = offset + __popc(ballot & ((1u << lane) - 1u));
        if (flag && pos < keep) indices[row * keep + pos] = t;
        __syncthreads();
        if (tid == 0) {
            int tot = 0;
            for (int w = 0; w < kStageThreads / 32; ++w) tot += warp_tot[w];
            running += tot;
        }
        __syncthreads();
    }
}

// The same selection for rows of any length (a whole prompt's candidates per head): radix select on the order
// keys, one CTA per row.  Four passes of 8-bit histograms find the key T of the keep-th largest entry and how
// many entries equal to T still belong to the selection; one more pass over the positions in ascending order
// emits every entry above T and the first of those equal to it (ties to the lower position, as above).
constexpr int kSelThreads = 1024;
__device__ __forceinline__ int block_exclusive_scan(int flag, int* warp_tot, int& total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const unsigned ballot = __ballot_sync(0xffffffffu, flag);
    __syncthreads();  // warp_tot is free again
    if (lane == 0) warp_tot[wid] = __popc(ballot);
    __syncthreads();
    int before = 0, sum = 0;
    for (int w = 0; w < kSelThreads / 32; ++w) {
        if (w == wid) before = sum;
        sum += warp_tot[w];
    }
    total = sum;
    return before + __popc(ballot & ((1u << lane) - 1u));
}

__global__ void __launch_bounds__(kSelThreads)
topk_rows_select_kernel(const float* __restrict__ signal, int64_t n, int64_t keep, long long* __restrict__ indices) {
    __shared__ unsigned hist[256];
    __shared__ unsigned s_prefix;
    __shared__ long long s_remaining;
    __shared__ int warp_tot[kSelThreads / 32];
    const int tid = threadIdx.x;
    const float* x = signal + (int64_t)blockIdx.x * n;
    long long* out = indices + (int64_t)blockIdx.x * keep;
    unsigned prefix = 0u, mask = 0u;
    long long remaining = keep;  // entries still to take among those whose key matches `prefix` under `mask`
    for (int shift = 24; shift >= 0; shift -= 8) {
        if (tid < 256) hist[tid] = 0u;
        __syncthreads();
        for (int64_t i = tid; i < n; i += kSelThreads) {
            const unsigned key = order_key(x[i]);
            if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            long long above = 0;
            int b = 255;
            for (; b > 0; --b) {
                if (above + hist[b] >= remaining) break;
                above += hist[b];
            }
            s_prefix = prefix | ((unsigned)b << shift);
            s_remaining = remaining - above;  // to take among the keys of bin b
        }
        __syncthreads();
        prefix = s_prefix;
        remaining = s_remaining;
        mask |= 255u << shift;
        __syncthreads();
    }
    const unsigned T = prefix;
    const long long need_eq = remaining;
    long long run_out = 0, run_eq = 0;
    for (int64_t base = 0; base < n; base += kSelThreads) {
        const int64_t i = base + tid;
        const unsigned key = i < n ? order_key(x[i]) : 0u;
        const int gt = i < n && key > T, eq = i < n && key == T;
        int eq_total, take_total;
        const int eq_before = block_exclusive_scan(eq, warp_tot, eq_total);
        const int take = gt || (eq && run_eq + eq_before < need_eq);
        const int pos = block_exclusive_scan(take, warp_tot, take_total);
        if (take && run_out + pos < keep) out[run_out + pos] = i;
        run_out += take_total;
        run_eq += eq_total;
    }
}

// dst[row][j][:] = src[row][indices[row][j]][:], token rows of `token_bytes` bytes moved as 16-byte words.
__global__ void __launch_bounds__(kStageThreads)
gather_tokens_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const long long* __restrict__ indices,
                     int64_t rows, int64_t src_tokens, int64_t keep, int words) {
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= rows * keep * words) return;
    const int w = (int)(tid % words);
    const int64_t j = (tid / words) % keep;
    const int64_t row = tid / ((int64_t)words * keep);
    const int64_t t = indices[row * keep + j];
    // an index outside the source is never dereferenced: the row comes out as zeros (callers validate indices
    // on the host where they can afford to; this keeps a bad index from becoming a stray read)
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t >= 0 && t < src_tokens) v = __ldg(src + (row * src_tokens + t) * words + w);
    dst[(row * keep + j) * words + w] = v;
}

unsigned grid_for(int64_t n) { return (unsigned)((n + kStageThreads - 1) / kStageThreads); }

}  // namespace
}  // namespace pkv

using namespace pkv;

extern "C" {

int pkv_fake_quant(const void* x, void* out, int dtype, int64_t outer, int64_t axis_len, int64_t inner,
                   int64_t outer_stride, int bits, int64_t group, pkv_stream_t stream) {
    if (bits < 1 || bits > 15) return PKV_E_BITS;
    if (outer < 0 || inner < 0 || axis_len <= 0 || group <= 0 || group > axis_len) return PKV_E_SHAPE;
    if (outer_stride == 0) outer_stride = axis_len * inner;
    if (outer_stride < axis_len * inner) return PKV_E_SHAPE;
    if (outer * inner == 0) return PKV_OK;
    if (!x || !out) return PKV_E_NULL;
    const int64_t n_groups = ceil_div(axis_len, group);
    const int64_t n = outer * n_groups * inner;
    if (n > (int64_t)INT32_MAX * kStageThreads) return PKV_E_LIMIT;
    const float qmax = (float)((1 << bits) - 1);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == PKV_DTYPE_F16)
        fake_quant_kernel<__half><<<grid_for(n), kStageThreads, 0, s>>>(
            static_cast<const __half*>(x), static_cast<__half*>(out), outer, axis_len, inner, outer_stride, group, n_groups, qmax);
    else if (dtype == PKV_DTYPE_BF16)
        fake_quant_kernel<__nv_bfloat16><<<grid_for(n), kStageThreads, 0, s>>>(
            static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), outer, axis_len, inner, outer_stride, group, n_groups, qmax);
    else if (dtype == PKV_DTYPE_F32)
        fake_quant_kernel<float><<<grid_for(n), kStageThreads, 0, s>>>(
            static_cast<const float*>(x), static_cast<float*>(out), outer, axis_len, inner, outer_stride, group, n_groups, qmax);
    else
        return PKV_E_LAYOUT;
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int pkv_value_norm(const void* v, int dtype, int64_t rows, int64_t row_stride, int64_t n_tokens, int head_dim,
                   float* out, pkv_stream_t stream) {
    if (rows < 0 || n_tokens < 0 || head_dim <= 0 || row_stride < n_tokens * head_dim) return PKV_E_SHAPE;
    if (rows * n_tokens == 0) return PKV_OK;
    if (!v || !out) return PKV_E_NULL;
    const int64_t threads = rows * n_tokens * 32;
    if (threads > (int64_t)INT32_MAX * kStageThreads) return PKV_E_LIMIT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == PKV_DTYPE_F16)
        value_norm_kernel<__half><<<grid_for(threads), kStageThreads, 0, s>>>(static_cast<const __half*>(v), rows, row_stride, n_tokens, head_dim, out);
    else if (dtype == PKV_DTYPE_BF16)
        value_norm_kernel<__nv_bfloat16><<<grid_for(threads), kStageThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(v), rows, row_stride, n_tokens, head_dim, out);
    else if (dtype == PKV_DTYPE_F32)
        value_norm_kernel<float><<<grid_for(threads), kStageThreads, 0, s>>>(static_cast<const float*>(v), rows, row_stride, n_tokens, head_dim, out);
    else
        return PKV_E_LAYOUT;
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int pkv_topk_rows(const float* signal, int64_t rows, int64_t n, int64_t keep, int64_t* indices, pkv_stream_t stream) {
    if (rows < 0 || n <= 0 || keep <= 0 || keep > n) return PKV_E_SHAPE;
    if (rows > INT32_MAX) return PKV_E_LIMIT;
    if (rows == 0) return PKV_OK;
    if (!signal || !indices) return PKV_E_NULL;
    if (n <= kTopkMax)
        topk_rows_kernel<<<(unsigned)rows, kStageThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            signal, n, keep, reinterpret_cast<long long*>(indices));
    else
        topk_rows_select_kernel<<<(unsigned)rows, kSelThreads, 0, static_cast<cudaStream_t>(stream)>>>(
            signal, n, keep, reinterpret_cast<long long*>(indices));
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int pkv_gather_tokens(const void* src, void* dst, const int64_t* indices, int64_t rows, int64_t src_tokens,
                      int64_t keep, int64_t token_bytes, pkv_stream_t stream) {
    if (rows < 0 || src_tokens <= 0 || keep <= 0 || token_bytes <= 0) return PKV_E_SHAPE;
    if (token_bytes % 16 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15u)) return PKV_E_LAYOUT;
    if (rows == 0) return PKV_OK;
    if (!src || !dst || !indices) return PKV_E_NULL;
    const int64_t n = rows * keep * (token_bytes / 16);
    if (n > (int64_t)INT32_MAX * kStageThreads) return PKV_E_LIMIT;
    gather_tokens_kernel<<<grid_for(n), kStageThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), reinterpret_cast<const long long*>(indices), rows,
        src_tokens, keep, (int)(token_bytes / 16));
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

}  // extern "C"

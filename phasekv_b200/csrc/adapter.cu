// The step of a model's attention layer that sits between the projections and decode attention: rotary position
// embedding of the new tokens' queries and keys, conversion to float16, and the write of the new keys and values
// into the float16 tier.  In the reference these are separate torch operations per layer and token
// (qwen2_attention.py:79-106: apply_rotary_pos_emb, three .to(float16), then two copy_ per appended token): about
// fifteen launches.  Here it is one launch for a whole chunk of tokens.
//
// The rotation is rounded where torch rounds it when it runs in the model's dtype T (float16 or bfloat16):
// x * cos -> T, rotate_half(x) * sin -> T, their sum -> T, and only then T -> float16.
#include <cuda_bf16.h>

#include "common.cuh"

namespace pkv {
namespace {

constexpr int kRopeThreads = 128;

template <class T> __device__ __forceinline__ float ld_f32(const T* p);
template <> __device__ __forceinline__ float ld_f32<__half>(const __half* p) { return __half2float(*p); }
template <> __device__ __forceinline__ float ld_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <> __device__ __forceinline__ float ld_f32<float>(const float* p) { return *p; }
template <class T> __device__ __forceinline__ float round_to(float v);
template <> __device__ __forceinline__ float round_to<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float round_to<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

struct RopeArgs {
    const void *q, *k, *v, *cos, *sin;
    __half *q_out, *hot_k, *hot_v;
    long long q_stride, k_stride, v_stride, rope_stride;  // elements between consecutive tokens
    long long capacity, slot;                             // hot buffers [Hkv, capacity, hd]; first slot written
    const int* slot_dev;                                  // optional: the first slot is *slot_dev + slot
    int n_tokens, Hq, Hkv, hd;
};

// grid (Hq + 2 * Hkv, n_tokens): one block per (token, head vector); thread d handles dimension d and its partner.
template <class T, class R>
__global__ void __launch_bounds__(kRopeThreads) rope_append_kernel(const RopeArgs a) {
    // Launched as a programmatic dependent: everything this kernel reads may come from the previous kernel of the
    // stream, so it waits for it first; the next kernel (decode attention) may then become resident and prefetch its
    // packed segments while this one runs (it waits for this grid before it reads q or the float16 tier).
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();
    const int t = blockIdx.y, h = blockIdx.x;
    const int half = a.hd >> 1;
    const long long slot = a.slot + (a.slot_dev ? (long long)*a.slot_dev : 0);
    const bool in_tier = slot >= 0 && slot + a.n_tokens <= a.capacity;  // (always true for a host-given slot)
    if (h >= a.Hq && !in_tier) return;
    if (h >= a.Hq + a.Hkv) {  // a value vector: converted and stored
        const int kvh = h - a.Hq - a.Hkv;
        const T* src = static_cast<const T*>(a.v) + t * a.v_stride + (long long)kvh * a.hd;
        __half* dst = a.hot_v + ((long long)kvh * a.capacity + slot + t) * a.hd;
        for (int d = threadIdx.x; d < a.hd; d += kRopeThreads) dst[d] = __float2half_rn(ld_f32(src + d));
        return;
    }
    const bool is_q = h < a.Hq;
    const int head = is_q ? h : h - a.Hq;
    const T* src = is_q ? static_cast<const T*>(a.q) + t * a.q_stride + (long long)head * a.hd
                        : static_cast<const T*>(a.k) + t * a.k_stride + (long long)head * a.hd;
    __half* dst = is_q ? a.q_out + ((long long)t * a.Hq + head) * a.hd
                       : a.hot_k + ((long long)head * a.capacity + slot + t) * a.hd;
    const R* cs = static_cast<const R*>(a.cos) + t * a.rope_stride;
    const R* sn = static_cast<const R*>(a.sin) + t * a.rope_stride;
    for (int d = threadIdx.x; d < a.hd; d += kRopeThreads) {
        const float x = ld_f32(src + d);
        // rotate_half: (-x[half:], x[:half])
        const float r = d < half ? -ld_f32(src + d + half) : ld_f32(src + d - half);
        // cos / sin take part in the model's dtype (transformers casts them to it before the product)
        const float c = round_to<T>(ld_f32(cs + d)), s = round_to<T>(ld_f32(sn + d));
        const float y = round_to<T>(__fadd_rn(round_to<T>(__fmul_rn(x, c)), round_to<T>(__fmul_rn(r, s))));
        dst[d] = __float2half_rn(y);
    }
}

template <class T>
int launch_rope(const RopeArgs& a, int rope_dtype, cudaStream_t s) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(a.Hq + 2 * a.Hkv), (unsigned)a.n_tokens);
    cfg.blockDim = dim3(kRopeThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    switch (rope_dtype) {
        case PKV_DTYPE_F16: PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, rope_append_kernel<T, __half>, a)); break;
        case PKV_DTYPE_BF16: PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, rope_append_kernel<T, __nv_bfloat16>, a)); break;
        case PKV_DTYPE_F32: PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, rope_append_kernel<T, float>, a)); break;
        default: return PKV_E_LAYOUT;
    }
    return PKV_OK;
}

}  // namespace
}  // namespace pkv

extern "C" int pkv_rope_append(const void* q, const void* k, const void* v, int dtype, int64_t q_token_stride,
                               int64_t k_token_stride, int64_t v_token_stride, const void* cos, const void* sin,
                               int rope_dtype, int64_t rope_token_stride, int n_tokens, int num_q_heads,
                               int num_kv_heads, int head_dim, void* q_out, void* hot_k, void* hot_v,
                               int64_t capacity, int64_t slot, const int32_t* slot_dev, pkv_stream_t stream) {
    using namespace pkv;
    if (!q || !k || !v || !cos || !sin || !q_out || !hot_k || !hot_v) return PKV_E_NULL;
    if (n_tokens <= 0 || n_tokens > 65535 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0 || (head_dim & 1))
        return PKV_E_SHAPE;
    if (!slot_dev && (slot < 0 || slot + n_tokens > capacity)) return PKV_E_SHAPE;
    if (n_tokens > capacity) return PKV_E_SHAPE;
    if (q_token_stride < (int64_t)num_q_heads * head_dim || k_token_stride < (int64_t)num_kv_heads * head_dim ||
        v_token_stride < (int64_t)num_kv_heads * head_dim || rope_token_stride < 0)
        return PKV_E_SHAPE;
    RopeArgs a;
    a.q = q, a.k = k, a.v = v, a.cos = cos, a.sin = sin;
    a.q_out = static_cast<__half*>(q_out), a.hot_k = static_cast<__half*>(hot_k), a.hot_v = static_cast<__half*>(hot_v);
    a.q_stride = q_token_stride, a.k_stride = k_token_stride, a.v_stride = v_token_stride, a.rope_stride = rope_token_stride;
    a.capacity = capacity, a.slot = slot, a.slot_dev = slot_dev;
    a.n_tokens = n_tokens, a.Hq = num_q_heads, a.Hkv = num_kv_heads, a.hd = head_dim;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == PKV_DTYPE_F16) return launch_rope<__half>(a, rope_dtype, s);
    if (dtype == PKV_DTYPE_BF16) return launch_rope<__nv_bfloat16>(a, rope_dtype, s);
    return PKV_E_LAYOUT;
}

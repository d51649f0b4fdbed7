// Shared helpers for the phasekv_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/phasekv_b200.h"

namespace pkv {

extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
    g_last_cuda_error = static_cast<int>(e);
    return PKV_E_CUDA;
}

#define PKV_CUDA_TRY(expr)                                   \
    do {                                                     \
        cudaError_t _e = (expr);                             \
        if (_e != cudaSuccess) return ::pkv::cuda_fail(_e);  \
    } while (0)

#define PKV_LAUNCH_CHECK() PKV_CUDA_TRY(cudaGetLastError())

inline bool valid_bits(int bits) { return bits == 2 || bits == 4 || bits == 8; }

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

__device__ __forceinline__ float h2f(const __half h) { return __half2float(h); }

// code i of a byte occupies bits [i*bits, (i+1)*bits)
template <int BITS>
__device__ __forceinline__ unsigned extract_code(unsigned byte, unsigned idx_in_byte) {
    return (byte >> (idx_in_byte * BITS)) & ((1u << BITS) - 1u);
}

__device__ __forceinline__ unsigned extract_code_rt(unsigned byte, unsigned idx_in_byte, int bits) {
    return (byte >> (idx_in_byte * bits)) & ((1u << bits) - 1u);
}


// Total order on float32 that matches torch.topk: NaN is the largest value, -0 equals +0, everything else
// compares as numbers.  Returns a key whose unsigned order is that order.
__device__ __forceinline__ unsigned order_key(float x) {
    if (x != x) return 0xffffffffu;
    const unsigned b = __float_as_uint(x + 0.0f);  // -0 + 0 = +0
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// rint((d / sc)) with the quotient rounded to float32 first, exactly as IEEE division gives it, at
// the cost of a multiply in the common case: d * (1/sc) is within two ulp of the true quotient, so
// the two can only round to different integers when the product lies within a hair of a half-integer;
// only then is the real division done.  (Quotients here are at most 255, two ulp < 3.1e-5.)
__device__ __forceinline__ float quantise_round(float d, float sc, float inv_sc) {
    const float r = d * inv_sc;
    const float t = rintf(r);
    if (fabsf(r - t) > 0.4999f) return rintf(__fdiv_rn(d, sc));
    return t;
}

// The same rounding for the hot loops of the pack kernels, without a branch per element.  Adding 1.5 * 2^23 to a
// value in [0, 2^22) rounds it to an integer, ties to even, and leaves that integer in the low mantissa bits:
// rint and the float-to-integer conversion in one addition.  `near` collects whether any product came within a
// hair of a half-integer (see quantise_round): the caller then redoes its handful of elements with the real
// division.  d >= 0 (a value minus its group's minimum), so only the upper clamp is needed, and the clamp may be
// applied before rounding because rounding is monotonic.
constexpr float kRoundMagic = 12582912.0f;
//
// How close is "a hair": the product is within 1.5 ulp of the quotient, so a margin of four ulp of the largest code
// around the half-integers is safe, and it is narrow enough that the redo stays rare even though it is taken by a
// whole warp when any of its lanes asks for it.
template <int BITS>
__device__ __forceinline__ constexpr float near_half() {
    return BITS == 2 ? 0.499999f : BITS == 4 ? 0.499996f : 0.49994f;
}
template <int BITS>
__device__ __forceinline__ unsigned quantise_bits(float d, float inv_sc, bool& near) {
    constexpr float QMAX = (float)((1 << BITS) - 1);
    const float r = fminf(d * inv_sc, QMAX);
    const float b = r + kRoundMagic;
    near |= fabsf(r - (b - kRoundMagic)) > near_half<BITS>();
    return __float_as_uint(b);  // the code sits in the low bits
}
__device__ __forceinline__ unsigned quantise_exact(float d, float sc, float qmax) {
    return (unsigned)fminf(fmaxf(rintf(__fdiv_rn(d, sc)), 0.f), qmax);
}
// bits [pos, pos + len) of `into` replaced by the low `len` bits of `field`
__device__ __forceinline__ unsigned insert_bits(unsigned field, unsigned into, int pos, int len) {
    unsigned r;
    asm("bfi.b32 %0, %1, %2, %3, %4;" : "=r"(r) : "r"(field), "r"(into), "r"(pos), "r"(len));
    return r;
}

}  // namespace pkv

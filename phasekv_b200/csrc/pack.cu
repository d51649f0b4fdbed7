// Sub-byte packing and grouped asymmetric min-max quantisation.
//
// Arithmetic contract (what makes codes, scales and zeros bit-identical to the reference's
// packing.py:115-155 executed on a CPU):
//   scale32 = max(max - min, 1e-8f) / qmax          IEEE float division, never a reciprocal
//   code    = clamp(rint((x - min) / scale32), 0, qmax)   round-half-to-even
//   stored scale = float16(scale32), stored zero = float16(min)   (round-to-nearest-even)
// The tail group is reduced over its real elements only: the reference pads it by repeating the
// last element, which changes neither the minimum nor the maximum.
#include "common.cuh"

namespace pkv {

thread_local int g_last_cuda_error = 0;

namespace {

constexpr int kThreads = 256;

template <int BITS>
__global__ void pack_low_bits_kernel(const uint8_t* __restrict__ codes, int64_t rows, int64_t len,
                                     int64_t nb, uint8_t* __restrict__ out) {
    constexpr int VPB = 8 / BITS;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * nb) return;
    const int64_t r = i / nb, b = i % nb;
    const uint8_t* c = codes + r * len + b * VPB;
    unsigned v = 0;
#pragma unroll
    for (int k = 0; k < VPB; ++k)
        if (b * VPB + k < len) v += (unsigned)c[k] << (k * BITS);
    out[i] = (uint8_t)v;
}

template <int BITS>
__global__ void unpack_low_bits_kernel(const uint8_t* __restrict__ packed, int64_t rows,
                                       int64_t row_bytes, int64_t len, uint8_t* __restrict__ out) {
    constexpr int VPB = 8 / BITS;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * len) return;
    const int64_t r = i / len, j = i % len;
    out[i] = (uint8_t)extract_code<BITS>(packed[r * row_bytes + j / VPB], (unsigned)(j % VPB));
}

// One thread quantises `run` consecutive positions of the axis for one (outer, inner) line.
// `run` is a multiple of lcm(group, 8/BITS), so a thread owns whole groups and whole bytes.
template <int BITS>
__global__ void quantize_pack_kernel(const __half* __restrict__ x, int64_t outer, int64_t A,
                                     int64_t inner, int64_t gs, int64_t run, int64_t n_runs,
                                     int64_t nb, int64_t ng, uint8_t* __restrict__ packed,
                                     __half* __restrict__ scale, __half* __restrict__ mins) {
    constexpr int VPB = 8 / BITS;
    constexpr float QMAX = (float)((1 << BITS) - 1);
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= outer * n_runs * inner) return;
    const int64_t j = tid % inner;
    const int64_t r = (tid / inner) % n_runs;
    const int64_t o = tid / (inner * n_runs);
    const int64_t a_begin = r * run;
    const int64_t a_end = min(A, a_begin + run);
    const __half* xp = x + o * A * inner + j;
    const int64_t row = o * inner + j;
    uint8_t* prow = packed + row * nb;

    unsigned long long word = 0;  // up to 8 finished bytes waiting to be stored
    int word_bytes = 0;
    int64_t word_first = a_begin / VPB;  // byte index of the first byte held in `word`
    unsigned cur = 0;

    for (int64_t g0 = a_begin; g0 < a_end; g0 += gs) {
        const int64_t g1 = min(g0 + gs, A);
        float lo = __half2float(xp[g0 * inner]);
        float hi = lo;
        for (int64_t a = g0 + 1; a < g1; ++a) {
            const float v = __half2float(xp[a * inner]);
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
        }
        const float sc = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), QMAX);
        const float inv = __frcp_rn(sc);
        for (int64_t a = g0; a < g1; ++a) {
            const float v = __half2float(xp[a * inner]);
            float qv = quantise_round(__fsub_rn(v, lo), sc, inv);
            qv = fminf(fmaxf(qv, 0.f), QMAX);
            const int pos = (int)(a % VPB);
            cur |= (unsigned)qv << (pos * BITS);
            if (pos == VPB - 1 || a == A - 1) {
                word |= (unsigned long long)cur << (8 * word_bytes);
                cur = 0;
                if (++word_bytes == 8) {
                    uint8_t* dst = prow + word_first;
                    if ((reinterpret_cast<uintptr_t>(dst) & 7u) == 0) {
                        *reinterpret_cast<unsigned long long*>(dst) = word;
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) dst[k] = (uint8_t)(word >> (8 * k));
                    }
                    word_first += 8;
                    word = 0;
                    word_bytes = 0;
                }
            }
        }
        scale[row * ng + g0 / gs] = __float2half_rn(sc);
        mins[row * ng + g0 / gs] = __float2half_rn(lo);
    }
    for (int k = 0; k < word_bytes; ++k) prow[word_first + k] = (uint8_t)(word >> (8 * k));
}

// Quantise 8 float16 values (one 16-byte word) of a group whose minimum and scale are known; returns the codes
// packed little-endian, BITS bits each (8 * BITS bits).
template <int BITS>
__device__ __forceinline__ unsigned long long quantise8(const uint4& raw, float lo, float sc, float inv) {
    constexpr float QMAX = (float)((1 << BITS) - 1);
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
    float d[8];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float2 f = __half22float2(h2[c]);
        d[2 * c] = __fsub_rn(f.x, lo);
        d[2 * c + 1] = __fsub_rn(f.y, lo);
    }
    unsigned w[2] = {0u, 0u};
    bool near = false;
#pragma unroll
    for (int i = 0; i < 8; ++i)
        w[(i * BITS) / 32] = insert_bits(quantise_bits<BITS>(d[i], inv, near), w[(i * BITS) / 32], (i * BITS) % 32, BITS);
    if (near) {  // rare: a product too close to a half-integer to trust; the whole word again with real divisions
        w[0] = w[1] = 0u;
#pragma unroll
        for (int i = 0; i < 8; ++i) w[(i * BITS) / 32] |= quantise_exact(d[i], sc, QMAX) << ((i * BITS) % 32);
    }
    return (unsigned long long)w[0] | ((unsigned long long)w[1] << 32);
}

// Fast path for the value layout: the axis is the contiguous last dimension (inner == 1), the group is 32
// elements and rows are multiples of 32 long.  A thread owns 8 consecutive elements (one 16-byte load, so a warp
// reads 512 contiguous bytes per instruction) and four neighbouring lanes own a group: minimum and maximum are
// combined with two shuffles, then every lane quantises its own 8 elements and stores its own BITS bytes (a warp
// writes 32 * BITS contiguous bytes per instruction).  The minimum and maximum are taken in float16, which is
// exact; everything after that is float32 as in the reference.
template <int BITS>
__global__ void __launch_bounds__(256)
quantize_pack_lastdim32_kernel(const __half* __restrict__ x, int64_t n_chunks, uint8_t* __restrict__ packed,
                               __half* __restrict__ scale, __half* __restrict__ mins) {
    constexpr float QMAX = (float)((1 << BITS) - 1);
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // 16-byte chunk; n_chunks % 4 == 0
    const bool live = c < n_chunks;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (live) raw = __ldg(reinterpret_cast<const uint4*>(x) + c);
    const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
    __half2 lo2 = __hmin2(__hmin2(h2[0], h2[1]), __hmin2(h2[2], h2[3]));
    __half2 hi2 = __hmax2(__hmax2(h2[0], h2[1]), __hmax2(h2[2], h2[3]));
#pragma unroll
    for (int o = 1; o <= 2; o <<= 1) {
        unsigned l = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<unsigned*>(&lo2), o);
        unsigned h = __shfl_xor_sync(0xffffffffu, *reinterpret_cast<unsigned*>(&hi2), o);
        lo2 = __hmin2(lo2, *reinterpret_cast<__half2*>(&l));
        hi2 = __hmax2(hi2, *reinterpret_cast<__half2*>(&h));
    }
    const float lo = fminf(__low2float(lo2), __high2float(lo2));
    const float hi = fmaxf(__low2float(hi2), __high2float(hi2));
    const float sc = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), QMAX);
    const float inv = __frcp_rn(sc);
    if (!live) return;
    const unsigned long long codes = quantise8<BITS>(raw, lo, sc, inv);
    if constexpr (BITS == 2) reinterpret_cast<unsigned short*>(packed)[c] = (unsigned short)codes;
    else if constexpr (BITS == 4) reinterpret_cast<unsigned*>(packed)[c] = (unsigned)codes;
    else reinterpret_cast<unsigned long long*>(packed)[c] = codes;
    if ((c & 3) == 0) {
        scale[c >> 2] = __float2half_rn(sc);
        mins[c >> 2] = __float2half_rn(lo);
    }
}

// Fast path for the key layout: the axis is strided (inner = head_dim contiguous), the group is 32 positions and
// the axis length a multiple of 32.  This is the transpose from token-major input to channel-major packed
// output.  A CTA of four warps takes a tile of 128 positions x 64 channels; warp g owns the tile's group g
// (32 positions), lane p the channel pair (2p, 2p + 1): the lane reads its pair at the 32 positions with 32
// independent 4-byte loads (each a fully coalesced 128-byte row segment for the warp, all in flight together) and
// keeps them in registers, so the input is read once and never staged: float16 minimum/maximum, float32 scale,
// codes.  Only the packed words go through shared memory, so that consecutive threads store consecutive 4-byte
// words of a channel row and every 32-byte sector of the output is written whole.
constexpr int kKeyTileTok = 128, kKeyTileCh = 64;
template <int BITS>
__global__ void __launch_bounds__(128)
quantize_pack_keytile_kernel(const __half* __restrict__ x, int64_t A, int64_t inner, int64_t nb, int64_t ng,
                             uint8_t* __restrict__ packed, __half* __restrict__ scale, __half* __restrict__ mins) {
    constexpr float QMAX = (float)((1 << BITS) - 1);
    constexpr int WPG = BITS;            // packed 32-bit words per (channel, group)
    constexpr int ROWW = 4 * WPG + 1;    // words per channel row of the output tile, padded against bank conflicts
    __shared__ unsigned out_w[kKeyTileCh][ROWW];
    __shared__ __half meta_s[2][kKeyTileCh][4];
    const int tid = threadIdx.x;
    const int64_t tiles_a = (A + kKeyTileTok - 1) / kKeyTileTok, tiles_c = inner / kKeyTileCh;
    const int64_t bc = blockIdx.x % tiles_c;
    const int64_t ba = (blockIdx.x / tiles_c) % tiles_a;
    const int64_t o = blockIdx.x / (tiles_c * tiles_a);
    const int64_t a0 = ba * kKeyTileTok;
    const int n_tok = (int)min((int64_t)kKeyTileTok, A - a0);  // a multiple of 32
    const int n_grp = n_tok / 32;

    // thread (p, g): channels 2p, 2p+1 of group g
    const int p = tid & 31, g = tid >> 5;
    if (g < n_grp) {
        const __half2* col = reinterpret_cast<const __half2*>(x + (o * A + a0 + 32 * g) * inner + bc * kKeyTileCh) + p;
        const int64_t stride = inner / 2;  // half2 per position
        __half2 v[32];
#pragma unroll
        for (int a = 0; a < 32; ++a) v[a] = __ldg(col + a * stride);
        __half2 lo2 = v[0], hi2 = v[0];
#pragma unroll
        for (int a = 1; a < 32; ++a) {
            lo2 = __hmin2(lo2, v[a]);
            hi2 = __hmax2(hi2, v[a]);
        }
        const float lo0 = __low2float(lo2), lo1 = __high2float(lo2);
        const float sc0 = __fdiv_rn(fmaxf(__fsub_rn(__low2float(hi2), lo0), 1e-8f), QMAX);
        const float sc1 = __fdiv_rn(fmaxf(__fsub_rn(__high2float(hi2), lo1), 1e-8f), QMAX);
        const float inv0 = __frcp_rn(sc0), inv1 = __frcp_rn(sc1);
        unsigned w0[WPG], w1[WPG];
#pragma unroll
        for (int k = 0; k < WPG; ++k) w0[k] = w1[k] = 0u;
#pragma unroll
        for (int k = 0; k < WPG; ++k) {  // one packed word (32 / BITS positions) of both channels at a time
            constexpr int PER = 32 / BITS;
            bool near = false;
#pragma unroll
            for (int j = 0; j < PER; ++j) {
                const float2 f = __half22float2(v[k * PER + j]);
                w0[k] = insert_bits(quantise_bits<BITS>(__fsub_rn(f.x, lo0), inv0, near), w0[k], j * BITS, BITS);
                w1[k] = insert_bits(quantise_bits<BITS>(__fsub_rn(f.y, lo1), inv1, near), w1[k], j * BITS, BITS);
            }
            if (near) {  // rare: some product was too close to a half-integer; the word again with real divisions
                w0[k] = w1[k] = 0u;
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const float2 f = __half22float2(v[k * PER + j]);
                    w0[k] |= quantise_exact(__fsub_rn(f.x, lo0), sc0, QMAX) << (j * BITS);
                    w1[k] |= quantise_exact(__fsub_rn(f.y, lo1), sc1, QMAX) << (j * BITS);
                }
            }
        }
#pragma unroll
        for (int k = 0; k < WPG; ++k) {
            out_w[2 * p][WPG * g + k] = w0[k];
            out_w[2 * p + 1][WPG * g + k] = w1[k];
        }
        meta_s[0][2 * p][g] = __float2half_rn(sc0);
        meta_s[0][2 * p + 1][g] = __float2half_rn(sc1);
        meta_s[1][2 * p][g] = __float2half_rn(lo0);
        meta_s[1][2 * p + 1][g] = __float2half_rn(lo1);
    }
    __syncthreads();

    // 3. consecutive threads store consecutive words of a channel row
    const int row_words = n_grp * WPG;
    const int64_t row0 = o * inner + bc * kKeyTileCh;
    for (int idx = tid; idx < kKeyTileCh * row_words; idx += 128) {
        const int ch = idx / row_words, w = idx - ch * row_words;
        *reinterpret_cast<unsigned*>(packed + (row0 + ch) * nb + a0 * BITS / 8 + 4 * w) = out_w[ch][w];
    }
    for (int idx = tid; idx < 2 * kKeyTileCh * n_grp; idx += 128) {
        const int which = idx / (kKeyTileCh * n_grp), rest = idx - which * (kKeyTileCh * n_grp);
        const int ch = rest / n_grp, gg = rest - ch * n_grp;
        (which ? mins : scale)[(row0 + ch) * ng + a0 / 32 + gg] = meta_s[which][ch][gg];
    }
}

template <int BITS>
__global__ void unpack_dequantize_kernel(const uint8_t* __restrict__ packed,
                                         const __half* __restrict__ scale,
                                         const __half* __restrict__ mins, int64_t outer, int64_t A,
                                         int64_t inner, int64_t gs, int64_t nb, int64_t ng,
                                         __half* __restrict__ out) {
    constexpr int VPB = 8 / BITS;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= outer * A * inner) return;
    const int64_t j = i % inner;
    const int64_t a = (i / inner) % A;
    const int64_t o = i / (inner * A);
    const int64_t row = o * inner + j;
    const float c = (float)extract_code<BITS>(packed[row * nb + a / VPB], (unsigned)(a % VPB));
    const float s = __half2float(scale[row * ng + a / gs]);
    const float m = __half2float(mins[row * ng + a / gs]);
    out[i] = __float2half_rn(__fadd_rn(__fmul_rn(c, s), m));  // two roundings, as the reference
}

int64_t gcd64(int64_t a, int64_t b) {
    while (b) {
        const int64_t t = a % b;
        a = b;
        b = t;
    }
    return a;
}

inline unsigned blocks_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads); }

}  // namespace
}  // namespace pkv

using namespace pkv;

extern "C" {

int pkv_abi_version(void) { return 2; }

int pkv_last_cuda_error(void) { return g_last_cuda_error; }

const char* pkv_strerror(int code) {
    switch (code) {
        case PKV_OK: return "ok";
        case PKV_E_BITS: return "bit width must be 2, 4 or 8";
        case PKV_E_SHAPE: return "invalid or inconsistent sizes";
        case PKV_E_NULL: return "a required pointer is NULL";
        case PKV_E_LAYOUT: return "segment layout or group size not supported";
        case PKV_E_WORKSPACE: return "scratch buffer too small";
        case PKV_E_CUDA: return "a CUDA runtime call failed";
        case PKV_E_LIMIT: return "a documented size limit was exceeded";
        default: return "unknown error";
    }
}

int pkv_device_sm_count(int device, int* sm_count) {
    if (!sm_count) return PKV_E_NULL;
    int v = 0;
    PKV_CUDA_TRY(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device));
    *sm_count = v;
    return PKV_OK;
}

int pkv_pack_low_bits(const uint8_t* codes, int64_t rows, int64_t len, int bits, uint8_t* out,
                      pkv_stream_t stream) {
    if (!valid_bits(bits)) return PKV_E_BITS;
    if (rows < 0 || len < 0) return PKV_E_SHAPE;
    const int64_t nb = ceil_div(len, 8 / bits);
    if (rows * nb == 0) return PKV_OK;
    if (!codes || !out) return PKV_E_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = blocks_for(rows * nb);
    if (bits == 2) pack_low_bits_kernel<2><<<grid, kThreads, 0, s>>>(codes, rows, len, nb, out);
    else if (bits == 4) pack_low_bits_kernel<4><<<grid, kThreads, 0, s>>>(codes, rows, len, nb, out);
    else pack_low_bits_kernel<8><<<grid, kThreads, 0, s>>>(codes, rows, len, nb, out);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int pkv_unpack_low_bits(const uint8_t* packed, int64_t rows, int64_t row_bytes, int64_t len, int bits,
                        uint8_t* out, pkv_stream_t stream) {
    if (!valid_bits(bits)) return PKV_E_BITS;
    if (rows < 0 || len < 0 || row_bytes < 0 || len > row_bytes * (8 / bits)) return PKV_E_SHAPE;
    if (rows * len == 0) return PKV_OK;
    if (!packed || !out) return PKV_E_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = blocks_for(rows * len);
    if (bits == 2) unpack_low_bits_kernel<2><<<grid, kThreads, 0, s>>>(packed, rows, row_bytes, len, out);
    else if (bits == 4) unpack_low_bits_kernel<4><<<grid, kThreads, 0, s>>>(packed, rows, row_bytes, len, out);
    else unpack_low_bits_kernel<8><<<grid, kThreads, 0, s>>>(packed, rows, row_bytes, len, out);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int pkv_quantize_pack(const void* x, int64_t outer, int64_t axis_len, int64_t inner, int bits,
                      int64_t group, uint8_t* packed, void* scale, void* mins, pkv_stream_t stream) {
    return pkv_quantize_pack_pitched(x, outer, axis_len, inner, bits, group, packed, scale, mins, 0, 0, stream);
}

int pkv_quantize_pack_pitched(const void* x, int64_t outer, int64_t axis_len, int64_t inner, int bits,
                              int64_t group, uint8_t* packed, void* scale, void* mins, int64_t packed_pitch,
                              int64_t meta_pitch, pkv_stream_t stream) {
    if (!valid_bits(bits)) return PKV_E_BITS;
    if (outer < 0 || inner < 0 || axis_len <= 0 || group <= 0 || group > axis_len) return PKV_E_SHAPE;
    if (outer * inner == 0) return PKV_OK;
    if (!x || !packed || !scale || !mins) return PKV_E_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int vpb = 8 / bits;
    const int64_t dense_nb = ceil_div(axis_len, vpb), dense_ng = ceil_div(axis_len, group);
    // row strides of the outputs: bytes of `packed`, elements of `scale` / `mins`
    const int64_t nb = packed_pitch ? packed_pitch : dense_nb, ng = meta_pitch ? meta_pitch : dense_ng;
    if (nb < dense_nb || ng < dense_ng) return PKV_E_SHAPE;
    const bool dense = nb == dense_nb && ng == dense_ng;
    const __half* xh = static_cast<const __half*>(x);
    __half* sc = static_cast<__half*>(scale);
    __half* mn = static_cast<__half*>(mins);

    const bool aligned = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0) &&
                         ((reinterpret_cast<uintptr_t>(packed) & 15u) == 0);
    if (inner == 1 && group == 32 && axis_len % 32 == 0 && aligned && dense) {
        const int64_t n_chunks = outer * (axis_len / 8);
        if (ceil_div(n_chunks, 256) > INT32_MAX) return PKV_E_LIMIT;
        const unsigned grid = (unsigned)ceil_div(n_chunks, 256);
        if (bits == 2) quantize_pack_lastdim32_kernel<2><<<grid, 256, 0, s>>>(xh, n_chunks, packed, sc, mn);
        else if (bits == 4) quantize_pack_lastdim32_kernel<4><<<grid, 256, 0, s>>>(xh, n_chunks, packed, sc, mn);
        else quantize_pack_lastdim32_kernel<8><<<grid, 256, 0, s>>>(xh, n_chunks, packed, sc, mn);
        PKV_LAUNCH_CHECK();
        return PKV_OK;
    }

    if (inner % kKeyTileCh == 0 && group == 32 && axis_len % 32 == 0 && aligned && nb % 4 == 0) {
        const int64_t blocks = outer * ceil_div(axis_len, kKeyTileTok) * (inner / kKeyTileCh);
        if (blocks > INT32_MAX) return PKV_E_LIMIT;
        const unsigned grid = (unsigned)blocks;
        if (bits == 2) quantize_pack_keytile_kernel<2><<<grid, 128, 0, s>>>(xh, axis_len, inner, nb, ng, packed, sc, mn);
        else if (bits == 4) quantize_pack_keytile_kernel<4><<<grid, 128, 0, s>>>(xh, axis_len, inner, nb, ng, packed, sc, mn);
        else quantize_pack_keytile_kernel<8><<<grid, 128, 0, s>>>(xh, axis_len, inner, nb, ng, packed, sc, mn);
        PKV_LAUNCH_CHECK();
        return PKV_OK;
    }

    // a thread's run: whole groups, whole bytes, and (when it costs nothing) >= 32 packed bytes
    const int64_t unit = group / gcd64(group, vpb) * vpb;
    int64_t per_thread = 1;
    while (unit * per_thread * bits < 32 * 8 && unit * per_thread < axis_len) per_thread *= 2;
    const int64_t run = unit * per_thread;
    const int64_t n_runs = ceil_div(axis_len, run);
    const unsigned grid = blocks_for(outer * n_runs * inner);
    if (bits == 2)
        quantize_pack_kernel<2><<<grid, kThreads, 0, s>>>(xh, outer, axis_len, inner, group, run, n_runs, nb, ng, packed, sc, mn);
    else if (bits == 4)
        quantize_pack_kernel<4><<<grid, kThreads, 0, s>>>(xh, outer, axis_len, inner, group, run, n_runs, nb, ng, packed, sc, mn);
    else
        quantize_pack_kernel<8><<<grid, kThreads, 0, s>>>(xh, outer, axis_len, inner, group, run, n_runs, nb, ng, packed, sc, mn);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int pkv_unpack_dequantize(const uint8_t* packed, const void* scale, const void* mins, int64_t outer,
                          int64_t axis_len, int64_t inner, int bits, int64_t group, void* out,
                          pkv_stream_t stream) {
    if (!valid_bits(bits)) return PKV_E_BITS;
    if (outer < 0 || inner < 0 || axis_len <= 0 || group <= 0) return PKV_E_SHAPE;
    if (outer * inner == 0) return PKV_OK;
    if (!packed || !scale || !mins || !out) return PKV_E_NULL;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int64_t nb = ceil_div(axis_len, 8 / bits), ng = ceil_div(axis_len, group);
    const unsigned grid = blocks_for(outer * axis_len * inner);
    const __half* sc = static_cast<const __half*>(scale);
    const __half* mn = static_cast<const __half*>(mins);
    __half* o = static_cast<__half*>(out);
    if (bits == 2)
        unpack_dequantize_kernel<2><<<grid, kThreads, 0, s>>>(packed, sc, mn, outer, axis_len, inner, group, nb, ng, o);
    else if (bits == 4)
        unpack_dequantize_kernel<4><<<grid, kThreads, 0, s>>>(packed, sc, mn, outer, axis_len, inner, group, nb, ng, o);
    else
        unpack_dequantize_kernel<8><<<grid, kThreads, 0, s>>>(packed, sc, mn, outer, axis_len, inner, group, nb, ng, o);
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

}  // extern "C"

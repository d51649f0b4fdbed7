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
#include <string.h>

#include "common.cuh"
#include "decode_plan.h"
#include "decode_mma.cuh"
#include "merge.cuh"

namespace pkv {
namespace {

constexpr int GMAX = 8;        // query heads served per CTA pass
constexpr int kThreads = 512;  // threads per CTA of the general kernel
constexpr int kChunk = 128;    // tokens per inner step
constexpr int kTokThreads = kThreads / kChunk;  // threads that share a token's score
constexpr int kMaxHeadDim = 256;
constexpr int kMaxParts = 8;   // token groups of the p * v phase

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

// Shared memory of the general kernel: q (float32, pre-scaled), the chunk's scores / probabilities, the running
// softmax state, then the chunk's keys and values DEQUANTISED to float16 — exactly the values the reference's
// unpack_dequantize yields (code * scale and + zero rounded separately in float32, then rounded to float16) — keys
// as [channel][token] so that one thread per token reads without bank conflicts, values as [token][channel].
constexpr int kPadK = 8, kPadV = 8;  // float16 elements of padding per staged row
inline size_t generic_smem_bytes(int hd) {
    return sizeof(float) * ((size_t)GMAX * hd + (size_t)kTokThreads * GMAX * kChunk + 3 * GMAX) +
           sizeof(__half) * ((size_t)hd * (kChunk + kPadK) + (size_t)kChunk * (hd + kPadV));
}

// Division by a run-time constant that usually is a power of two
struct Divisor {
    int d, shift;
    __device__ explicit Divisor(int d_) : d(d_), shift(-1) {
        if ((d_ & (d_ - 1)) == 0)
            for (shift = 0; (1 << shift) < d_; ++shift) {}
    }
    __device__ __forceinline__ int operator()(int x) const { return shift >= 0 ? x >> shift : x / d; }
};

__device__ __forceinline__ __half dequantise(unsigned code, __half scale, __half zero) {
    return __float2half_rn(__fadd_rn(__fmul_rn((float)code, __half2float(scale)), __half2float(zero)));
}

__global__ void __launch_bounds__(kThreads, 2)
decode_generic_kernel(const __grid_constant__ DecodeArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int hd = a.hd;
    float* q_s = smem;                    // [GMAX][hd], pre-multiplied by sm_scale
    float* p_s = q_s + GMAX * hd;         // [kTokThreads][GMAX][kChunk]: partial scores; [0] then holds the probabilities
    float* alpha_s = p_s + kTokThreads * GMAX * kChunk;  // [GMAX]
    float* m_s = alpha_s + GMAX;
    float* l_s = m_s + GMAX;
    __half* kd = reinterpret_cast<__half*>(l_s + GMAX);  // [hd][kChunk + kPadK]
    __half* vd = kd + (size_t)hd * (kChunk + kPadK);     // [kChunk][hd + kPadV]
    constexpr int KROW = kChunk + kPadK;
    const int VROW = hd + kPadV;

    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int w = blockIdx.x, kvh = blockIdx.y, hc = blockIdx.z;

    int si = 0;
    while (si + 1 < a.n_segs && w >= a.segs[si + 1].work_begin) ++si;
    const SegDev& sg = a.segs[si];
    const long long t0 = (long long)(w - sg.work_begin) * sg.split_len;
    // (a length kept in device memory is read behind everything earlier in the stream: this kernel is an ordinary launch)
    const long long S_eff = sg.len_dev ? min(sg.S, max(0LL, (long long)*sg.len_dev)) : sg.S;
    const long long t1 = min(S_eff, t0 + sg.split_len);  // an item past the end writes an empty partial (m = -inf, l = 0)

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
    // out += p * v: thread (part, d0) owns channel d0 for the tokens part, part + parts, ... of a chunk; the
    // parts are summed at the end
    const int parts = min(kMaxParts, kThreads / hd);
    const int part = tid / hd;
    const int d0 = tid - part * hd;
    const bool pv_thread = part < parts;
    float acc[GMAX];
#pragma unroll
    for (int h = 0; h < GMAX; ++h) acc[h] = 0.f;

    const int kbits = sg.kbits, vbits = sg.vbits;
    const int kvpb = 8 / kbits;
    const long long S = sg.S;
    const __half zero_h = __float2half_rn(0.f);

    for (long long c0 = t0; c0 < t1; c0 += kChunk) {
        const int nvalid = (int)min((long long)kChunk, t1 - c0);
        __syncthreads();  // the previous chunk's tiles are no longer read (and q_s / m_s are set, first time round)
        // ---- stage the chunk.  A work item is one code BYTE (8 / bits consecutive elements that share a scale and a
        // zero whenever the group size is a multiple of that count, which every caller's is); consecutive threads take
        // consecutive bytes of the memory layout at hand.  Index arithmetic is 32-bit and, where the sizes are powers
        // of two, shifts.
        if (sg.kind == PKV_SEG_KIVI) {
            const long long nbK = sg.k_pitch, ngK = sg.km_pitch;
            const uint8_t* kp = sg.kp + (size_t)kvh * hd * nbK;
            const __half* ks = sg.ks + (size_t)kvh * hd * ngK;
            const __half* km = sg.km + (size_t)kvh * hd * ngK;
            if (c0 % kvpb == 0 && sg.kgs % kvpb == 0) {
                // keys: channel rows, tokens along the row; kChunk / kvpb bytes of every row belong to the chunk
                const int bpr = kChunk / kvpb;  // a power of two
                const Divisor by_bpr(bpr), by_group(sg.kgs);
                const long long byte0 = c0 / kvpb, group0 = c0 / sg.kgs;
                const int in_group0 = (int)(c0 - group0 * sg.kgs);
                // the loads of a batch of work items are issued together, then the batch is dequantised and stored:
                // a CTA often has a single chunk, so nothing else hides the latency of a load
                constexpr int B = 8;
                const int total = hd * bpr;
                for (int base = tid; base < total; base += kThreads * B) {
                    unsigned byte[B];
                    __half sc[B], zr[B];
#pragma unroll
                    for (int u = 0; u < B; ++u) {
                        const int idx = base + u * kThreads;
                        const int d = by_bpr(idx), tok = (idx - d * bpr) * kvpb;
                        byte[u] = 0u, sc[u] = zr[u] = zero_h;
                        if (idx < total && tok < nvalid) {
                            const long long g = group0 + by_group(in_group0 + tok);
                            byte[u] = kp[(size_t)d * nbK + byte0 + (idx - d * bpr)];
                            sc[u] = ks[(size_t)d * ngK + g];
                            zr[u] = km[(size_t)d * ngK + g];
                        }
                    }
#pragma unroll
                    for (int u = 0; u < B; ++u) {
                        const int idx = base + u * kThreads;
                        if (idx >= total) break;
                        const int d = by_bpr(idx), tok = (idx - d * bpr) * kvpb;
                        __half* dst = kd + d * KROW + tok;
                        for (int e = 0; e < kvpb; ++e)
                            dst[e] = tok + e < nvalid ? dequantise(extract_code_rt(byte[u], e, kbits), sc[u], zr[u]) : zero_h;
                    }
                }
            } else {  // a chunk that starts inside a byte, or groups that split one: element by element
                const int tok = tid % kChunk;  // thread (tok, sub) walks channels sub, sub + kTokThreads, ...
                const long long n = c0 + tok;
                const long long byte_idx = n / kvpb, grp = n / sg.kgs;
                const unsigned pos = (unsigned)(n % kvpb);
                for (int d = tid / kChunk; d < hd; d += kTokThreads) {
                    __half val = zero_h;
                    if (tok < nvalid)
                        val = dequantise(extract_code_rt(kp[(size_t)d * nbK + byte_idx], pos, kbits),
                                         ks[(size_t)d * ngK + grp], km[(size_t)d * ngK + grp]);
                    kd[d * KROW + tok] = val;
                }
            }
        } else if (sg.kind == PKV_SEG_FP16) {
            const __half* kr = reinterpret_cast<const __half*>(sg.kp) + (size_t)kvh * sg.head_stride + (size_t)c0 * hd;
            for (int idx = tid; idx < hd * kChunk; idx += kThreads) {
                const int tok = idx / hd, d = idx - tok * hd;
                kd[d * KROW + tok] = tok < nvalid ? kr[(size_t)tok * hd + d] : zero_h;
            }
        }
        // rows of tokens with channels along the row: values of both packed layouts, keys of the per-token layout
        auto stage_token_rows = [&](const uint8_t* codes, const __half* scale, const __half* zero, size_t row0, int bits,
                                    int gs, bool transposed) {
            const int vpb = 8 / bits;
            const int nb = (hd + vpb - 1) / vpb, ng = (hd + gs - 1) / gs;
            const bool shared_meta = gs % vpb == 0 && hd % vpb == 0;
            const Divisor by_nb(nb), by_group(gs);
            constexpr int B = 8;
            const int total = nb * kChunk;
            for (int base = tid; base < total; base += kThreads * B) {
                unsigned byte[B];
                __half sc[B], zr[B];
#pragma unroll
                for (int u = 0; u < B; ++u) {  // all loads of the batch first
                    const int idx = base + u * kThreads;
                    const int tok = by_nb(idx), d = (idx - tok * nb) * vpb;
                    byte[u] = 0u, sc[u] = zr[u] = zero_h;
                    if (idx < total && tok < nvalid) {
                        byte[u] = codes[(row0 + tok) * nb + (idx - tok * nb)];
                        sc[u] = scale[(row0 + tok) * ng + by_group(d)];
                        zr[u] = zero[(row0 + tok) * ng + by_group(d)];
                    }
                }
#pragma unroll
                for (int u = 0; u < B; ++u) {
                    const int idx = base + u * kThreads;
                    if (idx >= total) break;
                    const int tok = by_nb(idx), d = (idx - tok * nb) * vpb;
                    const bool live = tok < nvalid;
                    for (int e = 0; e < vpb && d + e < hd; ++e) {
                        __half s_e = sc[u], z_e = zr[u];
                        if (live && !shared_meta) {
                            s_e = scale[(row0 + tok) * ng + by_group(d + e)];
                            z_e = zero[(row0 + tok) * ng + by_group(d + e)];
                        }
                        const __half val = live ? dequantise(extract_code_rt(byte[u], e, bits), s_e, z_e) : zero_h;
                        if (transposed) kd[(d + e) * KROW + tok] = val;
                        else vd[tok * VROW + d + e] = val;
                    }
                }
            }
        };
        if (sg.kind == PKV_SEG_PER_TOKEN)
            stage_token_rows(sg.kp, sg.ks, sg.km, (size_t)kvh * S + c0, kbits, sg.kgs, true);
        if (sg.kind == PKV_SEG_FP16) {
            const __half* vr = reinterpret_cast<const __half*>(sg.vp) + (size_t)kvh * sg.head_stride + (size_t)c0 * hd;
            for (int idx = tid; idx < hd * kChunk; idx += kThreads) {
                const int tok = idx / hd, d = idx - tok * hd;
                vd[tok * VROW + d] = tok < nvalid ? vr[(size_t)tok * hd + d] : zero_h;
            }
        } else {
            stage_token_rows(sg.vp, sg.vs, sg.vm, (sg.kind == PKV_SEG_KIVI ? (size_t)kvh * sg.v_head_tokens : (size_t)kvh * S) + c0,
                             vbits, sg.vgs, false);
        }
        __syncthreads();

        // ---- phase 1: kTokThreads threads per token, each over a quarter of the channels; partial scores of all heads
        {
            const int tok = tid % kChunk, sub = tid / kChunk;
            const long long n = c0 + tok;
            const bool counts = tok < nvalid && (sg.slot_tokens == 0 || (int)(n % sg.slot_tokens) < sg.slot_valid);
            float dot[GMAX];
#pragma unroll
            for (int h = 0; h < GMAX; ++h) dot[h] = 0.f;
            if (counts) {
                const int per = hd / kTokThreads;  // head_dim is a multiple of 4
                for (int d = sub * per; d < (sub + 1) * per; ++d) {
                    const float kv = __half2float(kd[d * KROW + tok]);
#pragma unroll
                    for (int h = 0; h < GMAX; ++h) dot[h] = fmaf(q_s[h * hd + d], kv, dot[h]);
                }
            }
#pragma unroll
            for (int h = 0; h < GMAX; ++h) p_s[(sub * GMAX + h) * kChunk + tok] = counts ? dot[h] : -INFINITY;
        }
        __syncthreads();

        // ---- phase 2: online softmax bookkeeping, one warp per head
        for (int h = wid; h < nh; h += kThreads / 32) {
            float v[kChunk / 32];
            float mx = -INFINITY;
#pragma unroll
            for (int i = 0; i < kChunk / 32; ++i) {
                float sum = 0.f;  // (-inf in every part for a token that does not count)
#pragma unroll
                for (int sub = 0; sub < kTokThreads; ++sub) sum += p_s[(sub * GMAX + h) * kChunk + lane + 32 * i];
                v[i] = sum;
                mx = fmaxf(mx, v[i]);
            }
            mx = warp_max(mx);
            const float m_old = m_s[h];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < kChunk / 32; ++i) {
                const float p = m_new == -INFINITY ? 0.f : expf(v[i] - m_new);  // -inf -> 0; a chunk of masked slots only
                p_s[h * kChunk + lane + 32 * i] = p;
                sum += p;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float alpha = m_new == -INFINITY ? 1.f : expf(m_old - m_new);  // first chunk: exp(-inf) = 0
                alpha_s[h] = alpha;
                m_s[h] = m_new;
                l_s[h] = l_s[h] * alpha + sum;
            }
        }
        __syncthreads();

        // ---- phase 3: acc += p * v
        if (pv_thread) {
#pragma unroll
            for (int h = 0; h < GMAX; ++h) acc[h] *= alpha_s[h];
            for (int i = part; i < nvalid; i += parts) {
                const float vv = __half2float(vd[i * VROW + d0]);
#pragma unroll
                for (int h = 0; h < GMAX; ++h) acc[h] = fmaf(p_s[h * kChunk + i], vv, acc[h]);
            }
        }
    }

    if (parts > 1) {  // sum the token groups (the staged tiles are free now)
        __syncthreads();
        float* red = reinterpret_cast<float*>(kd);  // [parts - 1][GMAX][hd]
        if (pv_thread && part > 0)
#pragma unroll
            for (int h = 0; h < GMAX; ++h) red[((size_t)(part - 1) * GMAX + h) * hd + d0] = acc[h];
        __syncthreads();
        if (part == 0)
            for (int p = 1; p < parts; ++p)
#pragma unroll
                for (int h = 0; h < GMAX; ++h) acc[h] += red[((size_t)(p - 1) * GMAX + h) * hd + d0];
    }
    __syncthreads();  // m_s / l_s of the last chunk (or their initial values, for an empty item)

    const size_t widx = (size_t)(a.work_offset + w);
    if (tid < nh) {
        a.pm[widx * a.Hq + h0 + tid] = m_s[tid];
        a.pl[widx * a.Hq + h0 + tid] = l_s[tid];
    }
    if (part == 0) {
#pragma unroll
        for (int h = 0; h < GMAX; ++h)
            if (h < nh) a.pacc[(widx * a.Hq + h0 + h) * hd + d0] = acc[h];
    }
}

__global__ void __launch_bounds__(kMergeThreads)
merge_partials_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                      const float* __restrict__ pacc, int n_parts, size_t ml_stride, size_t acc_stride, int hd,
                      __half* __restrict__ out, float* __restrict__ m_out,
                      float* __restrict__ l_out, float* __restrict__ acc_out) {
    // When launched as a programmatic dependent of the split-K kernel this grid may already be resident while
    // that kernel finishes; wait here for its results (a no-op for an ordinary launch).
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();  // the next kernel of the stream may start its own prologue
    merge_parts(pm, pl, pacc, n_parts, ml_stride, acc_stride, hd, blockIdx.x, out, m_out, l_out, acc_out);
}

int check_segments(const pkv_segment_t* segs, int n_segs, int Hq, int Hkv, int hd) {
    if (!segs) return PKV_E_NULL;
    if (n_segs <= 0 || n_segs > PKV_MAX_SEGMENTS) return PKV_E_LIMIT;
    if (Hq <= 0 || Hkv <= 0 || hd <= 0 || Hq % Hkv) return PKV_E_SHAPE;
    if (hd > kMaxHeadDim) return PKV_E_LIMIT;
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
        if (s.seq_len_dev && s.kind != PKV_SEG_KIVI) return PKV_E_LAYOUT;
        if (!valid_bits(s.k_bits) || !valid_bits(s.v_bits)) return PKV_E_BITS;
        if (s.k_group <= 0 || s.v_group <= 0) return PKV_E_LAYOUT;
        if (!s.k_scale || !s.k_mins || !s.v_scale || !s.v_mins) return PKV_E_NULL;
        if (s.slot_tokens || s.slot_valid || (s.kind != PKV_SEG_FP16 && s.head_stride)) {
            if (s.kind != PKV_SEG_KIVI) return PKV_E_LAYOUT;
            if (s.slot_tokens || s.slot_valid) {
                if ((s.slot_tokens != 32 && s.slot_tokens != 64) || s.slot_valid <= 0 || s.slot_valid > s.slot_tokens ||
                    s.k_group != 32 || s.seq_len % s.slot_tokens)
                    return PKV_E_LAYOUT;
            }
            if (s.head_stride && s.head_stride < s.seq_len) return PKV_E_SHAPE;
        }
        if (s.k_row_pitch || s.k_meta_pitch) {
            if (s.kind != PKV_SEG_KIVI) return PKV_E_LAYOUT;
            if ((s.k_row_pitch && s.k_row_pitch < ceil_div(s.seq_len * s.k_bits, 8)) ||
                (s.k_meta_pitch && s.k_meta_pitch < ceil_div(s.seq_len, s.k_group)))
                return PKV_E_SHAPE;
        }
    }
    return PKV_OK;
}

}  // namespace

// bytes-proportional cost of streaming a segment
static double seg_cost(const pkv_segment_t& s) {
    return (double)s.seq_len * (s.kind == PKV_SEG_FP16 ? 16 : s.k_bits);
}

// Device image of a segment descriptor (work-list fields left at zero).
static SegDev seg_dev_of(const pkv_segment_t& s) {
    SegDev d = {};
    d.kp = static_cast<const uint8_t*>(s.k_packed);
    d.ks = static_cast<const __half*>(s.k_scale);
    d.km = static_cast<const __half*>(s.k_mins);
    d.vp = static_cast<const uint8_t*>(s.v_packed);
    d.vs = static_cast<const __half*>(s.v_scale);
    d.vm = static_cast<const __half*>(s.v_mins);
    d.S = s.seq_len;
    d.head_stride = s.head_stride;
    d.kind = s.kind;
    d.fresh = (s.flags & PKV_SEG_FLAG_FRESH) != 0;
    d.kbits = s.kind == PKV_SEG_FP16 ? 8 : s.k_bits;
    d.vbits = s.kind == PKV_SEG_FP16 ? 8 : s.v_bits;
    d.kgs = s.kind == PKV_SEG_FP16 ? 1 : s.k_group;
    d.vgs = s.kind == PKV_SEG_FP16 ? 1 : s.v_group;
    d.v_head_tokens = s.seq_len;
    d.len_dev = s.seq_len_dev;
    if (s.kind == PKV_SEG_KIVI) {
        d.k_pitch = s.k_row_pitch ? s.k_row_pitch : ceil_div(s.seq_len * s.k_bits, 8);
        d.km_pitch = s.k_meta_pitch ? s.k_meta_pitch : ceil_div(s.seq_len, s.k_group);
        if (s.head_stride) d.v_head_tokens = s.head_stride;
        d.slot_tokens = s.slot_tokens;
        d.slot_valid = s.slot_valid;
    }
    return d;
}

DecodePlan plan_decode(const pkv_segment_t* segs, int n_segs, int Hq, int Hkv, int hd, int sm_count) {
    DecodePlan plan;
    const int G = Hq / Hkv;
    const int head_chunks = (G + GMAX - 1) / GMAX;
    sm_count = std::max(sm_count, 1);
    long long generic_tokens = 0;
    double fast_cost = 0.0;
    std::vector<char> is_fast(n_segs);
    // The tensor-core kernels take KIVI + float16 or per-token + float16 segments in one launch, not KIVI and
    // per-token together: in such a mix (no caller of the reference builds one) the per-token segments go to the
    // general kernel.
    bool any_kivi = false;
    for (int i = 0; i < n_segs; ++i) any_kivi |= segs[i].kind == PKV_SEG_KIVI;
    for (int i = 0; i < n_segs; ++i) {
        is_fast[i] = mma::eligible(segs[i], Hq, Hkv, hd) && !(any_kivi && segs[i].kind == PKV_SEG_PER_TOKEN);
        if (is_fast[i]) fast_cost += seg_cost(segs[i]);
        else generic_tokens += segs[i].seq_len;
    }
    // general kernel: two CTAs of 16 warps per SM over its share of the layer
    const long long target = std::max<long long>(1, (2LL * sm_count) / ((long long)Hkv * head_chunks));
    // tensor-core kernel: one CTA per SM (it owns the SM's shared memory), one wave
    const double fast_ctas_per_head = std::max(1.0, (double)sm_count * mma::CTAS_PER_SM / Hkv);
    for (int i = 0; i < n_segs; ++i) {
        const pkv_segment_t& s = segs[i];
        SegDev d = seg_dev_of(s);
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
            if (s.kind == PKV_SEG_KIVI && s.num_splits <= 0 && d.split_len > 4) d.split_len = (d.split_len + 3) / 4 * 4;
            d.n_splits = (int)ceil_div(tiles, d.split_len);
            d.work_begin = plan.fast_work;
            plan.fast_work += d.n_splits;
            plan.fast.push_back(d);
            plan.fast_index.push_back(i);
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

int pkv_decode_launches(const pkv_segment_t* segs, int n_segs, int num_q_heads, int num_kv_heads, int head_dim,
                        int sm_count, int* launches) {
    if (!launches) return PKV_E_NULL;
    const int rc = check_segments(segs, n_segs, num_q_heads, num_kv_heads, head_dim);
    if (rc != PKV_OK) return rc;
    const DecodePlan plan = plan_decode(segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_count);
    const int fast = (int)((plan.fast.size() + kMaxInlineSegs - 1) / kMaxInlineSegs);
    const int generic = (int)((plan.generic.size() + kMaxInlineSegs - 1) / kMaxInlineSegs);
    *launches = fast + generic + 1;  // the split-K launches and the merge
    return PKV_OK;
}

}  // extern "C"

namespace pkv {
// Validation, planning and the split-K launches of one decode call; the partials land in `workspace`.
int run_splitk(const void* q, const pkv_segment_t* segs, int n_segs, int num_q_heads, int num_kv_heads,
               int head_dim, float sm_scale, int sm_count, void* workspace, size_t workspace_bytes,
               cudaStream_t s, SplitKParts* parts) {
    const int rc = check_segments(segs, n_segs, num_q_heads, num_kv_heads, head_dim);
    if (rc != PKV_OK) return rc;
    if (!q || !workspace) return PKV_E_NULL;
    const DecodePlan plan = plan_decode(segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_count);
    const size_t W = (size_t)plan.total_work();
    const size_t need = W * num_q_heads * (head_dim + 2) * sizeof(float);
    if (workspace_bytes < need) return PKV_E_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(workspace) & 15u) return PKV_E_LAYOUT;
    // acc rows first: they are read as float4 and must start on 16 bytes
    float* pacc = static_cast<float*>(workspace);
    float* pm = pacc + W * num_q_heads * head_dim;
    float* pl = pm + W * num_q_heads;
    // function attributes are per device: set them the first time this thread launches on a device
    static thread_local bool carved_on[64] = {};
    int device = 0;
    PKV_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= 64) return PKV_E_LIMIT;
    bool& carved = carved_on[device];
    if (!carved) {
        // keep the SM's shared-memory split where the tensor-core kernel wants it, so alternating kernels do not
        // force a reconfiguration between launches
        cudaFuncSetAttribute(merge_partials_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(decode_generic_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        PKV_CUDA_TRY(cudaFuncSetAttribute(decode_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)generic_smem_bytes(kMaxHeadDim)));
        carved = true;
    }
    const int G = num_q_heads / num_kv_heads;

    // tensor-core kernel over the KIVI and float16 segments it takes
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
            a.segs[i].key_tma = 0;
        }
        // the longest KIVI segments of the launch get tensor maps (a short cold segment is one small super-tile)
        for (int slot = 0; slot < mma::kMaxKeyMaps; ++slot) {
            int best = -1;
            for (int i = 0; i < cnt; ++i)
                if (a.segs[i].kind == PKV_SEG_KIVI && !a.segs[i].key_tma && a.segs[i].S >= 256 &&
                    (best < 0 || a.segs[i].S > a.segs[best].S))
                    best = i;
            if (best < 0) break;
            a.segs[best].key_tma = mma::make_key_maps(segs[plan.fast_index[first + best]], num_kv_heads, &a.kmaps[slot])
                                       ? slot + 1 : -1;
        }
        for (int i = 0; i < cnt; ++i)
            if (a.segs[i].key_tma < 0) a.segs[i].key_tma = 0;  // could not be described: cp.async
        bool per_token = false;
        for (int i = 0; i < cnt; ++i) per_token |= a.segs[i].kind == PKV_SEG_PER_TOKEN;
        const int rc2 = per_token ? mma::launch_per_token(a, launch_work, num_kv_heads, s)
                                  : mma::launch(a, launch_work, num_kv_heads, s);
        if (rc2 != PKV_OK) return rc2;
    }
    // layout-generic kernel over everything else (float16 hot tier, per-token layout, ragged shapes)
    const size_t smem = generic_smem_bytes(head_dim);
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
    parts->n = W;
    parts->pm = pm;
    parts->pl = pl;
    parts->pacc = pacc;
    return PKV_OK;
}
}  // namespace pkv

extern "C" {

int pkv_decode_attention(const void* q, const pkv_segment_t* segs, int n_segs, int num_q_heads,
                         int num_kv_heads, int head_dim, float sm_scale, int sm_count, void* workspace,
                         size_t workspace_bytes, void* out, float* m, float* l, float* acc,
                         pkv_stream_t stream) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    SplitKParts parts;
    const int rc = run_splitk(q, segs, n_segs, num_q_heads, num_kv_heads, head_dim, sm_scale, sm_count, workspace,
                              workspace_bytes, s, &parts);
    if (rc != PKV_OK) return rc;
    const size_t W = parts.n;
    float *pm = parts.pm, *pl = parts.pl, *pacc = parts.pacc;
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
        PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_partials_kernel, cpm, cpl, cpacc, (int)W, (size_t)num_q_heads,
                                        (size_t)num_q_heads * head_dim, head_dim, static_cast<__half*>(out), m, l,
                                        acc));
    }
    return PKV_OK;
}

int pkv_merge_partials(const float* m, const float* l, const float* acc, int n_parts, int num_q_heads,
                       int head_dim, void* out, float* m_out, float* l_out, float* acc_out,
                       pkv_stream_t stream) {
    return pkv_merge_partials_strided(m, l, acc, n_parts, num_q_heads, (int64_t)num_q_heads * head_dim,
                                      num_q_heads, head_dim, out, m_out, l_out, acc_out, stream);
}

int pkv_merge_partials_strided(const float* m, const float* l, const float* acc, int n_parts, int64_t ml_stride,
                               int64_t acc_stride, int num_q_heads, int head_dim, void* out, float* m_out,
                               float* l_out, float* acc_out, pkv_stream_t stream) {
    if (!m || !l || !acc) return PKV_E_NULL;
    if (n_parts <= 0 || num_q_heads <= 0 || head_dim <= 0) return PKV_E_SHAPE;
    if (ml_stride < num_q_heads || acc_stride < (int64_t)num_q_heads * head_dim) return PKV_E_SHAPE;
    if (head_dim > 256) return PKV_E_LIMIT;
    if (head_dim % 4 || acc_stride % 4 || (reinterpret_cast<uintptr_t>(acc) & 15u)) return PKV_E_LAYOUT;
    merge_partials_kernel<<<num_q_heads, kMergeThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        m, l, acc, n_parts, (size_t)ml_stride, (size_t)acc_stride, head_dim, static_cast<__half*>(out), m_out, l_out,
        acc_out);
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

// ---------------------------------------------------------------------------------------------
// Batched decode (serving): many sequences, one split-K launch, one merge launch.
//
// The table the planner writes is position independent (offsets, no host pointers) so the caller can
// copy it to the device with any copy it likes and keep it there while lengths and pointers stay the
// same:  [BatchHeader][SegDev x n_segs][BatchWork x n_work][BatchRange x batch], each array 16-byte aligned.
namespace pkv {
namespace {

constexpr uint32_t kBatchMagic = 0x42564b50u;  // "PKVB"

struct BatchHeader {
    uint32_t magic;
    int32_t batch, n_segs, n_work, n_parts;
    int32_t Hq, Hkv, hd;
    uint32_t off_segs, off_work, off_ranges, bytes;
    uint32_t pad[4];
};
static_assert(sizeof(BatchHeader) == 64, "header is one 64-byte block");

// partials [part_begin, part_begin + n_parts) belong to one sequence
struct BatchRange {
    int32_t part_begin, n_parts;
};

inline size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

__global__ void __launch_bounds__(kMergeThreads)
merge_batched_kernel(const float* __restrict__ pm, const float* __restrict__ pl, const float* __restrict__ pacc,
                     const BatchRange* __restrict__ ranges, int Hq, int hd, __half* __restrict__ out) {
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();
    const int seq = blockIdx.y;
    const BatchRange r = ranges[seq];
    merge_parts(pm + (size_t)r.part_begin * Hq, pl + (size_t)r.part_begin * Hq,
                pacc + (size_t)r.part_begin * Hq * hd, r.n_parts, (size_t)Hq, (size_t)Hq * hd, hd, blockIdx.x,
                out + (size_t)seq * Hq * hd, nullptr, nullptr, nullptr);
}

// Tiles per work item.  `per_sm` is the layer's work per SM in 64-token tiles.  Few tiles per SM: one wave,
// the tiles spread evenly.  Many: about three waves of long items; the short cold and hot segments, sorted to
// the end of the work list, fill the tail (more, shorter items cost more: every item pays its first-load
// latency, warp merge and partial write once).  Items are whole super-tiles (what the CTA's warps compute side by side).
int item_tiles(double per_sm) {
    constexpr int kSuper = mma::Cfg<2>::NSUB;  // tiles the CTA's warps compute side by side
    const int waves = (int)std::max(1.0, std::min(3.0, per_sm / kSuper));
    int t = (int)std::ceil(per_sm / waves);
    t = std::max(1, std::min(t, 4096));
    if (t >= kSuper) t = (t + kSuper / 2) / kSuper * kSuper;
    else if (t > 4) t = (t + 3) / 4 * 4;
    return t;
}

}  // namespace
}  // namespace pkv

extern "C" int pkv_decode_batch_plan(const pkv_segment_t* segs, const int32_t* seg_offsets, int batch,
                                     int num_q_heads, int num_kv_heads, int head_dim, int sm_count, void* table,
                                     size_t table_capacity, size_t* table_bytes, size_t* workspace_bytes) {
    if (!segs || !seg_offsets || !table_bytes || !workspace_bytes) return PKV_E_NULL;
    if (batch <= 0 || seg_offsets[0] != 0) return PKV_E_SHAPE;
    for (int i = 0; i < batch; ++i)
        if (seg_offsets[i + 1] <= seg_offsets[i]) return PKV_E_SHAPE;  // every sequence attends to something
    const int n_segs = seg_offsets[batch];
    if (n_segs > (1 << 20)) return PKV_E_LIMIT;
    for (int first = 0; first < n_segs; first += PKV_MAX_SEGMENTS) {
        const int rc = check_segments(segs + first, std::min(PKV_MAX_SEGMENTS, n_segs - first), num_q_heads,
                                      num_kv_heads, head_dim);
        if (rc != PKV_OK) return rc;
    }
    double units = 0.0;  // 64-token tiles (a float16 tile of 32 tokens moves about as many bytes per token x4)
    for (int i = 0; i < n_segs; ++i) {
        if (!mma::eligible(segs[i], num_q_heads, num_kv_heads, head_dim) || segs[i].kind == PKV_SEG_PER_TOKEN)
            return PKV_E_LAYOUT;
        if (mma::tiles_of(segs[i]) > INT32_MAX) return PKV_E_LIMIT;
        units += (double)mma::tiles_of(segs[i]);
    }
    const int per_item = item_tiles(units * num_kv_heads / std::max(sm_count, 1));

    std::vector<mma::BatchWork> work;
    std::vector<BatchRange> ranges(batch);
    int parts = 0;
    for (int b = 0; b < batch; ++b) {
        ranges[b].part_begin = parts;
        for (int si = seg_offsets[b]; si < seg_offsets[b + 1]; ++si) {
            const long long tiles = mma::tiles_of(segs[si]);
            long long n = ceil_div(tiles, per_item);
            long long len = ceil_div(tiles, n);
            // an item that starts on a multiple of four tiles keeps the key scale rows 16-byte aligned
            if (segs[si].kind != PKV_SEG_FP16 && len > 4) len = (len + 3) / 4 * 4;
            n = ceil_div(tiles, len);
            for (long long k = 0; k < n; ++k) {
                mma::BatchWork w = {};
                w.seg = si;
                w.seq = b;
                w.tile_begin = (int)(k * len);
                w.n_tiles = (int)std::min(len, tiles - k * len);
                w.part = parts++;
                work.push_back(w);
            }
            if (parts > (1 << 24)) return PKV_E_LIMIT;
        }
        ranges[b].n_parts = parts - ranges[b].part_begin;
    }
    // longest first: the hardware hands CTAs out in index order, so short items fill the tail
    std::stable_sort(work.begin(), work.end(),
                     [](const mma::BatchWork& a, const mma::BatchWork& b) { return a.n_tiles > b.n_tiles; });

    BatchHeader h = {};
    h.magic = kBatchMagic;
    h.batch = batch;
    h.n_segs = n_segs;
    h.n_work = (int32_t)work.size();
    h.n_parts = parts;
    h.Hq = num_q_heads;
    h.Hkv = num_kv_heads;
    h.hd = head_dim;
    h.off_segs = (uint32_t)sizeof(BatchHeader);
    h.off_work = (uint32_t)align16(h.off_segs + (size_t)n_segs * sizeof(SegDev));
    h.off_ranges = (uint32_t)align16(h.off_work + work.size() * sizeof(mma::BatchWork));
    h.bytes = (uint32_t)align16(h.off_ranges + (size_t)batch * sizeof(BatchRange));
    *table_bytes = h.bytes;
    *workspace_bytes = (size_t)parts * num_q_heads * (head_dim + 2) * sizeof(float);
    if (!table) return PKV_OK;
    if (table_capacity < h.bytes) return PKV_E_WORKSPACE;
    if (reinterpret_cast<uintptr_t>(table) & 15u) return PKV_E_LAYOUT;
    char* base = static_cast<char*>(table);
    memset(base, 0, h.bytes);
    memcpy(base, &h, sizeof(h));
    SegDev* sd = reinterpret_cast<SegDev*>(base + h.off_segs);
    for (int i = 0; i < n_segs; ++i) sd[i] = seg_dev_of(segs[i]);
    memcpy(base + h.off_work, work.data(), work.size() * sizeof(mma::BatchWork));
    memcpy(base + h.off_ranges, ranges.data(), (size_t)batch * sizeof(BatchRange));
    return PKV_OK;
}

extern "C" int pkv_decode_chunk_plan(const pkv_segment_t* segs, int n_segments, int chunk_len, int num_q_heads,
                                     int num_kv_heads, int head_dim, int sm_count, void* table,
                                     size_t table_capacity, size_t* table_bytes, size_t* workspace_bytes) {
    if (!segs) return PKV_E_NULL;
    if (n_segments <= 0 || n_segments > PKV_MAX_SEGMENTS || chunk_len <= 0 || chunk_len > (1 << 16)) return PKV_E_SHAPE;
    const pkv_segment_t& hot = segs[n_segments - 1];
    if (hot.kind != PKV_SEG_FP16 || hot.seq_len < chunk_len) return PKV_E_SHAPE;
    // query i of the chunk is a "sequence" of its own: the same packed segments, and the float16 tier cut off
    // behind the token the query belongs to
    std::vector<pkv_segment_t> all((size_t)n_segments * chunk_len);
    std::vector<int32_t> offsets(chunk_len + 1);
    for (int i = 0; i < chunk_len; ++i) {
        offsets[i] = i * n_segments;
        for (int k = 0; k < n_segments; ++k) all[(size_t)i * n_segments + k] = segs[k];
        all[(size_t)i * n_segments + n_segments - 1].seq_len = hot.seq_len - (chunk_len - 1 - i);
        all[(size_t)i * n_segments + n_segments - 1].seq_len_dev = nullptr;  // the causal cut is a host length
    }
    offsets[chunk_len] = chunk_len * n_segments;
    return pkv_decode_batch_plan(all.data(), offsets.data(), chunk_len, num_q_heads, num_kv_heads, head_dim, sm_count,
                                 table, table_capacity, table_bytes, workspace_bytes);
}

extern "C" int pkv_decode_attention_batched(const void* q, const void* table_host, const void* table_device,
                                            float sm_scale, void* workspace, size_t workspace_bytes, void* out,
                                            pkv_stream_t stream) {
    if (!q || !table_host || !table_device || !workspace || !out) return PKV_E_NULL;
    BatchHeader h;
    memcpy(&h, table_host, sizeof(h));
    if (h.magic != kBatchMagic || h.batch <= 0 || h.n_work <= 0 || h.n_parts <= 0) return PKV_E_SHAPE;
    if ((reinterpret_cast<uintptr_t>(table_device) | reinterpret_cast<uintptr_t>(workspace)) & 15u) return PKV_E_LAYOUT;
    const size_t P = (size_t)h.n_parts;
    if (workspace_bytes < P * h.Hq * (h.hd + 2) * sizeof(float)) return PKV_E_WORKSPACE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* pacc = static_cast<float*>(workspace);
    float* pm = pacc + P * h.Hq * h.hd;
    float* pl = pm + P * h.Hq;
    const char* dev = static_cast<const char*>(table_device);

    mma::BatchArgs a;
    a.q = static_cast<const __half*>(q);
    a.pm = pm;
    a.pl = pl;
    a.pacc = pacc;
    a.Hq = h.Hq;
    a.Hkv = h.Hkv;
    a.G = h.Hq / h.Hkv;
    a.sm_scale = sm_scale;
    a.segs = reinterpret_cast<const SegDev*>(dev + h.off_segs);
    a.work = reinterpret_cast<const mma::BatchWork*>(dev + h.off_work);
    const int rc = mma::launch_batched(a, h.n_work, h.Hkv, s);
    if (rc != PKV_OK) return rc;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)h.Hq, (unsigned)h.batch);
    cfg.blockDim = dim3(kMergeThreads);
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const float* cpm = pm;
    const float* cpl = pl;
    const float* cpacc = pacc;
    const BatchRange* ranges = reinterpret_cast<const BatchRange*>(dev + h.off_ranges);
    PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, merge_batched_kernel, cpm, cpl, cpacc, ranges, (int)h.Hq, (int)h.hd,
                                    static_cast<__half*>(out)));
    return PKV_OK;
}

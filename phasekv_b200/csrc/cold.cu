// Lazy cold-tier maintenance for one layer in ONE launch: value-norm top-k selection of the
// aged hot tokens, quantise+pack of the kept ones (K along tokens, V along head_dim), and
// compaction of the hot buffers.  The reference does this with about fifty torch launches
// (phasekv_cache.py:322-340).  One CTA owns one (batch, KV head) row; the work is a few hundred
// tokens, so the kernel is latency-bound by design and keeps everything in one block.
//
// Selection rule: squared L2 norm of V over head_dim accumulated in float32, the `keep` largest
// kept, ties towards the lower position, result in ascending position order.
#include "common.cuh"

namespace pkv {
namespace {

constexpr int kColdThreads = 256;
constexpr int kMaxAged = 4096;  // aged tokens handled per row (shared-memory bound)

// Quantise positions [a_begin, a_end) of a line of length A whose element a is load(a).
// a_begin is a multiple of lcm(gs, 8/BITS): whole groups, whole bytes.
template <int BITS, class Load>
__device__ void quantize_run(Load load, int a_begin, int a_end, int A, int gs, uint8_t* prow,
                             __half* srow, __half* mrow) {
    constexpr int VPB = 8 / BITS;
    constexpr float QMAX = (float)((1 << BITS) - 1);
    unsigned cur = 0;
    for (int g0 = a_begin; g0 < a_end; g0 += gs) {
        const int g1 = min(g0 + gs, A);
        float lo = load(g0), hi = lo;
        for (int a = g0 + 1; a < g1; ++a) {
            const float v = load(a);
            lo = fminf(lo, v);
            hi = fmaxf(hi, v);
        }
        const float sc = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), QMAX);
        const float inv = __frcp_rn(sc);
        for (int a = g0; a < g1; ++a) {
            float qv = quantise_round(__fsub_rn(load(a), lo), sc, inv);
            qv = fminf(fmaxf(qv, 0.f), QMAX);
            const int pos = a % VPB;
            cur |= (unsigned)qv << (pos * BITS);
            if (pos == VPB - 1 || a == A - 1) {
                prow[a / VPB] = (uint8_t)cur;
                cur = 0;
            }
        }
        srow[g0 / gs] = __float2half_rn(sc);
        mrow[g0 / gs] = __float2half_rn(lo);
    }
}

__device__ __forceinline__ int gcd_i(int a, int b) {
    while (b) {
        const int t = a % b;
        a = b;
        b = t;
    }
    return a;
}

// Where one layer's cooling step reads and writes.  The outputs may be dense tensors of their own or a slot of a
// pre-allocated arena: rows of the key outputs are k_pitch bytes / k_meta_pitch elements apart, the value
// outputs of consecutive (batch, head) rows are v_row_tokens token rows apart.
struct ColdLayer {
    __half* hot_k;
    __half* hot_v;
    uint8_t* k_packed;
    __half* k_scale;
    __half* k_mins;
    uint8_t* v_packed;
    __half* v_scale;
    __half* v_mins;
    long long* indices;
};
static_assert(sizeof(ColdLayer) == sizeof(pkv_cold_layer_t), "the device table is an array of pkv_cold_layer_t");

// Grid (rows, layers): every layer of a model cools in the same launch (all layers hold the same number of hot
// tokens).  `slot_*`: byte / element / token-row offsets of this event's slot inside the layers' arenas, added to
// the table's base pointers (zero for dense outputs).
template <int BITS>
__global__ void __launch_bounds__(kColdThreads)
cold_select_pack_kernel(const ColdLayer* __restrict__ layers, const ColdLayer single, int capacity, int hd,
                        int hot_len, int aged, int keep, int gs_k, int gs_v, long long k_pitch,
                        long long k_meta_pitch, long long v_row_tokens, long long slot_k_bytes,
                        long long slot_k_groups, long long slot_v_tokens) {
    constexpr int VPB = 8 / BITS;
    const ColdLayer L = layers != nullptr ? layers[blockIdx.y] : single;  // one layer travels in the parameters
    __half* const hot_k = L.hot_k;
    __half* const hot_v = L.hot_v;
    long long* const indices = L.indices;
    const int v_nb = (hd + VPB - 1) / VPB, v_ng = (hd + gs_v - 1) / gs_v;
    uint8_t* const k_packed = L.k_packed + slot_k_bytes;
    __half* const k_scale = L.k_scale + slot_k_groups;
    __half* const k_mins = L.k_mins + slot_k_groups;
    uint8_t* const v_packed = L.v_packed + slot_v_tokens * v_nb;
    __half* const v_scale = L.v_scale + slot_v_tokens * v_ng;
    __half* const v_mins = L.v_mins + slot_v_tokens * v_ng;
    __shared__ float n2[kMaxAged];
    __shared__ int sel[kMaxAged];
    __shared__ int warp_tot[kColdThreads / 32];
    __shared__ int running;

    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    __half* hk = hot_k + (size_t)row * capacity * hd;
    __half* hv = hot_v + (size_t)row * capacity * hd;

    if (keep < aged) {
        // 1. squared value norms, one warp per token
        for (int t = wid; t < aged; t += kColdThreads / 32) {
            float s = 0.f;
            for (int d = lane; d < hd; d += 32) {
                const float v = __half2float(hv[(size_t)t * hd + d]);
                s = fmaf(v, v, s);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            if (lane == 0) n2[t] = s;
        }
        if (tid == 0) running = 0;
        __syncthreads();
        // 2. rank counting + ordered compaction of the kept positions
        for (int base = 0; base < aged; base += kColdThreads) {
            const int t = base + tid;
            int flag = 0;
            if (t < aged) {
                const unsigned mine = order_key(n2[t]);  // total order, NaN largest (torch.topk's)
                int rank = 0;
                for (int j = 0; j < aged; ++j) {
                    const unsigned o = order_key(n2[j]);
                    rank += (o > mine) || (o == mine && j < t);
                }
                flag = rank < keep;
            }
            const unsigned ballot = __ballot_sync(0xffffffffu, flag);
            const int before = __popc(ballot & ((1u << lane) - 1u));
            if (lane == 0) warp_tot[wid] = __popc(ballot);
            __syncthreads();
            int offset = running;
            for (int w = 0; w < wid; ++w) offset += warp_tot[w];
            if (flag) sel[offset + before] = t;
            __syncthreads();
            if (tid == 0) {
                int tot = 0;
                for (int w = 0; w < kColdThreads / 32; ++w) tot += warp_tot[w];
                running += tot;
            }
            __syncthreads();
        }
    } else {
        for (int t = tid; t < aged; t += kColdThreads) sel[t] = t;
        __syncthreads();
    }
    if (indices)
        for (int p = tid; p < keep; p += kColdThreads) indices[(size_t)row * keep + p] = sel[p];

    // 3. V: per kept token, groups along head_dim
    {
        const int nb = (hd + VPB - 1) / VPB, ng = (hd + gs_v - 1) / gs_v;
        const int unit = gs_v / gcd_i(gs_v, VPB) * VPB;
        const int runs = (hd + unit - 1) / unit;
        for (int i = tid; i < keep * runs; i += kColdThreads) {
            const int p = i / runs, r = i % runs;
            const __half* src = hv + (size_t)sel[p] * hd;
            auto load = [&](int a) { return __half2float(src[a]); };
            quantize_run<BITS>(load, r * unit, min(hd, (r + 1) * unit), hd, gs_v,
                               v_packed + ((size_t)row * v_row_tokens + p) * nb,
                               v_scale + ((size_t)row * v_row_tokens + p) * ng,
                               v_mins + ((size_t)row * v_row_tokens + p) * ng);
        }
    }
    // 4. K: per channel, groups along the kept tokens
    {
        const int unit = gs_k / gcd_i(gs_k, VPB) * VPB;
        const int runs = (keep + unit - 1) / unit;
        for (int i = tid; i < hd * runs; i += kColdThreads) {
            const int d = i % hd, r = i / hd;
            auto load = [&](int a) { return __half2float(hk[(size_t)sel[a] * hd + d]); };
            quantize_run<BITS>(load, r * unit, min(keep, (r + 1) * unit), keep, gs_k,
                               k_packed + ((size_t)row * hd + d) * k_pitch,
                               k_scale + ((size_t)row * hd + d) * k_meta_pitch,
                               k_mins + ((size_t)row * hd + d) * k_meta_pitch);
        }
    }
    __syncthreads();
    // 5. move the surviving hot tokens [aged, hot_len) to the start; chunks ascend, each chunk is
    //    read completely before it is written, so overlapping ranges are safe.
    const int total = (hot_len - aged) * hd;  // elements; rows are dense so this is a flat shift
    const int shift = aged * hd;
    if ((hd & 7) == 0 && ((reinterpret_cast<uintptr_t>(hk) | reinterpret_cast<uintptr_t>(hv)) & 15u) == 0) {
        // 16-byte words (row starts are 16-byte aligned when hd is a multiple of 8 and the buffers are)
        const int words = total >> 3, wshift = shift >> 3;
        uint4* k4 = reinterpret_cast<uint4*>(hk);
        uint4* v4 = reinterpret_cast<uint4*>(hv);
        for (int base = 0; base < words; base += kColdThreads) {
            const int i = base + tid;
            uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
            if (i < words) {
                a = k4[i + wshift];
                b = v4[i + wshift];
            }
            __syncthreads();
            if (i < words) {
                k4[i] = a;
                v4[i] = b;
            }
            __syncthreads();
        }
        return;
    }
    for (int base = 0; base < total; base += kColdThreads) {
        const int i = base + tid;
        __half a = __float2half(0.f), b = a;
        if (i < total) {
            a = hk[i + shift];
            b = hv[i + shift];
        }
        __syncthreads();
        if (i < total) {
            hk[i] = a;
            hv[i] = b;
        }
        __syncthreads();
    }
}

}  // namespace
}  // namespace pkv

using namespace pkv;

namespace {
int launch_cold(const ColdLayer* table_dev, const ColdLayer& single, int n_layers, int64_t rows, int64_t capacity, int head_dim, int64_t hot_len,
                int64_t aged, int64_t keep, int bits, int64_t group, int64_t k_pitch, int64_t k_meta_pitch,
                int64_t v_row_tokens, int64_t slot_k_bytes, int64_t slot_k_groups, int64_t slot_v_tokens,
                cudaStream_t s) {
    const int gs_k = (int)std::min<int64_t>(group, keep), gs_v = (int)std::min<int64_t>(group, head_dim);
    const dim3 grid((unsigned)rows, (unsigned)n_layers);
#define PKV_COLD_LAUNCH(B)                                                                                     \
    cold_select_pack_kernel<B><<<grid, kColdThreads, 0, s>>>(table_dev, single, (int)capacity, head_dim, (int)hot_len, \
                                                             (int)aged, (int)keep, gs_k, gs_v, k_pitch, k_meta_pitch, \
                                                             v_row_tokens, slot_k_bytes, slot_k_groups, slot_v_tokens)
    if (bits == 2) PKV_COLD_LAUNCH(2);
    else if (bits == 4) PKV_COLD_LAUNCH(4);
    else PKV_COLD_LAUNCH(8);
#undef PKV_COLD_LAUNCH
    PKV_LAUNCH_CHECK();
    return PKV_OK;
}

int check_cold(int64_t rows, int64_t capacity, int head_dim, int64_t hot_len, int64_t aged, int64_t keep, int bits,
               int64_t group) {
    if (!valid_bits(bits)) return PKV_E_BITS;
    if (rows <= 0 || head_dim <= 0 || group <= 0 || aged <= 0 || keep <= 0 || keep > aged ||
        aged > hot_len || hot_len > capacity)
        return PKV_E_SHAPE;
    if (aged > kMaxAged || capacity * (int64_t)head_dim > INT32_MAX || rows > 65535) return PKV_E_LIMIT;
    return PKV_OK;
}
}  // namespace

extern "C" int pkv_cold_select_pack_layers(const pkv_cold_layer_t* layers /* device */, int n_layers, int64_t rows,
                                           int64_t capacity, int head_dim, int64_t hot_len, int64_t aged, int64_t keep,
                                           int bits, int64_t group, int64_t k_row_pitch, int64_t k_meta_pitch,
                                           int64_t v_row_tokens, int64_t slot_k_bytes, int64_t slot_k_groups,
                                           int64_t slot_v_tokens, pkv_stream_t stream) {
    const int rc = check_cold(rows, capacity, head_dim, hot_len, aged, keep, bits, group);
    if (rc != PKV_OK) return rc;
    if (!layers) return PKV_E_NULL;
    if (n_layers <= 0 || n_layers > 65535) return PKV_E_LIMIT;
    const int64_t gs_k = std::min<int64_t>(group, keep);
    if (k_row_pitch < ceil_div(keep * bits, 8) || k_meta_pitch < ceil_div(keep, gs_k) || v_row_tokens < keep ||
        slot_k_bytes < 0 || slot_k_groups < 0 || slot_v_tokens < 0)
        return PKV_E_SHAPE;
    return launch_cold(reinterpret_cast<const ColdLayer*>(layers), ColdLayer{}, n_layers, rows, capacity, head_dim, hot_len, aged,
                       keep, bits, group, k_row_pitch, k_meta_pitch, v_row_tokens, slot_k_bytes, slot_k_groups,
                       slot_v_tokens, static_cast<cudaStream_t>(stream));
}

extern "C" int pkv_cold_select_pack(void* hot_k, void* hot_v, int64_t rows, int64_t capacity, int head_dim,
                                    int64_t hot_len, int64_t aged, int64_t keep, int bits, int64_t group,
                                    uint8_t* k_packed, void* k_scale, void* k_mins, uint8_t* v_packed,
                                    void* v_scale, void* v_mins, int64_t* indices, pkv_stream_t stream) {
    if (!valid_bits(bits)) return PKV_E_BITS;
    if (rows <= 0 || head_dim <= 0 || group <= 0 || aged <= 0 || keep <= 0 || keep > aged ||
        aged > hot_len || hot_len > capacity)
        return PKV_E_SHAPE;
    if (aged > kMaxAged || capacity * (int64_t)head_dim > INT32_MAX) return PKV_E_LIMIT;
    if (!hot_k || !hot_v || !k_packed || !k_scale || !k_mins || !v_packed || !v_scale || !v_mins)
        return PKV_E_NULL;
    // one layer, dense outputs
    const int64_t gs_k = std::min<int64_t>(group, keep);
    ColdLayer one = {static_cast<__half*>(hot_k), static_cast<__half*>(hot_v), k_packed, static_cast<__half*>(k_scale),
                     static_cast<__half*>(k_mins), v_packed, static_cast<__half*>(v_scale), static_cast<__half*>(v_mins),
                     reinterpret_cast<long long*>(indices)};
    return launch_cold(nullptr, one, 1, rows, capacity, head_dim, hot_len, aged, keep, bits, group,
                       ceil_div(keep * bits, 8), ceil_div(keep, gs_k), keep, 0, 0, 0, static_cast<cudaStream_t>(stream));
}

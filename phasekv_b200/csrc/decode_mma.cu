// Tensor-core split-K decode kernel for KIVI-packed segments; see decode_mma.cuh for the scheme.
#include <math.h>

#include "decode_mma.cuh"

namespace pkv {
namespace mma {
namespace {

constexpr float kLog2e = 1.4426950408889634f;
#ifndef PKV_K_UNROLL
#define PKV_K_UNROLL 4
#endif
constexpr int kKUnroll = PKV_K_UNROLL;
#ifndef PKV_KEY_TMA
#define PKV_KEY_TMA 1
#endif
// Keys through tiled TMA copies (tensor maps made on the host) where the layout allows; 0 = cp.async everywhere.
constexpr bool kKeyTma = PKV_KEY_TMA != 0;
#ifndef PKV_TMA_MIN_SUPER
#define PKV_TMA_MIN_SUPER 3
#endif
// CTAs with fewer super-tiles than this keep cp.async: with one or two super-tiles the barrier set-up costs what
// the copies save
constexpr int kTmaMinSuper = PKV_TMA_MIN_SUPER;
#ifndef PKV_PAIR_SPLIT
#define PKV_PAIR_SPLIT 1
#endif
// warp pairs share the tiles of short super-tiles (a pair pays the per-tile q loads, zero-term MMAs and state
// rescale twice, so full super-tiles keep one warp per tile)
constexpr bool kPairSplit = PKV_PAIR_SPLIT != 0;
#ifndef PKV_SMALL_FIRST
#define PKV_SMALL_FIRST 1
#endif
constexpr bool kSmallFirst = PKV_SMALL_FIRST != 0;  // the partial super-tile of a CTA's range is processed first
#ifndef PKV_PV_RESIDUAL_2BIT
#define PKV_PV_RESIDUAL_2BIT 0
#endif
// Low part of p * value_scale for 2-bit codes (wider codes always get it: their codes reach 15 or 255)
constexpr bool kPvResidual2 = PKV_PV_RESIDUAL_2BIT != 0;

struct WarpState {
    float m[2];        // running max (log2 domain) of heads 2t, 2t+1
    float l[2];        // this lane's share of the running sum of exp
    float o[4][2][4];  // out accumulators: [dim group][M-tile][C fragment]
    float pm[4];       // sum_n p * v_zero, rows = dim groups (lanes g < 4)
};

// ---- loads.  Shared-memory layouts are the memory layouts (16-byte cp.async; 4-byte copies throttled
// the load/store unit, and a copy costs one shared-memory write per 32-byte sector it gathers, so the
// scattered key rows are fetched in chunks as long as the super-tile allows):
//   K buffer : codes as boxes [channel][64 bytes, chunks swizzled], scale [channel][MROW bytes], zero likewise   (CTA-wide)
//   V stage  : codes [token row, one pad row per 8 tokens][hd*BITS/8 bytes], scale [token][4 f16], zero likewise
template <int BITS>
struct KSrc {
    using C = Cfg<BITS>;
    const uint8_t* kp;
    const char* ks;
    const char* km;
    long long nbK, ngK2;  // bytes per key code row / per key scale row
    bool meta16;          // scale rows can move in 16-byte copies
    bool aligned;         // code rows start on 16 bytes: cp.async path; otherwise load_sync

    __device__ KSrc(const SegDev& sg, int kvh, long long tile0) {
        nbK = sg.k_pitch;
        ngK2 = sg.km_pitch * 2;
        kp = sg.kp + (size_t)kvh * HD * nbK;
        ks = reinterpret_cast<const char*>(sg.ks) + (size_t)kvh * HD * ngK2;
        km = reinterpret_cast<const char*>(sg.km) + (size_t)kvh * HD * ngK2;
        // 16-byte copies need rows that start on 16 bytes and hold whole tiles (dense rows do when S is a
        // multiple of the tile, padded rows always); the partial last tile of a padded segment reads padding,
        // which only reaches masked tokens.
        const long long tiles = (sg.S + C::T - 1) / C::T;
        aligned = (nbK & 15) == 0 && (ngK2 & 3) == 0 && nbK >= tiles * C::KRB && ngK2 >= tiles * (C::NG * 2);
        meta16 = aligned && (ngK2 & 15) == 0 && (tile0 & 3) == 0;
    }

    // Ragged segments (any length, so any row alignment): the same K buffer image built with ordinary
    // loads.  A 16-byte chunk is read as aligned 32-bit words and realigned with funnel shifts; bytes past
    // the end of a row come out as the neighbouring row's bytes or zero and belong to masked tokens only.
    // Reads stay inside [tensor start, tensor end rounded up to 4 bytes).
    __device__ __forceinline__ void load_sync(long long tile, int n_sub, char* kb, int tid) const {
        const int cpr = n_sub * (C::KRB / 16);
        for (int idx = tid; idx < HD * cpr; idx += NTHREADS) {
            const int row = idx / cpr, ch = idx - row * cpr;
            const long long off = tile * C::KRB + 16 * ch;
            const long long valid = nbK - off;  // bytes of this row at and after the chunk start
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (valid > 0) {
                const uintptr_t ga = reinterpret_cast<uintptr_t>(kp + (size_t)row * nbK + off);
                const unsigned mis = (unsigned)(ga & 3u);
                const unsigned* wp = reinterpret_cast<const unsigned*>(ga - mis);
                const int last = (int)((mis + (valid < 16 ? valid : 16) - 1) >> 2);
                unsigned w[5];
#pragma unroll
                for (int i = 0; i < 5; ++i) w[i] = i <= last ? __ldg(wp + i) : 0u;
                const unsigned sh = 8u * mis;
                v.x = __funnelshift_r(w[0], w[1], sh);
                v.y = __funnelshift_r(w[1], w[2], sh);
                v.z = __funnelshift_r(w[2], w[3], sh);
                v.w = __funnelshift_r(w[3], w[4], sh);
            }
            *reinterpret_cast<uint4*>(kb + key_chunk_offset(row, ch)) = v;
        }
        const long long moff = tile * (C::NG * 2);
        for (int idx = tid; idx < HD * n_sub; idx += NTHREADS) {
            const int row = idx / n_sub, w = idx - row * n_sub;
            const long long off = moff + 4 * w;
            const long long valid = ngK2 - off;
            unsigned sv = 0u, mv = 0u;
            if (valid > 0) {
                const unsigned short* sp = reinterpret_cast<const unsigned short*>(ks + (size_t)row * ngK2 + off);
                const unsigned short* mp = reinterpret_cast<const unsigned short*>(km + (size_t)row * ngK2 + off);
                sv = __ldg(sp);
                mv = __ldg(mp);
                if (valid > 2) {
                    sv |= (unsigned)__ldg(sp + 1) << 16;
                    mv |= (unsigned)__ldg(mp + 1) << 16;
                }
            }
            *reinterpret_cast<unsigned*>(kb + C::OFF_KS + row * C::MROW + 4 * w) = sv;
            *reinterpret_cast<unsigned*>(kb + C::OFF_KM + row * C::MROW + 4 * w) = mv;
        }
    }

    // keys of tiles [tile, tile + n_sub) into the K buffer at `kb`; every thread of the CTA takes part.
    // FULL (n_sub == NSUB) makes every divisor a compile-time constant.
    template <bool FULL>
    __device__ __forceinline__ void issue_impl(long long tile, int n_sub_rt, unsigned kb, int tid) const {
        const int n_sub = FULL ? C::NSUB : n_sub_rt;
        const int cpr = n_sub * (C::KRB / 16);
        if (FULL && kHoisted) {
            issue_full_codes(tile, kb, tid);
        } else {
            const uint8_t* src = kp + tile * C::KRB;
            for (int idx = tid; idx < HD * cpr; idx += NTHREADS) {
                const int row = idx / cpr, ch = idx - row * cpr;
                cp_async16(kb + key_chunk_offset(row, ch), src + (size_t)row * nbK + 16 * ch);
            }
        }
        const long long moff = tile * (C::NG * 2);
        if (meta16) {
            const int row_bytes = n_sub * C::NG * 2, cpm = (row_bytes + 15) / 16;
            for (int idx = tid; idx < HD * cpm; idx += NTHREADS) {
                const int row = idx / cpm, ch = idx - row * cpm;
                const unsigned nbytes = min(16, row_bytes - 16 * ch);
                const size_t off = (size_t)row * ngK2 + moff + 16 * ch;
                cp_async16_zfill(kb + C::OFF_KS + row * C::MROW + 16 * ch, ks + off, nbytes);
                cp_async16_zfill(kb + C::OFF_KM + row * C::MROW + 16 * ch, km + off, nbytes);
            }
        } else {
            for (int idx = tid; idx < HD * n_sub; idx += NTHREADS) {
                const int row = idx / n_sub, w = idx - row * n_sub;
                const size_t off = (size_t)row * ngK2 + moff + 4 * w;
                cp_async4(kb + C::OFF_KS + row * C::MROW + 4 * w, ks + off);
                cp_async4(kb + C::OFF_KM + row * C::MROW + 4 * w, km + off);
            }
        }
    }
    // The same image through tiled TMA copies, issued by ONE thread: one 128-row x 64-byte box per 64 bytes of
    // the super-tile's rows (delivered with the 64-byte swizzle, i.e. in the layout key_chunk_offset describes)
    // and one box each for the scales and zeros.  Bytes that lie past the end of a row arrive as zeros.  The
    // first coordinate of every box is a multiple of 16 bytes because super-tiles start on multiples of 4 tiles.
    __device__ __forceinline__ void issue_tma(const KeyMaps* maps, int kvh, long long tile, int n_sub, unsigned kb,
                                              unsigned bar) const {
        const int nbox = (n_sub * C::KRB + C::KBOX - 1) / C::KBOX;
        mbar_arrive_expect_tx(bar, (unsigned)(nbox * C::KBOX_BYTES + 2 * HD * C::MROW));
        const int y = kvh * HD;
        for (int b = 0; b < nbox; ++b)
            tma_load_2d(kb + b * C::KBOX_BYTES, &maps->codes, (int)(tile * C::KRB) + b * C::KBOX, y, bar);
        tma_load_2d(kb + C::OFF_KS, &maps->scale, (int)(tile * C::NG), y, bar);
        tma_load_2d(kb + C::OFF_KM, &maps->mins, (int)(tile * C::NG), y, bar);
    }

    // The codes of a FULL super-tile with the addressing hoisted: the thread count is a multiple of the 16-byte chunks
    // per row, so a thread copies the same chunk column of rows row0, row0 + RPI, ... and both addresses advance by a
    // constant per pass (the swizzle of a chunk depends on (row >> 1) & 3, which RPI, a multiple of 8, leaves alone).
    static constexpr int CPR = C::NSUB * (C::KRB / 16);
    static constexpr int RPI = NTHREADS / CPR;
    static constexpr bool kHoisted = NTHREADS % CPR == 0 && RPI % 8 == 0;
    __device__ __forceinline__ void issue_full_codes(long long tile, unsigned kb, int tid) const {
        const int row0 = tid / CPR, ch = tid - row0 * CPR;
        const uint8_t* src = kp + tile * C::KRB + (size_t)row0 * nbK + 16 * ch;
        const unsigned dst = kb + key_chunk_offset(row0, ch);
        const size_t step = (size_t)RPI * nbK;
#pragma unroll
        for (int i = 0; i < (HD + RPI - 1) / RPI; ++i)
            if (HD % RPI == 0 || row0 + RPI * i < HD) cp_async16(dst + RPI * C::KBOX * i, src + step * i);
    }

    __device__ __forceinline__ void issue(long long tile, int n_sub, unsigned kb, int tid) const {
        if (n_sub == C::NSUB) issue_impl<true>(tile, n_sub, kb, tid);
        else issue_impl<false>(tile, n_sub, kb, tid);
    }
};

template <int BITS>
struct VSrc {
    using C = Cfg<BITS>;
    static constexpr int CPT = C::VWPT / 4;  // 16-byte chunks per token row
    static constexpr int TPI = 32 / CPT;     // tokens covered by one warp instruction
    const uint8_t* vc;
    const char* vs;
    const char* vm;
    unsigned d_vc;
    int lane;
    bool meta16;  // this head's scale rows start on 16 bytes

    // codes [heads][head_tokens][hd * BITS / 8 bytes], scale and zero [heads][head_tokens][4] float16: the values of
    // a KIVI segment, or the keys or the values of a per-token segment
    __device__ VSrc(const uint8_t* codes, const __half* scale, const __half* zero, long long head_tokens, int kvh,
                    int lane_) : lane(lane_) {
        meta16 = (((long long)kvh * head_tokens) & 1) == 0;
        vc = codes + (size_t)kvh * head_tokens * (C::VWPT * 4) + 16 * lane;
        const int lt = lane / CPT;
        d_vc = (lt + lt / 8) * (C::VWPT * 4) + 16 * (lane % CPT);
        vs = reinterpret_cast<const char*>(scale + (size_t)kvh * head_tokens * 4) + 16 * lane;
        vm = reinterpret_cast<const char*>(zero + (size_t)kvh * head_tokens * 4) + 16 * lane;
    }
    __device__ VSrc(const SegDev& sg, int kvh, int lane_) : VSrc(sg.vp, sg.vs, sg.vm, sg.v_head_tokens, kvh, lane_) {}

    // values of one tile into the stage at `sa`; one warp.  Rows of tokens >= n_valid are zero-filled
    // (their probabilities are zero, but garbage scales could be NaN).
    __device__ __forceinline__ void issue(long long tile, unsigned sa, int n_valid) const {
        const uint8_t* v = vc + tile * (C::T * C::VWPT * 4);
        const long long off = tile * (C::T * 8);
        if (n_valid >= C::T && meta16) {
#pragma unroll
            for (int it = 0; it < C::T / TPI; ++it) {
                const int tok0 = it * TPI;
                cp_async16(sa + d_vc + (tok0 + tok0 / 8) * (C::VWPT * 4), v + 512 * it);
            }
            cp_async16(sa + C::OFF_VS + 16 * lane, vs + off);
            cp_async16(sa + C::OFF_VM + 16 * lane, vm + off);
        } else {
            const int lt = lane / CPT;
#pragma unroll
            for (int it = 0; it < C::T / TPI; ++it) {
                const int tok0 = it * TPI;
                const bool ok = tok0 + lt < n_valid;
                cp_async16_zfill(sa + d_vc + (tok0 + tok0 / 8) * (C::VWPT * 4), ok ? v + 512 * it : vc, ok ? 16u : 0u);
            }
            // scale / zero rows are 8 bytes per token and, for an odd number of tokens per head, only 8-byte
            // aligned: two 8-byte copies per lane (tokens lane and lane + 32)
#pragma unroll
            for (int k = 0; k < 2; ++k) {
                const int tok = lane + 32 * k;
                const unsigned nb = tok < n_valid ? 8u : 0u;
                const long long so = nb ? off + 8 * tok - 16 * lane : -16 * (long long)lane;
                cp_async8_zfill(sa + C::OFF_VS + 8 * tok, vs + so, nb);
                cp_async8_zfill(sa + C::OFF_VM + 8 * tok, vm + so, nb);
            }
        }
    }
};

// Which of the eight 16-channel steps of the score contraction need the low part of q * scale.
// B = q * key_scale is rounded to float16 (relative error 2^-11); what the rounding drops only matters where
// |B| is large, i.e. on channels with outlier keys, so the second MMA that feeds it is issued only for steps
// that contain a channel with max_heads|q| * scale >= kResidualMin in one of the tile's two key groups.
// Bit 4kk of the result is set when step kk needs the low part.
// Steps that go without it add at most 2^-11 * kResidualMin * 3 to a raw score per channel.
constexpr unsigned kResidualMinBits = 0x4800u;  // 8.0 as float16
template <int BITS>
__device__ __forceinline__ unsigned residual_steps(const char* kb, int sub, const char* qabs, int lane) {
    using C = Cfg<BITS>;
    if (BITS != 2) return 0xffffffffu;  // wider codes multiply the rounding error by up to 15 or 255: always
    // Lane l looks at channels l, l + 32, l + 64, l + 96 (steps l/16 + 2i): consecutive lanes read consecutive
    // scale rows, the tile's word of the row (its two groups) is picked afterwards.
    const char* s = kb + C::OFF_KS + lane * C::MROW + 16 * (sub >> 2);
    const char* qa = qabs + 4 * lane;
    unsigned need = 0u;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        unsigned w;
        if (C::MROW % 16 == 0) {
            const uint4 row = ldp128(s + 32 * i * C::MROW);
            const int k = sub & 3;
            w = k == 0 ? row.x : k == 1 ? row.y : k == 2 ? row.z : row.w;
        } else {
            w = ldp32(s + 32 * i * C::MROW + 4 * (sub & 3));
        }
        const unsigned m = hmul2(w, ldp32(qa + 128 * i));
        // both factors are non-negative, so the float16 order is the integer order; NaN compares as large
        const unsigned big = ((m & 0x7fff7fffu) + (0x8000u - kResidualMinBits) * 0x10001u) & 0x80008000u;
        const unsigned b = __ballot_sync(0xffffffffu, big != 0u);
        need |= ((b & 0xffffu) ? 1u : 0u) << (8 * i);        // step 2i     -> bit 4 * (2i)
        need |= ((b >> 16) ? 1u : 0u) << (8 * i + 4);        // step 2i + 1 -> bit 4 * (2i + 1)
    }
    return need;
}

template <int BITS, int NGRP>
__device__ __forceinline__ void softmax_pv(float (&sacc)[NGRP * 2][4], const char* sa, WarpState& st,
                                           const LaneSel<BITS>& ls, int lane, int n_valid, int slot, int g_off);

// NGRP = 2: the whole 64-token tile.  NGRP = 1: only its 32-token group `g_off` (two warps share a tile when a
// super-tile has few tiles, so that the tail of a CTA's range is spread over all warps).
template <int BITS, int NGRP = 2>
__device__ __forceinline__ void compute_tile(const char* kb, int sub, const char* sa, const char* q_lane, float c_qk,
                                             WarpState& st, const LaneSel<BITS>& ls, int lane, int n_valid,
                                             const char* qabs, int slot, int g_off = 0) {
    using C = Cfg<BITS>;
    static_assert(C::NG == 2 && (NGRP == 1 || NGRP == 2), "a tile is two key groups");
    const int t = lane & 3;
    const unsigned res_steps = residual_steps<BITS>(kb, sub, qabs, lane);

    // ---------------- scores: S^T tile-by-tile, M = 16 tokens, N = 8 heads, K = channels
    float sacc[NGRP * 2][4];
#pragma unroll
    for (int i = 0; i < NGRP * 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
    float bacc[4] = {0.f, 0.f, 0.f, 0.f};
    // k-step kk contracts channels 16kk + {2t, 2t+1, 2t+8, 2t+9} in this lane (the natural MMA order)
    // key codes of this lane: channel rows 2t (+1, +8, +9) + 16kk; the lane's word of group G of tile `sub` lies in
    // 16-byte chunk ck of the super-tile row, stored at chunk (ck & 3) ^ ((row >> 1) & 3) = (ck & 3) ^ t of box ck >> 2
    const char* k_lane[2];
#pragma unroll
    for (int G = 0; G < 2; ++G) {
        const int in_tile = 4 * G * BITS + 4 * (int)ls.word;  // byte offset inside the tile's KRB bytes of a row
        const int ck = sub * (C::KRB / 16) + (in_tile >> 4);
        k_lane[G] = kb + (ck >> 2) * C::KBOX_BYTES + 2 * t * C::KBOX + ((((ck & 3) ^ t) & 3) << 4) + (in_tile & 15);
    }
    // Key scales and zeros of a super-tile sit as [channel][group] float16 rows; the MMA wants, per lane, the pair
    // (channel 2t, channel 2t + 1) of ONE group.  ldmatrix with .trans delivers exactly that pairing: from an 8 x 8
    // block (8 channels x the 8 groups of a 16-byte row chunk) lane (g, t) receives (block[2t][g], block[2t+1][g]),
    // i.e. the channel pair of group column g.  For the zeros that IS the A operand of the zero-term MMA (rows =
    // the chunk's 8 groups); for the scales the pair of the tile's own group is fetched from the lanes that hold
    // its column with one shuffle.  One ldmatrix.x4 covers 32 channels = two k-steps.
    const int mcol = 2 * (sub & 3);  // column of the tile's first group inside its 16-byte chunk
    const unsigned meta_row = (unsigned)__cvta_generic_to_shared(kb) + (8 * (lane >> 3) + (lane & 7)) * C::MROW +
                              16 * (sub >> 2);
    // partially unrolled: the fully unrolled loop made the kernel instruction-fetch bound on short contexts
#pragma unroll (kKUnroll / 2)
    for (int kp = 0; kp < 4; ++kp) {
        unsigned zs[4], zm[4];
        ldmatrix_x4_trans(meta_row + C::OFF_KS + 32 * kp * C::MROW, zs[0], zs[1], zs[2], zs[3]);
        ldmatrix_x4_trans(meta_row + C::OFF_KM + 32 * kp * C::MROW, zm[0], zm[1], zm[2], zm[3]);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int kk = 2 * kp + hh;
            const bool residual = ((res_steps >> (4 * kk)) & 1u) != 0u;  // the same in every lane
            const unsigned qf0 = ldp32(q_lane + 32 * kk);       // head g, channels 16kk + 2t, +1
            const unsigned qf1 = ldp32(q_lane + 32 * kk + 16);  // channels 16kk + 2t + 8, +9
            // sum_d q[h,d] * zero[d,G] for the 8 groups of the chunk (rows 0..7); the tile's own rows are read back
            mma16816(bacc, zm[2 * hh], 0u, zm[2 * hh + 1], 0u, qf0, qf1);
#pragma unroll
            for (int e = 0; e < NGRP; ++e) {
                const int G = NGRP == 2 ? e : g_off;
                const int src = 4 * (mcol + G) + t;  // the lane that holds this lane's channel pair of group G
                const unsigned s0p = __shfl_sync(0xffffffffu, zs[2 * hh], src);
                const unsigned s1p = __shfl_sync(0xffffffffu, zs[2 * hh + 1], src);
                const unsigned b0 = hmul2(qf0, s0p), b1 = hmul2(qf1, s1p);
                uint4 kc;
                const char* kl = NGRP == 2 ? k_lane[e] : (g_off ? k_lane[1] : k_lane[0]);
                kc.x = ldp32(kl + (16 * kk + 0) * C::KBOX);
                kc.y = ldp32(kl + (16 * kk + 1) * C::KBOX);
                kc.z = ldp32(kl + (16 * kk + 8) * C::KBOX);
                kc.w = ldp32(kl + (16 * kk + 9) * C::KBOX);
                unsigned ra[4], rb[4];
                extract4<BITS>(kc.x, kc.y, ls, ra);
                extract4<BITS>(kc.z, kc.w, ls, rb);
                mma16816(sacc[2 * e + 0], ra[0], ra[1], rb[0], rb[1], b0, b1);
                mma16816(sacc[2 * e + 1], ra[2], ra[3], rb[2], rb[3], b0, b1);
                // q*scale does not fit float16 exactly; its rounding error (2^-11 of products that reach
                // tens on outlier channels) would dominate the score error, so on steps with such a channel
                // the residual goes through the tensor core as well (the A operands are already built)
                if (residual) {
                    const unsigned b0l = hfma2_residual(qf0, s0p, b0), b1l = hfma2_residual(qf1, s1p, b1);
                    mma16816(sacc[2 * e + 0], ra[0], ra[1], rb[0], rb[1], b0l, b1l);
                    mma16816(sacc[2 * e + 1], ra[2], ra[3], rb[2], rb[3], b0l, b1l);
                }
            }
        }
    }

    // undo the power-of-two code scaling, add the zero terms, go to the log2 domain
#pragma unroll
    for (int e = 0; e < NGRP; ++e) {
        const int G = NGRP == 2 ? e : g_off;
        const float bias0 = __shfl_sync(0xffffffffu, bacc[0], 4 * (mcol + G) + t);
        const float bias1 = __shfl_sync(0xffffffffu, bacc[1], 4 * (mcol + G) + t);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float* s = sacc[2 * e + j];
            s[0] = (s[0] * unscale<BITS>(2 * j) + bias0) * c_qk;
            s[1] = (s[1] * unscale<BITS>(2 * j) + bias1) * c_qk;
            s[2] = (s[2] * unscale<BITS>(2 * j + 1) + bias0) * c_qk;
            s[3] = (s[3] * unscale<BITS>(2 * j + 1) + bias1) * c_qk;
        }
    }
    softmax_pv<BITS, NGRP>(sacc, sa, st, ls, lane, n_valid, slot, g_off);
}

// Online softmax (log2 domain) over the scores of one tile and out^T += V^T P with the values staged at `sa`.
// sacc[2e + j] holds, for key group G (= e, or g_off when NGRP == 1) of the tile, the scores of tokens
// 32G + 4g + 2j (elements 0, 1: heads 2t, 2t+1) and 32G + 4g + 2j + 1 (elements 2, 3).
template <int BITS, int NGRP>
__device__ __forceinline__ void softmax_pv(float (&sacc)[NGRP * 2][4], const char* sa, WarpState& st,
                                           const LaneSel<BITS>& ls, int lane, int n_valid, int slot, int g_off) {
    using C = Cfg<BITS>;
    const int g = lane >> 2, t = lane & 3;
    const unsigned sel_lo = 0x5410u, sel_hi = 0x7632u;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int e = 0; e < NGRP; ++e) {
        const int G = NGRP == 2 ? e : g_off;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            float* s = sacc[2 * e + j];
            if (n_valid < C::T) {  // last tile of a ragged segment: rows are tokens 32G + 4g + 2j (+1)
                const int tok = 32 * G + 4 * g + 2 * j;
                if (tok >= n_valid) s[0] = s[1] = -INFINITY;
                if (tok + 1 >= n_valid) s[2] = s[3] = -INFINITY;
            }
            if (slot) {  // a run of padded slots: only the first (slot >> 8) tokens of every (slot & 255) count
                const int in_slot = (32 * G + 4 * g + 2 * j) & ((slot & 255) - 1);
                if (in_slot >= (slot >> 8)) s[0] = s[1] = -INFINITY;
                if (in_slot + 1 >= (slot >> 8)) s[2] = s[3] = -INFINITY;
            }
            mx[0] = fmaxf(mx[0], fmaxf(s[0], s[2]));
            mx[1] = fmaxf(mx[1], fmaxf(s[1], s[3]));
        }
    }
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
    }
    const float m0 = fmaxf(st.m[0], mx[0]), m1 = fmaxf(st.m[1], mx[1]);
    const float al0 = ex2(st.m[0] - m0), al1 = ex2(st.m[1] - m1);  // first tile: ex2(-inf) = 0
    st.m[0] = m0;
    st.m[1] = m1;
    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
    for (int i = 0; i < NGRP * 2; ++i) {
        sacc[i][0] = ex2(sacc[i][0] - m0);
        sacc[i][1] = ex2(sacc[i][1] - m1);
        sacc[i][2] = ex2(sacc[i][2] - m0);
        sacc[i][3] = ex2(sacc[i][3] - m1);
        ls0 += sacc[i][0] + sacc[i][2];
        ls1 += sacc[i][1] + sacc[i][3];
    }
    st.l[0] = st.l[0] * al0 + ls0;
    st.l[1] = st.l[1] * al1 + ls1;
#pragma unroll
    for (int d = 0; d < 4; ++d)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            st.o[d][j][0] *= al0;
            st.o[d][j][1] *= al1;
            st.o[d][j][2] *= al0;
            st.o[d][j][3] *= al1;
        }
    st.pm[0] *= al0;
    st.pm[1] *= al1;
    st.pm[2] *= al0;
    st.pm[3] *= al1;

    // ---------------- out^T += V^T P: M = 16 dims, N = 8 heads, K = the 16 tokens of one score tile
    const unsigned vsel = (g & 1) ? sel_hi : sel_lo;
    const char* vc_lane = sa + 4 * (9 * t * C::VWPT + ls.word);  // row 9t: pad row per 8 tokens
    const char* vs_lane = sa + C::OFF_VS + 64 * t;
    const char* vm_lane = sa + C::OFF_VM + 64 * t + 4 * ((g >> 1) & 1);  // word holding zero[.][g], g < 4
#pragma unroll
    for (int e = 0; e < NGRP; ++e) {
        const int G = NGRP == 2 ? e : g_off;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float* p = sacc[2 * e + j];
            const unsigned pb0 = movmatrix_trans(pack_half2(p[0], p[1]));  // tokens of rows 2t, 2t+1; head g
            const unsigned pb1 = movmatrix_trans(pack_half2(p[2], p[3]));  // tokens of rows 2t+8, 2t+9
            // tokens of rows 2t, 2t+1, 2t+8, 2t+9 of this score tile: 32G + 8t + {2j, 2j+4, 2j+1, 2j+5}
            constexpr int kRow = C::VWPT * 4;
            const int r[4] = {2 * j, 2 * j + 4, 2 * j + 1, 2 * j + 5};
            uint2 vs[4];
            unsigned vmw[4];
            unsigned vw[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                vs[i] = ldp64(vs_lane + 8 * (32 * G + r[i]));
                vmw[i] = ldp32(vm_lane + 8 * (32 * G + r[i]));
#pragma unroll
                for (int d = 0; d < 4; ++d) vw[i][d] = ldp32(vc_lane + kRow * (36 * G + r[i]) + 4 * BITS * d);
            }
            {   // sum_n p[h,n] * zero[n,D]: rows = dim groups; only rows g < 4 are read back
                unsigned a0 = prmt(vmw[0], vmw[1], vsel);
                unsigned a2 = prmt(vmw[2], vmw[3], vsel);
                mma16816(st.pm, a0, 0u, a2, 0u, pb0, pb1);
            }
#pragma unroll
            for (int d = 0; d < 4; ++d) {
                const unsigned sel = (d & 1) ? sel_hi : sel_lo;
                const unsigned s01 = prmt((d & 2) ? vs[0].y : vs[0].x, (d & 2) ? vs[1].y : vs[1].x, sel);
                const unsigned s23 = prmt((d & 2) ? vs[2].y : vs[2].x, (d & 2) ? vs[3].y : vs[3].x, sel);
                const unsigned b0 = hmul2(pb0, s01), b1 = hmul2(pb1, s23);
                unsigned ra[4], rb[4];
                extract4<BITS>(vw[0][d], vw[1][d], ls, ra);
                extract4<BITS>(vw[2][d], vw[3][d], ls, rb);
                mma16816(st.o[d][0], ra[0], ra[1], rb[0], rb[1], b0, b1);
                mma16816(st.o[d][1], ra[2], ra[3], rb[2], rb[3], b0, b1);
                // same for p*scale: feed what float16 rounding dropped (matters when few tokens dominate)
                if (BITS != 2 || kPvResidual2) {
                    const unsigned b0l = hfma2_residual(pb0, s01, b0), b1l = hfma2_residual(pb1, s23, b1);
                    mma16816(st.o[d][0], ra[0], ra[1], rb[0], rb[1], b0l, b1l);
                    mma16816(st.o[d][1], ra[2], ra[3], rb[2], rb[3], b0l, b1l);
                }
            }
        }
    }
}

// Per-warp epilogue and cross-warp merge.  BITS > 0: packed tile accumulators (undo the power-of-two
// code scaling, add the zero terms).  BITS == 0: float16 tile accumulators (plain).
template <int BITS>
__device__ __forceinline__ void finish_cta(const CtaCtx& a, WarpState& st, int kvh, float* smem_f) {
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int h0 = kvh * a.G;
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        st.l[0] += __shfl_xor_sync(0xffffffffu, st.l[0], o);
        st.l[1] += __shfl_xor_sync(0xffffffffu, st.l[1], o);
    }
    __syncthreads();  // every ring is idle: reuse shared memory for the cross-warp merge
    float* o_s = smem_f + wid * (8 * HD + 16);  // [head 8][dim 128], then m[8], l[8]
    if (BITS > 0) {
        constexpr int B = BITS > 0 ? BITS : 2;
#pragma unroll
        for (int d = 0; d < 4; ++d) {
            const float z0 = __shfl_sync(0xffffffffu, st.pm[0], 4 * d + t);
            const float z1 = __shfl_sync(0xffffffffu, st.pm[1], 4 * d + t);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int dim = 32 * d + 4 * g + 2 * j;
                o_s[(2 * t) * HD + dim] = st.o[d][j][0] * unscale<B>(2 * j) + z0;
                o_s[(2 * t + 1) * HD + dim] = st.o[d][j][1] * unscale<B>(2 * j) + z1;
                o_s[(2 * t) * HD + dim + 1] = st.o[d][j][2] * unscale<B>(2 * j + 1) + z0;
                o_s[(2 * t + 1) * HD + dim + 1] = st.o[d][j][3] * unscale<B>(2 * j + 1) + z1;
            }
        }
    } else {
#pragma unroll
        for (int d = 0; d < 4; ++d)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int dim = 16 * (2 * d + j) + g;
                o_s[(2 * t) * HD + dim] = st.o[d][j][0];
                o_s[(2 * t + 1) * HD + dim] = st.o[d][j][1];
                o_s[(2 * t) * HD + dim + 8] = st.o[d][j][2];
                o_s[(2 * t + 1) * HD + dim + 8] = st.o[d][j][3];
            }
    }
    if (g == 0) {
        o_s[8 * HD + 2 * t] = st.m[0];
        o_s[8 * HD + 2 * t + 1] = st.m[1];
        o_s[8 * HD + 8 + 2 * t] = st.l[0];
        o_s[8 * HD + 8 + 2 * t + 1] = st.l[1];
    }
    __syncthreads();

    // ---------------- merge the warps' states into one partial per CTA
    // one thread per head: maximum, the warps' weights (kept in shared memory for the next step), denominator
    const size_t widx = a.widx;
    float* s_wgt = smem_f + NWARPS * (8 * HD + 16);  // [warp][8 heads]
    if (tid < a.G) {
        const int h = tid;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, smem_f[w * (8 * HD + 16) + 8 * HD + h]);
        float l = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float* ws = smem_f + w * (8 * HD + 16);
            const float wgt = ex2(ws[8 * HD + h] - M);
            s_wgt[8 * w + h] = wgt;
            l = fmaf(wgt, ws[8 * HD + 8 + h], l);
        }
        a.pm[widx * a.Hq + h0 + h] = M * (1.0f / kLog2e);  // back to the natural-log domain
        a.pl[widx * a.Hq + h0 + h] = l;
    }
    __syncthreads();
    // one thread per four dims of a head
    for (int idx = tid; idx < a.G * (HD / 4); idx += NTHREADS) {
        const int h = idx >> 5, d4 = idx & 31;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float wgt = s_wgt[8 * w + h];
            const float4 v = *reinterpret_cast<const float4*>(smem_f + w * (8 * HD + 16) + h * HD + 4 * d4);
            acc.x = fmaf(wgt, v.x, acc.x);
            acc.y = fmaf(wgt, v.y, acc.y);
            acc.z = fmaf(wgt, v.z, acc.z);
            acc.w = fmaf(wgt, v.w, acc.w);
        }
        *reinterpret_cast<float4*>(a.pacc + (widx * a.Hq + h0 + h) * HD + 4 * d4) = acc;
    }
}

__device__ __forceinline__ void init_state(WarpState& st) {
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
#pragma unroll
    for (int d = 0; d < 4; ++d)
#pragma unroll
        for (int j = 0; j < 2; ++j) st.o[d][j][0] = st.o[d][j][1] = st.o[d][j][2] = st.o[d][j][3] = 0.f;
    st.pm[0] = st.pm[1] = st.pm[2] = st.pm[3] = 0.f;
}

// ---------------------------------------------------------------- float16 (hot tier) tiles
// 32 tokens per tile, K and V rows padded to 272 bytes so that ldmatrix row addresses spread over
// all banks.  Tokens past the segment end are zero-filled by cp.async and masked to -inf.
constexpr int TH = 32;
constexpr int HROW = HD + 8;                      // halves per padded row
constexpr int HOT_TILE_BYTES = TH * HROW * 2;     // one of K or V
constexpr int HOT_RING_BYTES = 2 * HOT_TILE_BYTES;

__device__ __forceinline__ void issue_hot_tile(const SegDev& sg, long long S, int kvh, long long tile, unsigned sa,
                                               int lane) {
    const __half* kb = reinterpret_cast<const __half*>(sg.kp) + (size_t)kvh * sg.head_stride;
    const __half* vb = reinterpret_cast<const __half*>(sg.vp) + (size_t)kvh * sg.head_stride;
#pragma unroll 4
    for (int it = 0; it < TH * 16 / 32; ++it) {
        const int idx = it * 32 + lane, tok = idx >> 4, ch = idx & 15;
        const long long gt = tile * TH + tok;
        const unsigned nbytes = gt < S ? 16u : 0u;
        const size_t off = (size_t)min(gt, S - 1) * HD + ch * 8;
        cp_async16_zfill(sa + (tok * HROW + ch * 8) * 2, kb + off, nbytes);
        cp_async16_zfill(sa + HOT_TILE_BYTES + (tok * HROW + ch * 8) * 2, vb + off, nbytes);
    }
    cp_async_commit();
}

__device__ __forceinline__ void compute_hot_tile(unsigned sa, const unsigned (&qh)[8][2], float c_qk, WarpState& st,
                                                 int valid, int lane) {
    const int g = lane >> 2;
    const int mi = lane >> 3, mr = lane & 7;  // ldmatrix: this lane addresses row mr of matrix mi
    float sacc[2][4];
#pragma unroll
    for (int m = 0; m < 2; ++m) sacc[m][0] = sacc[m][1] = sacc[m][2] = sacc[m][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
#pragma unroll
        for (int m = 0; m < 2; ++m) {
            unsigned a0, a1, a2, a3;
            ldmatrix_x4(sa + ((16 * m + (mi & 1) * 8 + mr) * HROW + 16 * kk + (mi >> 1) * 8) * 2, a0, a1, a2, a3);
            mma16816(sacc[m], a0, a1, a2, a3, qh[kk][0], qh[kk][1]);
        }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        const bool v0 = 16 * m + g < valid, v1 = 16 * m + g + 8 < valid;
        sacc[m][0] = v0 ? sacc[m][0] * c_qk : -INFINITY;
        sacc[m][1] = v0 ? sacc[m][1] * c_qk : -INFINITY;
        sacc[m][2] = v1 ? sacc[m][2] * c_qk : -INFINITY;
        sacc[m][3] = v1 ? sacc[m][3] * c_qk : -INFINITY;
        mx[0] = fmaxf(mx[0], fmaxf(sacc[m][0], sacc[m][2]));
        mx[1] = fmaxf(mx[1], fmaxf(sacc[m][1], sacc[m][3]));
    }
#pragma unroll
    for (int o = 4; o <= 16; o <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
    }
    const float m0 = fmaxf(st.m[0], mx[0]), m1 = fmaxf(st.m[1], mx[1]);
    const float al0 = ex2(st.m[0] - m0), al1 = ex2(st.m[1] - m1);
    st.m[0] = m0;
    st.m[1] = m1;
    float ls0 = 0.f, ls1 = 0.f;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        sacc[m][0] = ex2(sacc[m][0] - m0);
        sacc[m][1] = ex2(sacc[m][1] - m1);
        sacc[m][2] = ex2(sacc[m][2] - m0);
        sacc[m][3] = ex2(sacc[m][3] - m1);
        ls0 += sacc[m][0] + sacc[m][2];
        ls1 += sacc[m][1] + sacc[m][3];
    }
    st.l[0] = st.l[0] * al0 + ls0;
    st.l[1] = st.l[1] * al1 + ls1;
#pragma unroll
    for (int d = 0; d < 4; ++d)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            st.o[d][j][0] *= al0;
            st.o[d][j][1] *= al1;
            st.o[d][j][2] *= al0;
            st.o[d][j][3] *= al1;
        }
    const unsigned va = sa + HOT_TILE_BYTES;
#pragma unroll
    for (int m = 0; m < 2; ++m) {
        const unsigned pb0 = movmatrix_trans(pack_half2(sacc[m][0], sacc[m][1]));
        const unsigned pb1 = movmatrix_trans(pack_half2(sacc[m][2], sacc[m][3]));
#pragma unroll
        for (int dt = 0; dt < 8; ++dt) {
            unsigned a0, a1, a2, a3;
            ldmatrix_x4_trans(va + ((16 * m + (mi >> 1) * 8 + mr) * HROW + 16 * dt + (mi & 1) * 8) * 2, a0, a1, a2, a3);
            mma16816(st.o[dt >> 1][dt & 1], a0, a1, a2, a3, pb0, pb1);
        }
    }
}

// S: the tokens that count (the segment's length, or what its device-resident length says)
__device__ __forceinline__ void run_cta_fp16(const CtaCtx& a, const SegDev& sg, long long S, long long tile0,
                                             long long tile1, int kvh, float* smem_f) {
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_f);
    const int h0 = kvh * a.G;
    cudaGridDependencySynchronize();  // the hot tier and q may have been written by the previous kernel
    cudaTriggerProgrammaticLaunchCompletion();
    WarpState st;
    init_state(st);
    // q as the B operand in natural channel order: k = 2t, 2t+1 | 2t+8, 2t+9 of each 16-channel step
    unsigned qh[8][2];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        qh[kk][0] = qh[kk][1] = 0u;
        if (g < a.G) {
            const __half* qp = a.q + (size_t)(h0 + g) * HD + 16 * kk + 2 * t;
            qh[kk][0] = *reinterpret_cast<const unsigned*>(qp);
            qh[kk][1] = *reinterpret_cast<const unsigned*>(qp + 8);
        }
    }
    const float c_qk = a.sm_scale * kLog2e;
    constexpr int kHotWarps = kSmemBytes / HOT_RING_BYTES < NWARPS ? kSmemBytes / HOT_RING_BYTES : NWARPS;
    const unsigned ring = smem_base + wid * HOT_RING_BYTES;
    for (long long tile = tile0 + wid; wid < kHotWarps && tile < tile1; tile += kHotWarps) {
        issue_hot_tile(sg, S, kvh, tile, ring, lane);
        cp_async_wait<0>();
        __syncwarp();
        compute_hot_tile(ring, qh, c_qk, st, (int)min((long long)TH, S - tile * TH), lane);
        __syncwarp();
    }
    finish_cta<0>(a, st, kvh, smem_f);
}

// A CTA walks its token range in super-tiles of up to NSUB tiles: the keys of a super-tile are fetched for the
// whole CTA into one of two buffers (tiled TMA copies issued by one thread where the host could describe the
// segment and the range is long enough to pay for the barrier set-up, 16-byte cp.async by every thread otherwise,
// ordinary loads for ragged rows), each warp streams the values of its own tile, one __syncthreads per super-tile.
template <int BITS>
__device__ __forceinline__ void run_cta(const CtaCtx& a, const SegDev& sg, long long S, const KeyMaps* kmaps,
                                        long long tile0, long long tile1, int kvh, float* smem_f) {
    using C = Cfg<BITS>;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_f);
    const int h0 = kvh * a.G;
    // tokens of tile `tl` that exist (the last tile of a ragged segment is partial)
    auto valid_of = [&](long long tl) { return (int)min((long long)C::T, S - tl * C::T); };

    const KSrc<BITS> ksrc(sg, kvh, tile0);

    WarpState st;
    init_state(st);

    // smem: [mbarriers][q][K buffer 0][K buffer 1][value stages of warp 0][of warp 1]...
    const char* smem_c = reinterpret_cast<const char*>(smem_f);
    const unsigned kbuf = smem_base + kHeadBytes;
    // value ring of tile `vt` of a super-tile (the ring of the warp, or of the warp pair, that computes it)
    auto ring_of = [&](int vt) { return kbuf + 2 * C::KBUF_BYTES + vt * (NSTAGE * C::VSTAGE_BYTES); };
    const VSrc<BITS> vsrc(sg, kvh, lane);
    const int n_tiles_cta = (int)(tile1 - tile0);
    const int n_super = (n_tiles_cta + C::NSUB - 1) / C::NSUB;
    // The partial super-tile goes FIRST: nothing can be computed until the first super-tile has landed, and every
    // SM asks for its first one at the same moment, so a short first fetch shortens the exposed start, while the
    // full ones behind it are fetched under compute.  (Only when the partial one is a multiple of four tiles, so
    // that the later super-tiles keep their key scale rows 16-byte aligned.)
    const int rem_tiles = n_tiles_cta - (n_super - 1) * C::NSUB;  // 1 .. NSUB
    const bool small_first = kSmallFirst && n_super > 1 && rem_tiles < C::NSUB && (rem_tiles & 3) == 0;
    auto sp_count = [&](int sp) {
        return small_first ? (sp == 0 ? rem_tiles : C::NSUB) : min(C::NSUB, n_tiles_cta - sp * C::NSUB);
    };
    auto sp_first = [&](int sp) {
        return small_first ? (sp == 0 ? tile0 : tile0 + rem_tiles + (long long)(sp - 1) * C::NSUB)
                           : tile0 + (long long)sp * C::NSUB;
    };
    // A super-tile with at most NSUB / 2 tiles (the tail of a CTA's range, or all of a short one) is computed by
    // warp pairs: warp w takes key group (w & 1) of tile (w >> 1), and the pair shares the value stage of its
    // even warp, which alone fetches it.  v_tile_of: the tile whose values this warp fetches, or -1.
    auto split_of = [&](int n) { return kPairSplit && 2 * n <= C::NSUB; };
    auto v_tile_of = [&](int n) {
        if (split_of(n)) return ((wid & 1) == 0 && wid < 2 * n) ? (wid >> 1) : -1;
        return wid < n ? wid : -1;
    };
    // Keys come through tiled TMA copies when the host could describe the segment with tensor maps (rows and scale
    // rows a multiple of 16 bytes apart), this CTA's super-tiles start on multiples of four tiles and there are
    // enough of them to pay for the barrier set-up; otherwise every thread issues 16-byte cp.async copies into
    // the same shared-memory image.
    const bool ktma = kKeyTma && kmaps != nullptr && ksrc.aligned && (tile0 & 3) == 0 && n_super >= kTmaMinSuper;
    const unsigned kbar = smem_base;  // [2] mbarriers, one per key buffer
    bool timed_out = false;
    if (ktma && tid == 0) {  // the same thread issues the first copies; everyone else meets the barriers after
        mbar_init(kbar, 1);  // the __syncthreads() below
        mbar_init(kbar + 8, 1);
        fence_mbar_init();
    }
    auto issue_keys = [&](long long tile, int n, int buf) {
        if (ktma) {
            if (tid == 0) ksrc.issue_tma(kmaps, kvh, tile, n, kbuf + buf * C::KBUF_BYTES, kbar + 8 * buf);
        } else {
            ksrc.issue(tile, n, kbuf + buf * C::KBUF_BYTES, tid);
        }
    };
    auto issue_first = [&]() {
        const int n_sub = sp_count(0);
        issue_keys(tile0, n_sub, 0);
        const int vt = v_tile_of(n_sub);
        if (vt >= 0) vsrc.issue(tile0 + vt, ring_of(vt), valid_of(tile0 + vt));
        cp_async_commit();
    };

    // Super-tile 0 of a settled packed segment is fetched before the dependency wait.  A segment that the kernel
    // launched just before this one may have written (flagged by the caller) is read only after it.
    const bool early = !sg.fresh && sg.len_dev == nullptr;
    if (!early) cudaGridDependencySynchronize();
    if (ksrc.aligned) issue_first();
    if (ktma) __syncthreads();  // the mbarriers are initialised for every thread that will wait on them
    if (early) cudaGridDependencySynchronize();  // everything below may depend on the previous kernel of the stream
    // q of the GQA group, staged once per CTA behind the first copies (rows padded against bank
    // conflicts; zero rows for heads >= G)
    if (tid < 128) {
        const int head = tid >> 4, ch = tid & 15;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (head < a.G) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(h0 + head) * HD + 8 * ch);
        *reinterpret_cast<uint4*>(reinterpret_cast<char*>(smem_f) + kBarBytes + head * kQRowBytes + 16 * ch) = v;
    } else if (tid < 256) {
        // per channel the largest |q| over the group's heads, twice (one per key group of a scale word)
        const int d = tid - 128;
        unsigned short mx = 0;
        for (int h = 0; h < a.G; ++h) {
            const unsigned short v = *reinterpret_cast<const unsigned short*>(a.q + (size_t)(h0 + h) * HD + d) & 0x7fffu;
            mx = v > mx ? v : mx;  // the order of non-negative float16 numbers is the order of their bits
        }
        *reinterpret_cast<unsigned*>(reinterpret_cast<char*>(smem_f) + kOffQAbs + 4 * d) = mx * 0x10001u;
    }
    // let a programmatic dependent (the next launch of the stream) be scheduled as soon as SMs free up; it still
    // waits for this grid to complete before it reads anything this grid writes
    cudaTriggerProgrammaticLaunchCompletion();
    const LaneSel<BITS> ls(g);
    const float c_qk = a.sm_scale * kLog2e;
    const int slot = sg.slot_tokens ? (sg.slot_valid << 8) | sg.slot_tokens : 0;
    for (int sp = 0; sp < n_super; ++sp) {
        const int n_sub = sp_count(sp);
        const long long first = sp_first(sp);
        int buf = sp & 1;
        if (ksrc.aligned) {
            cp_async_wait<0>();
            // bounded: a copy that never completes poisons this CTA's partial instead of hanging the GPU
            if (ktma && !mbar_wait(kbar + 8 * buf, (sp >> 1) & 1)) timed_out = true;
            __syncthreads();  // super-tile sp has landed for everyone; everyone is done with sp - 1
            if (sp + 1 < n_super) {
                const long long next = sp_first(sp + 1);
                const int n_next = sp_count(sp + 1);
                const int nb = (sp + 1) & 1;
                if (ktma && tid == 0) fence_proxy_async();  // the buffer was last read through the generic proxy
                issue_keys(next, n_next, nb);
                const int vt = v_tile_of(n_next);
                if (vt >= 0) vsrc.issue(next + vt, ring_of(vt) + nb * C::VSTAGE_BYTES, valid_of(next + vt));
                cp_async_commit();
            }
        } else {
            // ragged segment: keys through ordinary loads into buffer 0, no overlap with the compute
            buf = 0;
            __syncthreads();  // everyone is done with the previous super-tile
            const int vt = v_tile_of(n_sub);
            if (vt >= 0) vsrc.issue(first + vt, ring_of(vt), valid_of(first + vt));
            cp_async_commit();
            ksrc.load_sync(first, n_sub, reinterpret_cast<char*>(smem_f) + kHeadBytes, tid);
            cp_async_wait<0>();
            __syncthreads();
        }
        const char* kb_c = smem_c + kHeadBytes + buf * C::KBUF_BYTES;
        const char* v0_c = smem_c + kHeadBytes + 2 * C::KBUF_BYTES + buf * C::VSTAGE_BYTES;  // stage `buf` of warp 0's ring
        const char* q_c = smem_c + kBarBytes + g * kQRowBytes + 4 * t;
        const char* qabs_c = smem_c + kOffQAbs;
        if (split_of(n_sub)) {
            const int sub = wid >> 1, half = wid & 1;
            if (wid < 2 * n_sub) {
                const int nv = valid_of(first + sub);
                if (32 * half < nv)  // a group without a single token contributes nothing
                    compute_tile<BITS, 1>(kb_c, sub, v0_c + sub * (NSTAGE * C::VSTAGE_BYTES), q_c, c_qk, st, ls, lane,
                                          nv, qabs_c, slot, half);
            }
        } else if (wid < n_sub) {
            compute_tile<BITS>(kb_c, wid, v0_c + wid * (NSTAGE * C::VSTAGE_BYTES), q_c, c_qk, st, ls, lane,
                               valid_of(first + wid), qabs_c, slot);
        }
    }
    if (ktma) {
        __syncthreads();  // nobody waits on the barriers any more: release their memory
        if (tid == 0) {
            mbar_inval(kbar);
            mbar_inval(kbar + 8);
        }
        // a wait that gave up means the result of this CTA cannot be trusted: poison it rather than hang
        if (timed_out) st.m[0] = st.m[1] = __int_as_float(0x7fc00000);
    }
    finish_cta<BITS>(a, st, kvh, smem_f);
}

// ---------------------------------------------------------------- per-token layout (keys packed along head_dim)
// Keys of this layout look exactly like values: per token a row of hd * BITS / 8 code bytes and four (scale, zero)
// pairs, one per group of 32 channels.  The score contraction runs over channels, which now lie NEXT to each other
// in a word, so an A operand (rows = tokens) pairs two fields of ONE word: field f of the low half with field f of
// the high half, isolated by a single AND (after a byte shift for fields in the upper byte of a half).  The MMA does
// not care which channel sits at which k index as long as q is permuted the same way, and the power of two a field
// position implies is folded into q.  Scale and zero belong to the ROW (token) here, so they cannot ride on the B
// operand: every group of 32 channels (two k-steps) gets a fresh accumulator and
//   score(n, h) = sum_G  scale[n, G] * 2^24 * acc_G(n, h)  +  zero[n, G] * sum_{d in G} q[h, d].
// The B operands (q, permuted and scaled) are the same for every tile and stay in registers.
//
// Channels (relative to 16 * kk) at the lane's k indices (2t, 2t+1 | 2t+8, 2t+9) and the factor q carries:
//   2 bits: (t, t+8 | t+4, t+12) * 4^-t      4 bits: (t, t+4 | t+8, t+12) * 16^-(t&1)      8 bits: (4t, 4t+2 | 4t+1, 4t+3)
template <int BITS>
__device__ __forceinline__ void per_token_q(const char* q_s /* [8][kQRowBytes] */, int lane, unsigned (&qb)[8][2]) {
    const int g = lane >> 2, t = lane & 3;
    const __half* row = reinterpret_cast<const __half*>(q_s + g * kQRowBytes);
    const float f = BITS == 2 ? 1.0f / (float)(1 << (2 * t)) : BITS == 4 ? ((t & 1) ? 0.0625f : 1.0f) : 1.0f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
        int c0, c1, c2, c3;
        if (BITS == 2) c0 = t, c1 = t + 8, c2 = t + 4, c3 = t + 12;
        else if (BITS == 4) c0 = t, c1 = t + 4, c2 = t + 8, c3 = t + 12;
        else c0 = 4 * t, c1 = 4 * t + 2, c2 = 4 * t + 1, c3 = 4 * t + 3;
        const __half* r = row + 16 * kk;
        // exact unless the scaled value is a float16 subnormal (|q| < 0.004): then it is off by at most 2^-25
        qb[kk][0] = pack_half2(__half2float(r[c0]) * f, __half2float(r[c1]) * f);
        qb[kk][1] = pack_half2(__half2float(r[c2]) * f, __half2float(r[c3]) * f);
    }
}

// NGRP = 2: the whole 64-token tile; NGRP = 1: only its 32-token half `g_off`.
template <int BITS, int NGRP>
__device__ __forceinline__ void per_token_scores(const char* ka, const unsigned (&qb)[8][2], const float (&qs)[2][4],
                                                 float c24, int lane, float (&sacc)[NGRP * 2][4], int g_off) {
    using C = Cfg<BITS>;
    constexpr int kRow = C::VWPT * 4;
    const int g = lane >> 2, t = lane & 3;
    const unsigned mask = BITS == 2 ? 0x00030003u << (2 * t) : BITS == 4 ? 0x000F000Fu << (4 * (t & 1)) : 0x00FF00FFu;
    const int sh = BITS == 4 ? 8 * (t >> 1) : 0;
#pragma unroll
    for (int ii = 0; ii < NGRP * 2; ++ii) {  // i = 2G + j: tokens 32G + 4g + 2j and the one after
        const int i = NGRP == 2 ? ii : 2 * g_off + ii;
        const int tok = 32 * (i >> 1) + 4 * g + 2 * (i & 1);
        const char* ra = ka + (tok + tok / 8) * kRow;  // one pad row per 8 tokens; tok is even, so tok + 1 is in the same block
        const char* rb = ra + kRow;
        const uint2 sa2 = ldp64(ka + C::OFF_VS + 8 * tok), sb2 = ldp64(ka + C::OFF_VS + 8 * tok + 8);
        const uint2 za2 = ldp64(ka + C::OFF_VM + 8 * tok), zb2 = ldp64(ka + C::OFF_VM + 8 * tok + 8);
        float out[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int G = 0; G < 4; ++G) {
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int kk = 2 * G + hh;
                unsigned a0, a1, a2, a3;
                if (BITS == 2) {
                    const unsigned x = ldp32(ra + 4 * kk), y = ldp32(rb + 4 * kk);
                    a0 = x & mask, a2 = (x >> 8) & mask, a1 = y & mask, a3 = (y >> 8) & mask;
                } else if (BITS == 4) {
                    const uint2 x = ldp64(ra + 8 * kk), y = ldp64(rb + 8 * kk);
                    a0 = (x.x >> sh) & mask, a2 = (x.y >> sh) & mask, a1 = (y.x >> sh) & mask, a3 = (y.y >> sh) & mask;
                } else {
                    const unsigned x = ldp32(ra + 16 * kk + 4 * t), y = ldp32(rb + 16 * kk + 4 * t);
                    a0 = x & mask, a2 = (x >> 8) & mask, a1 = y & mask, a3 = (y >> 8) & mask;
                }
                mma16816(acc, a0, a1, a2, a3, qb[kk][0], qb[kk][1]);
            }
            const unsigned sw_a = (G & 2) ? sa2.y : sa2.x, sw_b = (G & 2) ? sb2.y : sb2.x;
            const unsigned zw_a = (G & 2) ? za2.y : za2.x, zw_b = (G & 2) ? zb2.y : zb2.x;
            const __half2 sh_a = *reinterpret_cast<const __half2*>(&sw_a), sh_b = *reinterpret_cast<const __half2*>(&sw_b);
            const __half2 zh_a = *reinterpret_cast<const __half2*>(&zw_a), zh_b = *reinterpret_cast<const __half2*>(&zw_b);
            const float ks_a = ((G & 1) ? __high2float(sh_a) : __low2float(sh_a)) * c24;
            const float ks_b = ((G & 1) ? __high2float(sh_b) : __low2float(sh_b)) * c24;
            const float kz_a = (G & 1) ? __high2float(zh_a) : __low2float(zh_a);
            const float kz_b = (G & 1) ? __high2float(zh_b) : __low2float(zh_b);
            out[0] = fmaf(ks_a, acc[0], fmaf(kz_a, qs[0][G], out[0]));
            out[1] = fmaf(ks_a, acc[1], fmaf(kz_a, qs[1][G], out[1]));
            out[2] = fmaf(ks_b, acc[2], fmaf(kz_b, qs[0][G], out[2]));
            out[3] = fmaf(ks_b, acc[3], fmaf(kz_b, qs[1][G], out[3]));
        }
        sacc[ii][0] = out[0], sacc[ii][1] = out[1], sacc[ii][2] = out[2], sacc[ii][3] = out[3];
    }
}

// Warps that can hold a two-stage ring of (key stage, value stage) each
template <int BITS>
struct PerTokenWarps {
    static constexpr int kFit = (kSmemBytes - kHeadBytes) / (2 * NSTAGE * Cfg<BITS>::VSTAGE_BYTES);
    static constexpr int value = kFit < NWARPS ? kFit : NWARPS;
};

// Every warp streams its own tiles (keys and values of 64 tokens each) through a private two-stage ring: no CTA
// barrier inside the loop.
template <int BITS>
__device__ __forceinline__ void run_cta_per_token(const CtaCtx& a, const SegDev& sg, long long tile0, long long tile1,
                                                  int kvh, float* smem_f) {
    using C = Cfg<BITS>;
    constexpr int W = PerTokenWarps<BITS>::value;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const unsigned smem_base = (unsigned)__cvta_generic_to_shared(smem_f);
    const char* smem_c = reinterpret_cast<const char*>(smem_f);
    const int h0 = kvh * a.G;
    auto valid_of = [&](long long tl) { return (int)min((long long)C::T, sg.S - tl * C::T); };
    const VSrc<BITS> ksrc(sg.kp, sg.ks, sg.km, sg.S, kvh, lane), vsrc(sg.vp, sg.vs, sg.vm, sg.S, kvh, lane);
    constexpr int kStage = 2 * C::VSTAGE_BYTES;  // keys, then values
    const int ring = kHeadBytes + wid * (NSTAGE * kStage);
    auto issue = [&](long long tile, int stage) {
        const int nv = valid_of(tile);
        ksrc.issue(tile, smem_base + ring + stage * kStage, nv);
        vsrc.issue(tile, smem_base + ring + stage * kStage + C::VSTAGE_BYTES, nv);
    };
    WarpState st;
    init_state(st);
    // Warp w takes tiles w, w + W, ...  When the last round has at most W / 2 tiles it is dealt out in 32-token halves
    // (warp w: half w & 1 of tile w >> 1 of that round; each warp stages the tile for itself), so that the tail of a
    // CTA's range costs half a tile time instead of a whole one.
    const int n_tiles = (int)(tile1 - tile0);
    const int full_rounds = n_tiles / W, rem = n_tiles - full_rounds * W;
    const bool halves = rem > 0 && 2 * rem <= W;
    const int my_full = wid < W ? full_rounds + ((!halves && wid < rem) ? 1 : 0) : 0;  // whole tiles of this warp
    const bool my_half = halves && wid < 2 * rem;
    auto tile_of = [&](int it) {  // the it-th tile this warp stages (whole tiles first, then its half tile)
        return it < my_full ? tile0 + wid + (long long)it * W : tile0 + (long long)full_rounds * W + (wid >> 1);
    };
    const int my_count = my_full + (my_half ? 1 : 0);
    const bool mine = my_count > 0;
    const bool early = !sg.fresh;
    if (!early) cudaGridDependencySynchronize();
    if (mine) issue(tile_of(0), 0);
    cp_async_commit();
    if (early) cudaGridDependencySynchronize();
    // q of the GQA group (zero rows for heads >= G), and per head and channel group the sum of q
    if (tid < 128) {
        const int head = tid >> 4, ch = tid & 15;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (head < a.G) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(h0 + head) * HD + 8 * ch);
        *reinterpret_cast<uint4*>(reinterpret_cast<char*>(smem_f) + kBarBytes + head * kQRowBytes + 16 * ch) = v;
    } else if (tid < 160) {
        const int head = (tid - 128) >> 2, grp = (tid - 128) & 3;
        float sum = 0.f;
        if (head < a.G)
            for (int d = 0; d < 32; ++d) sum += __half2float(a.q[(size_t)(h0 + head) * HD + 32 * grp + d]);
        reinterpret_cast<float*>(reinterpret_cast<char*>(smem_f) + kOffQAbs)[4 * head + grp] = sum;
    }
    cudaTriggerProgrammaticLaunchCompletion();
    __syncthreads();
    const float c_qk = a.sm_scale * kLog2e;
    unsigned qb[8][2];
    per_token_q<BITS>(smem_c + kBarBytes, lane, qb);
    float qs[2][4];
#pragma unroll
    for (int G = 0; G < 4; ++G) {
        qs[0][G] = reinterpret_cast<const float*>(smem_c + kOffQAbs)[4 * (2 * t) + G] * c_qk;
        qs[1][G] = reinterpret_cast<const float*>(smem_c + kOffQAbs)[4 * (2 * t + 1) + G] * c_qk;
    }
    const LaneSel<BITS> ls(g);
    for (int it = 0; it < my_count; ++it) {
        const long long tile = tile_of(it);
        if (it + 1 < my_count) issue(tile_of(it + 1), (it + 1) & 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncwarp();
        const char* stage = smem_c + ring + (it & 1) * kStage;
        const int nv = valid_of(tile);
        if (it < my_full) {
            float sacc[4][4];
            per_token_scores<BITS, 2>(stage, qb, qs, c_qk * 16777216.f, lane, sacc, 0);
            softmax_pv<BITS, 2>(sacc, stage + C::VSTAGE_BYTES, st, ls, lane, nv, 0, 0);
        } else if (32 * (wid & 1) < nv) {  // (a half without a single token contributes nothing)
            float sacc[2][4];
            per_token_scores<BITS, 1>(stage, qb, qs, c_qk * 16777216.f, lane, sacc, wid & 1);
            softmax_pv<BITS, 1>(sacc, stage + C::VSTAGE_BYTES, st, ls, lane, nv, 0, wid & 1);
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    finish_cta<BITS>(a, st, kvh, smem_f);
}

__device__ __forceinline__ long long tiles_in(const SegDev& sg, long long S) {
    return sg.kind == PKV_SEG_FP16 ? (S + TH - 1) / TH : (S + 63) / 64;
}

// The tokens of a segment that count: its length, or, for a segment whose length lives in device memory, what that
// says now (never more than the capacity the launch was sized for).  The value may have been written by the
// previous kernel of the stream, so it is read behind the dependency wait.
__device__ __forceinline__ long long live_length(const SegDev& sg) {
    if (sg.len_dev == nullptr) return sg.S;
    cudaGridDependencySynchronize();
    return min(sg.S, max(0LL, (long long)*sg.len_dev));
}

// A work item past the end of a segment whose length shrank below the launch's capacity: nothing to attend to.
__device__ __forceinline__ void write_empty_partial(const CtaCtx& a, int kvh) {
    cudaGridDependencySynchronize();
    cudaTriggerProgrammaticLaunchCompletion();
    const int h0 = kvh * a.G;
    for (int idx = threadIdx.x; idx < a.G * (HD / 4); idx += NTHREADS)
        *reinterpret_cast<float4*>(a.pacc + (a.widx * a.Hq + h0) * HD + 4 * idx) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (threadIdx.x < a.G) {
        a.pm[a.widx * a.Hq + h0 + threadIdx.x] = -INFINITY;
        a.pl[a.widx * a.Hq + h0 + threadIdx.x] = 0.f;
    }
}

// Tiles [tile0, tile0 + n_tiles) of segment `sg` for KV head `kvh`, one partial written to row a.widx.
__device__ __forceinline__ void run_item(const CtaCtx& a, const SegDev& sg, const KeyMaps* kmaps, long long tile0,
                                         long long n_tiles, int kvh, float* smem_f) {
    const long long S = live_length(sg);
    const long long tile1 = min(tiles_in(sg, S), tile0 + n_tiles);
    if (tile0 >= tile1) return write_empty_partial(a, kvh);
    if (sg.kind == PKV_SEG_FP16) run_cta_fp16(a, sg, S, tile0, tile1, kvh, smem_f);
    else if (sg.kbits == 2) run_cta<2>(a, sg, S, kmaps, tile0, tile1, kvh, smem_f);
    else if (sg.kbits == 4) run_cta<4>(a, sg, S, kmaps, tile0, tile1, kvh, smem_f);
    else run_cta<8>(a, sg, S, kmaps, tile0, tile1, kvh, smem_f);
}

// Which work item a CTA of the single-sequence kernels has
__device__ __forceinline__ void item_of(const MmaArgs& a, int& si, int& split) {
    const int w = blockIdx.x;
    si = 0;
    while (si + 1 < a.n_segs && w >= a.segs[si + 1].work_begin) ++si;
    split = w - a.segs[si].work_begin;
}

// One sequence, segment descriptors inside the parameter block; work item w of a segment covers
// split_len tiles.
__global__ void __launch_bounds__(NTHREADS, CTAS_PER_SM) decode_mma_kernel(const __grid_constant__ MmaArgs a) {
    extern __shared__ __align__(1024) float smem_f[];
    int si, split;
    item_of(a, si, split);
    const SegDev& sg = a.segs[si];
    const int kvh = blockIdx.y;
    const CtaCtx ctx = {a.q, a.pm, a.pl, a.pacc, (size_t)a.work_offset + blockIdx.x, a.Hq, a.G, a.sm_scale};
    run_item(ctx, sg, sg.key_tma ? &a.kmaps[sg.key_tma - 1] : nullptr, (long long)split * sg.split_len, sg.split_len, kvh, smem_f);
}

// The same for launches whose packed segments are in the per-token layout (float16 segments ride along).  A
// kernel of its own: the KIVI kernel is sensitive to its code size and register count.
__global__ void __launch_bounds__(NTHREADS, CTAS_PER_SM) decode_mma_per_token_kernel(const __grid_constant__ MmaArgs a) {
    extern __shared__ __align__(1024) float smem_f[];
    int si, split;
    item_of(a, si, split);
    const SegDev& sg = a.segs[si];
    const int kvh = blockIdx.y;
    const CtaCtx ctx = {a.q, a.pm, a.pl, a.pacc, (size_t)a.work_offset + blockIdx.x, a.Hq, a.G, a.sm_scale};
    const long long S = live_length(sg);
    const long long tile0 = (long long)split * sg.split_len, tile1 = min(tiles_in(sg, S), tile0 + sg.split_len);
    if (tile0 >= tile1) return write_empty_partial(ctx, kvh);
    if (sg.kind == PKV_SEG_FP16) run_cta_fp16(ctx, sg, S, tile0, tile1, kvh, smem_f);
    else if (sg.kbits == 2) run_cta_per_token<2>(ctx, sg, tile0, tile1, kvh, smem_f);
    else if (sg.kbits == 4) run_cta_per_token<4>(ctx, sg, tile0, tile1, kvh, smem_f);
    else run_cta_per_token<8>(ctx, sg, tile0, tile1, kvh, smem_f);
}

// Many sequences, descriptors and an explicit work list in device memory (see BatchTable).
__global__ void __launch_bounds__(NTHREADS, CTAS_PER_SM) decode_mma_batched_kernel(const __grid_constant__ BatchArgs a) {
    extern __shared__ __align__(1024) float smem_f[];
    const BatchWork wk = a.work[blockIdx.x];
    const SegDev& sg = a.segs[wk.seg];
    const CtaCtx ctx = {a.q + (size_t)wk.seq * a.Hq * HD, a.pm, a.pl, a.pacc, (size_t)wk.part, a.Hq, a.G, a.sm_scale};
    run_item(ctx, sg, nullptr, wk.tile_begin, wk.n_tiles, blockIdx.y, smem_f);
}

}  // namespace

bool eligible(const pkv_segment_t& s, int Hq, int Hkv, int hd) {
    if (hd != HD || Hq / Hkv > 8) return false;
    if (s.kind == PKV_SEG_FP16) {
        const uintptr_t bits = reinterpret_cast<uintptr_t>(s.k_packed) | reinterpret_cast<uintptr_t>(s.v_packed);
        return (bits & 15u) == 0 && s.head_stride % 8 == 0;
    }
    if (s.kind != PKV_SEG_KIVI && s.kind != PKV_SEG_PER_TOKEN) return false;
    // a segment shorter than one group has its key group clamped to its length: still one group per 32 tokens
    const bool k_group_ok = s.k_group == 32 || (s.kind == PKV_SEG_KIVI && s.seq_len < 32 && s.k_group == s.seq_len);
    if (s.k_bits != s.v_bits || !k_group_ok || s.v_group != 32) return false;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(s.k_packed) | reinterpret_cast<uintptr_t>(s.k_scale) |
                           reinterpret_cast<uintptr_t>(s.k_mins) | reinterpret_cast<uintptr_t>(s.v_packed) |
                           reinterpret_cast<uintptr_t>(s.v_scale) | reinterpret_cast<uintptr_t>(s.v_mins);
    return (bits & 15u) == 0;
}

// Tiles of a segment as the tensor-core kernel counts them.
long long tiles_of(const pkv_segment_t& s) {
    if (s.kind == PKV_SEG_FP16) return (s.seq_len + TH - 1) / TH;
    return (s.seq_len + tile_tokens(s.k_bits) - 1) / tile_tokens(s.k_bits);
}

namespace {
template <class Kernel, class Args>
int launch_pdl(Kernel kernel, const Args& a, int work, int Hkv, cudaStream_t stream, bool* configured) {
    int dev = 0;
    PKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return PKV_E_LIMIT;
    if (!configured[dev]) {
        PKV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        configured[dev] = true;
    }
    // Programmatic dependent launch: the grid may become resident while the previous kernel of the stream
    // drains.  Until cudaGridDependencySynchronize() it only touches the frozen packed segments, which no
    // earlier kernel of a decode step writes; q, the hot tier and the scratch are touched after it.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)work, (unsigned)Hkv);
    cfg.blockDim = dim3(NTHREADS);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    PKV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, a));
    return PKV_OK;
}
}  // namespace

int launch(const MmaArgs& a, int work, int Hkv, cudaStream_t stream) {
    static thread_local bool configured[64] = {};
    return launch_pdl(decode_mma_kernel, a, work, Hkv, stream, configured);
}

int launch_per_token(const MmaArgs& a, int work, int Hkv, cudaStream_t stream) {
    static thread_local bool configured[64] = {};
    return launch_pdl(decode_mma_per_token_kernel, a, work, Hkv, stream, configured);
}

int launch_batched(const BatchArgs& a, int work, int Hkv, cudaStream_t stream) {
    static thread_local bool configured[64] = {};
    return launch_pdl(decode_mma_batched_kernel, a, work, Hkv, stream, configured);
}

}  // namespace mma
}  // namespace pkv

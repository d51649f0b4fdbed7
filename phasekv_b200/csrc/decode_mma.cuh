// Tensor-core split-K decode over packed segments (head_dim 128, group 32, GQA group <= 8): KIVI layout, and the
// per-token layout in a kernel of its own (see run_cta_per_token).
//
// Idea.  The packed codes are never converted to numbers by arithmetic.  A b-bit code c sitting at
// bit position p (p + b <= 10) of a 16-bit lane IS the float16 subnormal c * 2^(p-24), and
// mma.sync multiplies float16 subnormals exactly, so one AND with a mask turns two packed bytes into
// a half2 MMA operand.  The affine dequantisation is moved onto the small operands:
//   score(n,h) = sum_d (q[h,d] * ks[d,G]) * kc[n,d]  +  sum_d q[h,d] * km[d,G]      (G = group of n)
//   out(h,e)   = sum_n (p[h,n] * vs[n,D]) * vc[n,e]  +  sum_n p[h,n] * vm[n,D]      (D = group of e)
// i.e. the f16 products q*ks and p*vs are the B operands, the raw codes are the A operands, the two
// "zero" terms are one extra MMA each, and the power of two 2^(24-p) is applied to the accumulator.
// K is packed along tokens but contracted along channels (V the other way round); the PRMT that
// builds the half2 from two bytes of two neighbouring channel rows (token rows) does that transpose.
//
// Work split: a CTA owns a token range of one (segment, KV head); its warps take tiles of the range
// round-robin, each warp streaming its own tiles through a private 2-stage cp.async ring (no CTA
// barrier in the loop), with a private online-softmax state that is merged through shared memory at
// the end into ONE un-normalised partial (m, l, acc) per CTA.
#pragma once

#include <cuda.h>  // CUtensorMap (types only: the encoder is fetched from the driver at run time)

#include "common.cuh"
#include "decode_plan.h"

namespace pkv {
namespace mma {

constexpr int HD = 128;
#ifndef PKV_MMA_WARPS
#define PKV_MMA_WARPS 12
#endif
constexpr int NWARPS = PKV_MMA_WARPS;
#ifndef PKV_MMA_CTAS_PER_SM
#define PKV_MMA_CTAS_PER_SM 1
#endif
constexpr int CTAS_PER_SM = PKV_MMA_CTAS_PER_SM;  // co-resident CTAs drift apart and mix their phases
constexpr int NSTAGE = 2;
constexpr int NTHREADS = NWARPS * 32;
constexpr int kSmemBytes = (CTAS_PER_SM == 1 ? 225 : 112) * 1024;  // dynamic shared memory per CTA (227 KB per SM)
constexpr int kBarBytes = 256;           // mbarriers of the two key buffers
constexpr int kQRowBytes = 272;          // 128 f16 + 16 pad bytes
constexpr int kQBytes = 2304;            // q of the GQA group as float16 [8 heads][128], shared by all warps
constexpr int kQAbsBytes = 512;          // per channel max over the group's heads of |q|, as a float16 pair
constexpr int kOffQAbs = kBarBytes + kQBytes;
constexpr int kHeadBytes = kBarBytes + kQBytes + kQAbsBytes;  // shared memory in front of the key buffers

// Shared memory of a CTA:  [q][K buffer 0][K buffer 1][value ring of warp 0][value ring of warp 1]...
// A K buffer holds the keys of one SUPER-TILE (NSUB consecutive 64-token tiles of the CTA's range) for
// all warps: long row chunks make the scattered key rows cheap to fetch.  Warp w computes tile w of
// the super-tile and streams that tile's values through its own 2-stage ring.
template <int BITS>
struct Cfg {
    static constexpr int T = 64;                    // tokens per tile
    static constexpr int NG = T / 32;               // key groups per tile
    // tiles per super-tile: one per warp if the buffers fit
    static constexpr int NSUB_WANT = CTAS_PER_SM == 1 ? (BITS == 2 ? NWARPS : BITS == 4 ? 8 : 4)
                                                      : (BITS == 2 ? NWARPS : BITS == 4 ? 4 : 2);
    // a multiple of four tiles, so that a super-tile is a whole number of 64-byte key boxes at every width
    static constexpr int NSUB = (NSUB_WANT < NWARPS ? NSUB_WANT : NWARPS) / 4 * 4;
    static constexpr int KRB = T * BITS / 8;        // key code bytes per channel row of a tile (16/32/64)
    // Key codes of a super-tile sit in shared memory as boxes of 128 channel rows x 64 bytes (the shape a tiled
    // TMA copy delivers), with the four 16-byte chunks of a row permuted by (row >> 1) & 3 (the 64-byte swizzle
    // pattern): the four channel rows a lane reads per step then fall into different banks without padding.
    static constexpr int KBOX = 64;                 // bytes of a key code row inside a box
    static constexpr int KBOX_BYTES = HD * KBOX;    // 8 KB
    static constexpr int NBOX = NSUB * KRB / KBOX;  // boxes per super-tile
    static_assert(NSUB * KRB % KBOX == 0, "a super-tile is a whole number of boxes");
    static constexpr int MROW = (NSUB * NG * 2 + 15) / 16 * 16;  // key scale (or zero) row of a super-tile: f16 per group, 16-byte rows
    static constexpr int KBUF_BYTES = NBOX * KBOX_BYTES + 2 * HD * MROW;
    static constexpr int OFF_KS = NBOX * KBOX_BYTES;  // byte offsets inside a K buffer
    static constexpr int OFF_KM = OFF_KS + HD * MROW;
    static constexpr int VWPT = HD * BITS / 32;     // value code words per token (8/16/32)
    static constexpr int VROWS = T + T / 8;         // one pad row per 8 tokens spreads the four token
                                                    // blocks a load touches over different banks
    static constexpr int OFF_VS = VROWS * VWPT * 4; // byte offsets inside a value stage: codes, scale, zero
    static constexpr int OFF_VM = OFF_VS + T * 8;
    static constexpr int VSTAGE_BYTES = OFF_VM + T * 8;
    static constexpr int SMEM_BYTES = kHeadBytes + 2 * KBUF_BYTES + NSUB * NSTAGE * VSTAGE_BYTES;
};

constexpr int kMergeBytes = NWARPS * (8 * HD + 16) * 4 + NWARPS * 8 * 4;  // per-warp O[8][128] + m[8] + l[8], then the warps' weights
static_assert(kMergeBytes + kHeadBytes <= kSmemBytes && Cfg<2>::SMEM_BYTES <= kSmemBytes &&
              Cfg<4>::SMEM_BYTES <= kSmemBytes && Cfg<8>::SMEM_BYTES <= kSmemBytes, "shared memory budget");
static_assert(Cfg<2>::NG == 2 && Cfg<2>::VSTAGE_BYTES % 16 == 0, "tile geometry");
static_assert(kHeadBytes % 512 == 0 && Cfg<2>::KBUF_BYTES % 512 == 0 && Cfg<4>::KBUF_BYTES % 512 == 0 &&
              Cfg<8>::KBUF_BYTES % 512 == 0, "key boxes start on 512 bytes (the swizzle period)");

// Byte offset of 16-byte chunk `chunk` (counted along the super-tile's row) of channel row `row` inside the
// key code area of a K buffer.
__host__ __device__ constexpr int key_chunk_offset(int row, int chunk) {
    return (chunk >> 2) * (HD * 64) + row * 64 + ((((chunk & 3) ^ (row >> 1)) & 3) << 4);
}

inline int tile_tokens(int) { return 64; }

// Tensor maps of one KIVI segment's keys: codes as uint8 [Hkv*128 rows][row bytes] with 64-byte x 128-row boxes
// and the 64-byte swizzle; scales and zeros as float16 [Hkv*128 rows][groups] with boxes of one super-tile's
// groups x 128 rows.
struct KeyMaps {
    CUtensorMap codes;
    CUtensorMap scale;
    CUtensorMap mins;
};

// Segments of a launch whose keys travel through TMA (the longest ones; every map adds 384 bytes of parameters).
constexpr int kMaxKeyMaps = 4;

struct MmaArgs {
    const __half* q;
    float* pm;
    float* pl;
    float* pacc;
    int Hq, Hkv, G;
    float sm_scale;
    int n_segs;
    int work_offset;
    SegDev segs[kMaxInlineSegs];  // split_len counts TILES here
    KeyMaps kmaps[kMaxKeyMaps];  // segs[i].key_tma - 1 indexes this array (0 = no map)
};

// What a CTA needs besides its segment: the query rows of its sequence and where its partial goes.
struct CtaCtx {
    const __half* q;  // [Hq][128] of this CTA's sequence
    float* pm;
    float* pl;
    float* pacc;
    size_t widx;      // row of the partial arrays this CTA writes
    int Hq, G;
    float sm_scale;
};

// Batched decode: segment descriptors of all sequences and an explicit work list, both in device memory.
struct BatchWork {
    int seg;         // index into the segment table
    int seq;         // sequence (row block of q and out)
    int tile_begin;  // first tile of the item inside the segment
    int n_tiles;
    int part;        // row of the partial arrays
    int pad[3];
};
static_assert(sizeof(BatchWork) == 32, "work items are read as two 16-byte words");

struct BatchArgs {
    const __half* q;  // [batch][Hq][128]
    float* pm;
    float* pl;
    float* pacc;
    int Hq, Hkv, G;
    float sm_scale;
    const SegDev* segs;
    const BatchWork* work;
};

// ------------------------------------------------------------------ small PTX helpers
__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void tma_load_2d(unsigned smem_dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned addr, unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ unsigned prmt(unsigned a, unsigned b, unsigned sel) {
    unsigned r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(a));
    return r;
}
__device__ __forceinline__ unsigned hmul2(unsigned a, unsigned b) {
    unsigned r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ unsigned hmax2(unsigned a, unsigned b) {
    unsigned r;
    asm("max.NaN.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// a * b - hi in one fused float16x2 operation: the part of the product that `hi` = rn(a * b) lost
__device__ __forceinline__ unsigned hfma2_residual(unsigned a, unsigned b, unsigned hi) {
    unsigned r;
    asm("{.reg .b32 n; neg.f16x2 n, %3; fma.rn.f16x2 %0, %1, %2, n;}" : "=r"(r) : "r"(a), "r"(b), "r"(hi));
    return r;
}
__device__ __forceinline__ unsigned pack_half2(float lo, float hi) {
    unsigned r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void cp_async4(unsigned smem_addr, const void* g) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(g));
}
__device__ __forceinline__ void cp_async16(unsigned smem_addr, const void* g) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(g));
}
__device__ __forceinline__ void cp_async16_ca(unsigned smem_addr, const void* g) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(smem_addr), "l"(g));
}
__device__ __forceinline__ void cp_async16_zfill(unsigned smem_addr, const void* g, unsigned src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(g), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async8_zfill(unsigned smem_addr, const void* g, unsigned src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(smem_addr), "l"(g), "r"(src_bytes));
}
// ---- TMA copies global -> shared complete on an mbarrier that counts bytes.  One thread issues them and they
// bypass the load/store unit, which 16-byte cp.async copies at HBM rate keep busy.
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_inval(unsigned bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar));
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait: returns false if the phase did not complete within the iteration budget (the caller poisons
// its result instead of hanging the GPU).
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity) {
    for (int it = 0; it < (1 << 22); ++it) {
        unsigned ok;
        asm volatile(
            "{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ uint4 lds128(unsigned addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// plain loads through pointers derived from the shared array: the compiler folds constant offsets into the
// instruction, which hand-written ld.shared with a computed address register cannot
__device__ __forceinline__ unsigned ldp32(const char* p) { return *reinterpret_cast<const unsigned*>(p); }
__device__ __forceinline__ uint2 ldp64(const char* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ uint4 ldp128(const char* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ unsigned lds32(unsigned addr) {
    unsigned v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(unsigned addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// For lane row g: which word of a 32-element group holds its four codes, and the PRMT selectors that
// bring the byte(s) holding them to byte 0 (from the first source) and byte 2 (from the second).
template <int BITS>
struct LaneSel {
    unsigned word;    // word index inside the group
    unsigned sel[4];  // selectors (as many as the width needs)
    __device__ explicit LaneSel(int g) {
        auto mk = [](unsigned k) { return k | (k << 4) | ((4u + k) << 8) | ((4u + k) << 12); };
        if (BITS == 2) {
            word = g >> 2;
            sel[0] = mk(g & 3);
            sel[1] = sel[2] = sel[3] = sel[0];
        } else if (BITS == 4) {
            word = g >> 1;
            sel[0] = mk(2 * (g & 1));
            sel[1] = mk(2 * (g & 1) + 1);
            sel[2] = sel[3] = sel[0];
        } else {
            word = g;
            for (unsigned k = 0; k < 4; ++k) sel[k] = mk(k);
        }
    }
};

// r[i] = half2(code_i of wa, code_i of wb) as float16 subnormals, i = 0..3 (the lane's four codes).
// The value of r[i] is code * 2^(pos<BITS>(i) - 24).
template <int BITS>
__device__ __forceinline__ void extract4(unsigned wa, unsigned wb, const LaneSel<BITS>& ls, unsigned (&r)[4]) {
    if (BITS == 2) {
        const unsigned x = prmt(wa, wb, ls.sel[0]);
        r[0] = x & 0x00030003u;
        r[1] = x & 0x000C000Cu;
        r[2] = x & 0x00300030u;
        r[3] = x & 0x00C000C0u;
    } else if (BITS == 4) {
        const unsigned x0 = prmt(wa, wb, ls.sel[0]);
        const unsigned x1 = prmt(wa, wb, ls.sel[1]);
        r[0] = x0 & 0x000F000Fu;
        r[1] = x0 & 0x00F000F0u;
        r[2] = x1 & 0x000F000Fu;
        r[3] = x1 & 0x00F000F0u;
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) r[i] = prmt(wa, wb, ls.sel[i]) & 0x00FF00FFu;
    }
}
// 2^(24 - bit position of code i)
template <int BITS>
__device__ __forceinline__ constexpr float unscale(int i) {
    return BITS == 2 ? (i == 0 ? 16777216.f : i == 1 ? 4194304.f : i == 2 ? 1048576.f : 262144.f)
         : BITS == 4 ? ((i & 1) ? 1048576.f : 16777216.f)
                     : 16777216.f;
}

}  // namespace mma
}  // namespace pkv

namespace pkv {
namespace mma {
// Whether the tensor-core kernel can take this segment (otherwise the generic kernel does).
bool eligible(const pkv_segment_t& s, int Hq, int Hkv, int hd);
long long tiles_of(const pkv_segment_t& s);
// Launch over `work` CTAs per KV head; a.segs[*].work_begin is relative to this launch.  KIVI and float16 segments.
int launch(const MmaArgs& a, int work, int Hkv, cudaStream_t stream);
// The same for per-token and float16 segments.
int launch_per_token(const MmaArgs& a, int work, int Hkv, cudaStream_t stream);
// Launch over a device-resident work list of `work` items per KV head.
int launch_batched(const BatchArgs& a, int work, int Hkv, cudaStream_t stream);
// Tensor maps for the keys of `s` (a KIVI segment the tensor-core kernel takes).  False when the layout cannot be
// described (rows or scale rows not a multiple of 16 bytes apart) or the driver refuses: the kernel then
// fetches the keys with cp.async.  Maps are cached per thread by pointers and sizes.
bool make_key_maps(const pkv_segment_t& s, int Hkv, KeyMaps* out);
}  // namespace mma
}  // namespace pkv

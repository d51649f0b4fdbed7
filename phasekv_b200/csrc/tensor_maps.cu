// Tensor maps for the key tensors of KIVI segments (host side of the tiled TMA path of the split-K kernel).
//
// cuTensorMapEncodeTiled is a driver entry point; it is looked up through the runtime
// (cudaGetDriverEntryPoint), so the library links against nothing but the CUDA runtime.  Encoding a map is a
// pure host computation of a few hundred nanoseconds; maps are kept per thread, keyed by pointers and sizes,
// because a decode loop presents the same frozen segments again and again.
#include <string.h>

#include <vector>

#include "decode_mma.cuh"

namespace pkv {
namespace mma {
namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encoder() {
    static EncodeFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeFn>(p);
    }();
    return fn;
}

// rank-2 map over [rows][dim0] with `pitch_bytes` between rows and a box of box0 x 128 elements
bool encode_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t dim0,
               uint64_t rows, uint64_t pitch_bytes, uint32_t box0, CUtensorMapSwizzle swizzle) {
    EncodeFn fn = encoder();
    if (!fn || dim0 == 0 || rows == 0) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u) || pitch_bytes < dim0 * elem_bytes) return false;
    if ((box0 * elem_bytes) & 15u || box0 > 256) return false;
    const cuuint64_t dims[2] = {dim0, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {box0, (cuuint32_t)HD};
    const cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct Entry {
    const void *kp, *ks, *km;
    int64_t S, pitch, meta_pitch;
    int bits, Hkv, device;
    KeyMaps maps;
};
constexpr size_t kCacheEntries = 512;

}  // namespace

bool make_key_maps(const pkv_segment_t& s, int Hkv, KeyMaps* out) {
    if (s.kind != PKV_SEG_KIVI || s.k_bits != s.v_bits) return false;
    const int64_t pitch = s.k_row_pitch ? s.k_row_pitch : ceil_div(s.seq_len * s.k_bits, 8);
    const int64_t meta_pitch = s.k_meta_pitch ? s.k_meta_pitch : ceil_div(s.seq_len, 32);
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return false;
    static thread_local std::vector<Entry> cache;
    static thread_local size_t next = 0;
    for (const Entry& e : cache)
        if (e.kp == s.k_packed && e.ks == s.k_scale && e.km == s.k_mins && e.S == s.seq_len && e.pitch == pitch &&
            e.meta_pitch == meta_pitch && e.bits == s.k_bits && e.Hkv == Hkv && e.device == device) {
            *out = e.maps;
            return true;
        }
    const uint64_t rows = (uint64_t)Hkv * HD;
    const uint64_t row_bytes = (uint64_t)ceil_div(s.seq_len * s.k_bits, 8);
    const uint64_t groups = (uint64_t)ceil_div(s.seq_len, 32);
    const uint32_t meta_box = s.k_bits == 2 ? Cfg<2>::NSUB * Cfg<2>::NG
                            : s.k_bits == 4 ? Cfg<4>::NSUB * Cfg<4>::NG : Cfg<8>::NSUB * Cfg<8>::NG;
    Entry e = {s.k_packed, s.k_scale, s.k_mins, s.seq_len, pitch, meta_pitch, s.k_bits, Hkv, device, {}};
    if (!encode_2d(&e.maps.codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, s.k_packed, row_bytes, rows, (uint64_t)pitch, 64,
                   CU_TENSOR_MAP_SWIZZLE_64B) ||
        !encode_2d(&e.maps.scale, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, s.k_scale, groups, rows, (uint64_t)meta_pitch * 2,
                   meta_box, CU_TENSOR_MAP_SWIZZLE_NONE) ||
        !encode_2d(&e.maps.mins, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, s.k_mins, groups, rows, (uint64_t)meta_pitch * 2,
                   meta_box, CU_TENSOR_MAP_SWIZZLE_NONE))
        return false;
    if (cache.size() < kCacheEntries) {
        cache.push_back(e);
    } else {
        cache[next] = e;
        next = (next + 1) % kCacheEntries;
    }
    *out = e.maps;
    return true;
}

}  // namespace mma
}  // namespace pkv

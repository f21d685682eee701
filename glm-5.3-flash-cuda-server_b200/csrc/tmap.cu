// tmap.cu -- TMA tensor maps over byte matrices, encoded once and remembered.
//
// A CUtensorMap is a pure function of (base address, extent, row pitch, box, swizzle), so a map
// that was encoded once for a weight can be reused by every later call on that weight: the gemv
// and gemm entry points then cost a table look-up instead of a driver call per tensor (about a
// microsecond each, twelve per fused sibling launch).  The table is a small direct-mapped cache;
// a colliding key simply replaces the older entry, and an entry can never be stale because the
// key is everything the map depends on.
#include "b200_internal.h"
#include <cuda.h>
#include <cstring>
#include <mutex>

namespace b200 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

bool tmap_available() { return encode_fn() != nullptr; }

static bool encode(void* out, const void* base, size_t rows, size_t row_bytes, int box_bytes, int box_rows, bool swz) {
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {(cuuint32_t)box_bytes, (cuuint32_t)box_rows};
    const cuuint32_t es[2] = {1, 1};
    EncodeTiledFn fn = encode_fn();
    return fn && fn(static_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {
struct Key { const void* base; size_t rows, row_bytes; int box_bytes, box_rows, swz, used; };
struct Entry { Key k; alignas(64) unsigned char map[128]; };
constexpr int CACHE_SLOTS = 2048;
Entry g_cache[CACHE_SLOTS];
std::mutex g_cache_mu;
}  // namespace

bool tmap_u8_2d(void* out, const void* base, size_t rows, size_t row_bytes, int box_bytes, int box_rows, bool swz, bool cached) {
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    if (!cached) return encode(out, base, rows, row_bytes, box_bytes, box_rows, swz);
    size_t h = (size_t)((uintptr_t)base >> 4) * 0x9E3779B97F4A7C15ull;
    h ^= (rows * 1315423911u) ^ (row_bytes << 7) ^ ((size_t)box_rows << 20) ^ ((size_t)box_bytes << 3) ^ (size_t)swz;
    Entry& e = g_cache[(h >> 17) % CACHE_SLOTS];
    std::lock_guard<std::mutex> lk(g_cache_mu);
    if (e.k.used && e.k.base == base && e.k.rows == rows && e.k.row_bytes == row_bytes && e.k.box_bytes == box_bytes &&
        e.k.box_rows == box_rows && e.k.swz == (int)swz) {
        memcpy(out, e.map, 128);
        return true;
    }
    if (!encode(e.map, base, rows, row_bytes, box_bytes, box_rows, swz)) { e.k.used = 0; return false; }
    e.k = Key{base, rows, row_bytes, box_bytes, box_rows, (int)swz, 1};
    memcpy(out, e.map, 128);
    return true;
}

// Scale slabs of a weight with K columns: 128-byte swizzled boxes when K/16 is a multiple of 128,
// one plain box of K/16 bytes when that is at most 256.
bool scale_box(int K, int* box, int* swz) {
    if ((K / 16) % 128 == 0) { *box = 128; *swz = 1; return true; }
    if (K / 16 <= 256) { *box = K / 16; *swz = 0; return true; }
    return false;
}

}  // namespace b200

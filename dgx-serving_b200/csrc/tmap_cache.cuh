// Host-side TMA tensor maps (cuTensorMapEncodeTiled through the runtime's driver entry point; the library links only
// the CUDA runtime) and a small cache of them.  A tensor map depends only on the address and the shape it describes,
// never on the data, so a map built for a weight tensor stays valid for as long as a tensor of that shape lives at
// that address; decode loops call with the same weights step after step and skip the encoding (about a microsecond
// per map) on every call but the first.
#pragma once
#include <cuda.h>
#include <cstring>
#include "common.cuh"

namespace w4a8 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D byte tensor [rows][row_bytes] (pitch = row_bytes), box [box_rows][box_bytes].
inline int make_tmap_u8(CUtensorMap *tm, const void *ptr, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes,
                        uint32_t box_rows, CUtensorMapSwizzle swz,
                        CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_128B) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(W4A8_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, swz, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(W4A8_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
    return W4A8_OK;
}

// The same through a direct-mapped cache (single host thread per device, the library's convention).  The map is
// copied out, so a later call that evicts the slot cannot change a map already handed to a launch.
inline int tmap_cached(CUtensorMap *out, const void *ptr, uint64_t row_bytes, uint64_t rows, uint32_t box_bytes,
                       uint32_t box_rows, CUtensorMapSwizzle swz, CUtensorMapL2promotion promo) {
    struct Key { const void *ptr; uint64_t row_bytes, rows; uint32_t box_bytes, box_rows; int swz, promo; };
    struct Slot { Key key; CUtensorMap map; bool used; };
    constexpr int SLOTS = 1024;
    static Slot *slots = nullptr;
    if (!slots) slots = new Slot[SLOTS]();
    Key k;
    memset(&k, 0, sizeof(k));
    k.ptr = ptr; k.row_bytes = row_bytes; k.rows = rows; k.box_bytes = box_bytes; k.box_rows = box_rows;
    k.swz = (int)swz; k.promo = (int)promo;
    uint64_t h = reinterpret_cast<uintptr_t>(ptr) * 0x9E3779B97F4A7C15ull;
    h ^= (row_bytes * 0xC2B2AE3D27D4EB4Full) ^ (rows << 17) ^ ((uint64_t)box_bytes << 7) ^ ((uint64_t)box_rows << 3) ^ (uint64_t)k.swz;
    Slot &s = slots[(h >> 20) & (SLOTS - 1)];
    if (!s.used || memcmp(&s.key, &k, sizeof(k)) != 0) {
        int rc = make_tmap_u8(&s.map, ptr, row_bytes, rows, box_bytes, box_rows, swz, promo);
        if (rc != W4A8_OK) { s.used = false; return rc; }
        s.key = k;
        s.used = true;
    }
    *out = s.map;
    return W4A8_OK;
}

}  // namespace w4a8

// Tensor maps for the tiled bulk copies (TMA).  The encoder lives in the driver; it is looked up
// through the runtime so that the library needs no link against the driver library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <mutex>

namespace b200wkv {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tmap_encoder() {
    static std::once_flag once;
    static EncodeTiledFn fn = nullptr;
    std::call_once(once, []() {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// bf16 matrix [rows][cols] (cols contiguous), box of box_rows x box_cols elements: the box lands in shared
// memory row-major with box_cols * 2 bytes per row.  With `swizzle128` (rows of exactly 128 bytes, destination
// 1024-byte aligned) the 16-byte pieces of row r are stored at piece index XOR (r mod 8), so that threads which
// own consecutive rows read one piece each without bank conflicts.
inline bool make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                              uint32_t box_cols, bool swizzle128 = false) {
    EncodeTiledFn enc = tmap_encoder();
    if (enc == nullptr || base == nullptr || (reinterpret_cast<uintptr_t>(base) & 15u) != 0) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
               CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor maps of up to seven bf16 streams viewed as [B*T tokens][H*64 channels]; a box is the 64 rows
// x 64 channels of one head from one token on (8 KB, rows of 128 bytes in shared memory).
struct StreamMaps {
    CUtensorMap m[7];
};

// A tensor map depends only on (base address, shape), and a training loop calls with the same buffers
// step after step, so each host thread remembers the last few sets it encoded (thread-local: no lock,
// nothing shared between the executor threads of different devices).
struct StreamMapKey {
    const void* base[7];
    int count, B, T, H, swizzle;
};
inline bool make_stream_maps(StreamMaps* out, const void* const* bases, int count, int B, int T, int H, bool swizzle128 = false) {
    constexpr int kSlots = 8;
    struct Slot { StreamMapKey key; StreamMaps maps; bool used; };
    thread_local Slot cache[kSlots];
    thread_local int next = 0;
    StreamMapKey key;
    memset(&key, 0, sizeof(key));
    for (int m = 0; m < 7; ++m) key.base[m] = bases[m < count ? m : 0];
    key.count = count; key.B = B; key.T = T; key.H = H; key.swizzle = swizzle128 ? 1 : 0;
    for (int i = 0; i < kSlots; ++i)
        if (cache[i].used && memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
            *out = cache[i].maps;
            return true;
        }
    for (int m = 0; m < 7; ++m)
        if (!make_tmap_bf16_2d(&out->m[m], key.base[m], (uint64_t)B * T, (uint64_t)H * 64, 64, 64, swizzle128)) return false;
    Slot& s = cache[next];
    next = (next + 1) % kSlots;
    s.key = key; s.maps = *out; s.used = true;
    return true;
}

}  // namespace b200wkv

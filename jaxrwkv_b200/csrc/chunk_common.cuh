// Constants and small helpers shared by the chunked (tcgen05) forward and backward kernels.
#pragma once
#include "common.cuh"

namespace b200wkv {

constexpr int kC = 64;                 // tokens per full chunk == checkpoint spacing
constexpr int CB64 = 1040;             // column-block pitch of a 64-row operand slab (64*16 + 16 pad)
constexpr int CB128 = 2064;            // ... of a 128-row slab
constexpr int SLAB64 = 8 * CB64;       // 8320
constexpr int SLAB128 = 8 * CB128;     // 16512
constexpr int LF_PITCH = 68;           // floats per row of fp32 matrices kept in shared memory
constexpr float kCumFloor = -60.f;     // floor of the in-chunk cumulative log-decay (keeps 1/L finite)

// Residual written by the chunked forward for the chunked backward (all fp32):
//   [B*H][ceil(T/64)][64][64]  state entering every 64-token block (before a start flag is applied)
//   [B*H][64][64]              state at position `length` (what the forward returns as s_out)
inline size_t chunk_residual_floats(int B, int T, int H) {
    return (size_t)B * H * ((size_t)((T + kC - 1) / kC) + 1) * kN * kN;
}

__device__ __forceinline__ uint32_t pack2(float x, float y) {
    __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
    return make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
}
__device__ __forceinline__ void unpack8(uint4 raw, float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x; f[2 * i + 1] = t.y;
    }
}
// 16-byte store of row `row`, column block `cblk` of a slab
__device__ __forceinline__ void slab_store(unsigned char* slab, int cb, int row, int cblk, uint4 val) {
    *reinterpret_cast<uint4*>(slab + cblk * cb + row * 16) = val;
}


}  // namespace b200wkv

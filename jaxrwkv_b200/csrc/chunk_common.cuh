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


// ---------------------------------------------------------------------------------------------
// X = (I - L)^-1 for a 64x64 strictly lower triangular L, by all NT threads of the CTA, in fp32.
// L and X are row-major with LF_PITCH floats per row; scr holds 32 x TRI_SCR_PITCH floats.
// Recursive blocking: the four 16x16 diagonal blocks by forward substitution, then
// X21 = X22 (L21 X11) for the two 32x32 blocks and once more for the whole matrix.
// Every thread must call it (it synchronises the CTA); X is complete when it returns.
constexpr int TRI_SCR_PITCH = 36;
constexpr int TRI_SCR_FLOATS = 32 * TRI_SCR_PITCH;

template <int NT>
__device__ __forceinline__ void tri_inverse_64(const float* __restrict__ L, float* __restrict__ X,
                                               float* __restrict__ scr, int tid) {
    // ---- diagonal blocks (threads 0..63) and zero fill of the blocks above the diagonal (the rest)
    if (tid < 64) {
        const int d = tid >> 4, c = tid & 15, o = d * 16;
        float x[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            float acc = (t == c) ? 1.f : 0.f;
#pragma unroll
            for (int m = 0; m < t; ++m) acc = fmaf(L[(o + t) * LF_PITCH + o + m], x[m], acc);
            x[t] = acc;
        }
#pragma unroll
        for (int t = 0; t < 16; ++t) X[(o + t) * LF_PITCH + o + c] = x[t];
    } else {
        for (int idx = tid - 64; idx < 6 * 256; idx += NT - 64) {
            const int blk = idx >> 8, e = idx & 255;
            // blocks (bi, bj) with bj > bi: (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
            const int bi = (blk < 3) ? 0 : (blk < 5 ? 1 : 2);
            const int bj = (blk < 3) ? blk + 1 : (blk < 5 ? blk - 1 : 3);
            X[(bi * 16 + (e >> 4)) * LF_PITCH + bj * 16 + (e & 15)] = 0.f;
        }
    }
    __syncthreads();
    // ---- 16 -> 32: two independent merges; W_q = L21 X11, then X21 = X22 W_q
    for (int idx = tid; idx < 512; idx += NT) {
        const int q = idx >> 8, i = (idx >> 4) & 15, j = idx & 15, o = q * 32;
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) acc = fmaf(L[(o + 16 + i) * LF_PITCH + o + m], X[(o + m) * LF_PITCH + o + j], acc);
        scr[(q * 16 + i) * TRI_SCR_PITCH + j] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < 512; idx += NT) {
        const int q = idx >> 8, i = (idx >> 4) & 15, j = idx & 15, o = q * 32;
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) acc = fmaf(X[(o + 16 + i) * LF_PITCH + o + 16 + m], scr[(q * 16 + m) * TRI_SCR_PITCH + j], acc);
        X[(o + 16 + i) * LF_PITCH + o + j] = acc;
    }
    __syncthreads();
    // ---- 32 -> 64: W = L21 X11 (32x32x32), then X21 = X22 W ; four outputs per step and thread
    for (int idx = tid; idx < 256; idx += NT) {
        const int i = idx >> 3, j0 = (idx & 7) * 4;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
        for (int m = 0; m < 32; ++m) {
            const float l = L[(32 + i) * LF_PITCH + m];
            const float4 x4 = *reinterpret_cast<const float4*>(&X[m * LF_PITCH + j0]);
            a0 = fmaf(l, x4.x, a0); a1 = fmaf(l, x4.y, a1); a2 = fmaf(l, x4.z, a2); a3 = fmaf(l, x4.w, a3);
        }
        *reinterpret_cast<float4*>(&scr[i * TRI_SCR_PITCH + j0]) = make_float4(a0, a1, a2, a3);
    }
    __syncthreads();
    for (int idx = tid; idx < 256; idx += NT) {
        const int i = idx >> 3, j0 = (idx & 7) * 4;
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
        for (int m = 0; m < 32; ++m) {
            const float l = X[(32 + i) * LF_PITCH + 32 + m];
            const float4 w4 = *reinterpret_cast<const float4*>(&scr[m * TRI_SCR_PITCH + j0]);
            a0 = fmaf(l, w4.x, a0); a1 = fmaf(l, w4.y, a1); a2 = fmaf(l, w4.z, a2); a3 = fmaf(l, w4.w, a3);
        }
        *reinterpret_cast<float4*>(&X[(32 + i) * LF_PITCH + j0]) = make_float4(a0, a1, a2, a3);
    }
    __syncthreads();
}

// bf16 copy of a 64x64 fp32 matrix (pitch LF_PITCH) into rows 0..63 of an operand slab
template <int NT>
__device__ __forceinline__ void fp32_to_slab64(const float* __restrict__ X, unsigned char* slab, int cb, int tid) {
    for (int idx = tid; idx < 512; idx += NT) {
        const int row = idx & 63, blk = idx >> 6;
        float f[8];
        *reinterpret_cast<float4*>(&f[0]) = *reinterpret_cast<const float4*>(&X[row * LF_PITCH + blk * 8]);
        *reinterpret_cast<float4*>(&f[4]) = *reinterpret_cast<const float4*>(&X[row * LF_PITCH + blk * 8 + 4]);
        slab_store(slab, cb, row, blk, pack8(f));
    }
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

}  // namespace b200wkv

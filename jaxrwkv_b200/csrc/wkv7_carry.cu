// RWKV-7 WKV backward, part 1 of 2: the state-gradient carry.
//
// The forward leaves, for every 64-token block it walked as one chunk, what makes the block an affine
// map of the state that enters it (S0, row = value index i, column = key index j):
//     S_C = S0 diag(L_C) + S0 M' + (terms without S0)          M' = W~^T B^      (64 x 64)
//     y_t = R-_t S0^T    + (terms without S0)                   R- = R~ + P_rb W~ (64 tokens x 64)
// so the gradient of the state entering the block follows from the gradient dS of the state leaving it by
//     dS0 = dS diag(L_C) + dS M'^T + dY^T R-
// This is the only sequential part of the backward: two 64x64x64 products per block and sequence.  One
// CTA of four warps walks one sequence from its last block to its first with the state gradient in
// registers (fp32, each warp 16 rows as mma.sync accumulator tiles): an accumulator tile is already in the
// register layout of the next product's left operand, so nothing passes through shared memory between
// blocks.  M', R-, dY and L_C of the blocks ahead arrive by cp.async, two or three blocks deep.  The gradient
// leaving every block goes to global memory in bf16; the second part (wkv7_grad.cu) turns it, block by
// block and in parallel over all blocks, into the gradients of the six streams.
//
// Handles the sequences the forward marked as walked in full saved blocks (T a multiple of 64, start
// flags only at multiples of 64, length 0, a multiple of 64, or >= T); the others are left to the
// one-kernel backward (wkv7_chunk_bwd.cu).
//
// Semantics: reverse-mode derivative of BaseRWKV.inner_loop of jaxrwkv (src/jaxrwkv/rwkv7.py:199-220).
#include "common.cuh"
#include "chunk_common.cuh"
#include "device_once.cuh"

namespace b200wkv {

namespace {

constexpr int PITCH = 72;                       // bf16 per shared-memory row (144 bytes): ldmatrix and 4-byte reads hit 32 different banks
// Depth of the cp.async ring: three stages (two CTAs per SM) while every sequence has a resident CTA anyway, two stages
// (four CTAs per SM) when there are more sequences than that, so that more of these latency-bound chains run at once.
struct CarryStage {
    __nv_bfloat16 m[8][kC][8];                  // M'[j][j'] as it lies in the residual: 8 column blocks of [64 rows j][8 columns j']
                                                // (a linear copy; the eight rows of an ldmatrix tile are 128 contiguous bytes)
    __nv_bfloat16 rb[kC][PITCH];                // R-[t][j]
    __nv_bfloat16 dy[kC][PITCH];                // dY[t][i]
    float lam[kN];                              // L_C[j]
};
template <int kStages>
constexpr int carry_smem() { return kStages * (int)sizeof(CarryStage); }

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(row)));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(row)));
}
// D(16x8, fp32) += A(16x16, bf16, row) B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int kStages>
__global__ void __launch_bounds__(128)
wkv7_carry_bwd_kernel(int Tlen, int H, const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                      const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ds_out,
                      const __nv_bfloat16* __restrict__ mprime, const __nv_bfloat16* __restrict__ rbar,
                      const float* __restrict__ lam, const int* __restrict__ fast, const int* __restrict__ residual_mark,
                      __nv_bfloat16* __restrict__ dstate, __nv_bfloat16* __restrict__ ds0) {
    if (*residual_mark != 0) return;            // the forward fell back to the sequential kernels
    const int bh = blockIdx.x;
    if (fast[bh] == 0) return;                  // left to the one-kernel backward
    extern __shared__ __align__(128) unsigned char smem[];
    CarryStage* stages = reinterpret_cast<CarryStage*>(smem);
    const int bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, q = lane & 3;
    const int i0 = warp * 16;                   // this warp's rows of the state gradient
    const int L = min((int)length[bi], Tlen);
    const int nBlk = Tlen / kC;
    const size_t tok_stride = (size_t)H * kN;
    const size_t seq_base = (size_t)bi * Tlen * tok_stride + (size_t)h * kN;
    const size_t st_base = (size_t)bh * kN * kN;

    auto issue = [&](int blk) {
        if (blk >= 0) {
            CarryStage& s = stages[blk % kStages];
            const size_t slot = (size_t)bh * nBlk + blk;
            for (int c = tid; c < 512; c += 128) {
                const int rr = c >> 3, c8 = (c & 7) * 8;
                cp_async16(&s.m[c >> 6][c & 63][0], mprime + slot * (kN * kN) + (size_t)c * 8);
                cp_async16(&s.rb[rr][c8], rbar + seq_base + (size_t)(blk * kC + rr) * tok_stride + c8);
                if (dy != nullptr) cp_async16(&s.dy[rr][c8], dy + seq_base + (size_t)(blk * kC + rr) * tok_stride + c8);
            }
            if (tid < 16) cp_async16(&s.lam[tid * 4], lam + slot * kN + tid * 4);
        }
        cp_async_commit();                      // an empty group keeps the group count in step
    };

    float acc[8][4];                            // dS rows i0 + g, i0 + g + 8; column tile nt: columns 8 nt + 2q, + 1
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;

    auto add_ds_out = [&]() {
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(ds_out + st_base + (size_t)(i0 + g) * kN + nt * 8 + 2 * q);
            const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(ds_out + st_base + (size_t)(i0 + g + 8) * kN + nt * 8 + 2 * q);
            const float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(hi);
            acc[nt][0] += a.x; acc[nt][1] += a.y; acc[nt][2] += b.x; acc[nt][3] += b.y;
        }
    };

#pragma unroll
    for (int i = 1; i < kStages; ++i) issue(nBlk - i);
    uint8_t flag_here = new_starts[(size_t)bi * Tlen + (size_t)(nBlk - 1) * kC];   // start flag of the block's first token
    for (int blk = nBlk - 1; blk >= 0; --blk) {
        cp_async_wait<kStages - 2>();           // the copies of block blk have landed (younger groups may be in flight)
        __syncthreads();                        // ... for every thread; and everyone is done with the stage refilled next
        issue(blk - (kStages - 1));
        const uint8_t flag_next = (blk > 0) ? new_starts[(size_t)bi * Tlen + (size_t)(blk - 1) * kC] : 0;   // asked for a block ahead
        const CarryStage& s = stages[blk % kStages];
        const int p1 = (blk + 1) * kC;
        // cotangent of the returned state enters behind token length - 1
        if (p1 == L && ds_out != nullptr) add_ds_out();
        // the gradient leaving this block, in bf16: to global memory for the gradient kernel, and as the left
        // operand of the next product
        uint32_t afrag[4][4];
        {
            __nv_bfloat16* out = dstate + ((size_t)bh * nBlk + blk) * kN * kN;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const uint32_t lo = pack2(acc[nt][0], acc[nt][1]), hi = pack2(acc[nt][2], acc[nt][3]);
                // (8 column blocks of [64 rows][8]: eight lanes' rows are one 128-byte line)
                *reinterpret_cast<uint32_t*>(out + nt * (kN * 8) + (i0 + g) * 8 + 2 * q) = lo;
                *reinterpret_cast<uint32_t*>(out + nt * (kN * 8) + (i0 + g + 8) * 8 + 2 * q) = hi;
                afrag[nt >> 1][(nt & 1) * 2] = lo;
                afrag[nt >> 1][(nt & 1) * 2 + 1] = hi;
            }
        }
        // dS diag(L_C) in fp32
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float2 l2 = *reinterpret_cast<const float2*>(&s.lam[nt * 8 + 2 * q]);
            acc[nt][0] *= l2.x; acc[nt][1] *= l2.y; acc[nt][2] *= l2.x; acc[nt][3] *= l2.y;
        }
        // += dS M'^T : B[k = j'][n = j] = M'[j][j'], read along the rows of M'
        // (one ldmatrix.x4 fetches the two 8x8 blocks of each of two column tiles: rows j of M', 16 values of j')
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;    // (tile 2 np: b0, b2), (tile 2 np + 1: b1, b3)
                ldmatrix_x4(b0, b1, b2, b3, &s.m[ks * 2 + (lane >> 4)][np * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)][0]);
                mma_bf16(acc[2 * np], afrag[ks][0], afrag[ks][1], afrag[ks][2], afrag[ks][3], b0, b2);
                mma_bf16(acc[2 * np + 1], afrag[ks][0], afrag[ks][1], afrag[ks][2], afrag[ks][3], b1, b3);
            }
        // += dY^T R- : A[m = i][k = t] = dY[t][i] and B[k = t][n = j] = R-[t][j], both fetched transposed
        if (dy != nullptr) {
            const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4_trans(a0, a1, a2, a3, &s.dy[ks * 16 + (mi >> 1) * 8 + r8][i0 + (mi & 1) * 8]);
#pragma unroll
                for (int np = 0; np < 4; ++np) {
                    uint32_t b0, b1, b2, b3;    // column tiles 2 np (b0, b1) and 2 np + 1 (b2, b3)
                    ldmatrix_x4_trans(b0, b1, b2, b3, &s.rb[ks * 16 + (mi & 1) * 8 + r8][(np * 2 + (mi >> 1)) * 8]);
                    mma_bf16(acc[np * 2], a0, a1, a2, a3, b0, b1);
                    mma_bf16(acc[np * 2 + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        // a start flag on the block's first token cuts the dependency on everything before it
        if (flag_here != 0) {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
        }
        flag_here = flag_next;
    }
    if (L == 0 && ds_out != nullptr) add_ds_out();   // the returned state IS the input state
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
        *reinterpret_cast<uint32_t*>(ds0 + st_base + (size_t)(i0 + g) * kN + nt * 8 + 2 * q) = pack2(acc[nt][0], acc[nt][1]);
        *reinterpret_cast<uint32_t*>(ds0 + st_base + (size_t)(i0 + g + 8) * kN + nt * 8 + 2 * q) = pack2(acc[nt][2], acc[nt][3]);
    }
}

}  // namespace

int wkv7_carry_bwd(cudaStream_t st, int B, int T, int H, const uint32_t* length, const uint8_t* ns, const void* dy,
                   const void* ds_out, void* residual, const int* residual_mark, void* ds0) {
    typedef __nv_bfloat16 bf;
    static DeviceOnce smem_attr;
    if (!smem_attr.ok([]() {
            cudaError_t e = cudaFuncSetAttribute(wkv7_carry_bwd_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, carry_smem<3>());
            if (e != cudaSuccess) return e;
            return cudaFuncSetAttribute(wkv7_carry_bwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, carry_smem<2>());
        }))
        return B200WKV_ELAUNCH;
    const CarryLayout lay = carry_layout(B, T, H);
    char* base = static_cast<char*>(residual);
    const bool deep = (long long)B * H <= 2LL * sm_count_of_current_device();
    auto launch = deep ? wkv7_carry_bwd_kernel<3> : wkv7_carry_bwd_kernel<2>;
    launch<<<B * H, 128, deep ? carry_smem<3>() : carry_smem<2>(), st>>>(T, H, length, ns, (const bf*)dy, (const bf*)ds_out, (const bf*)(base + lay.mprime),
                                                                         (const bf*)(base + lay.rbar), (const float*)(base + lay.lam),
                                                                         (const int*)(base + lay.fast), residual_mark, (bf*)(base + lay.dstate), (bf*)ds0);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace b200wkv

// RWKV-7 WKV backward, part 2 of 2: the gradients of the six streams, one 64-token block at a time and
// all blocks in parallel (bf16 I/O, tcgen05.mma with fp32 accumulators in TMEM).
//
// Part 1 (wkv7_carry.cu) has left the gradient dS of the state leaving every block; the forward has left
// the state S0 entering it and its operands T = (I - A_ab)^-1, A_ak, P_rb, P_rk, sa.  With those a block no
// longer depends on its neighbours, so the blocks of all sequences form one flat work list that persistent
// CTAs (two per SM: 113 KB of shared memory and 256 TMEM columns each) take in turn.  Per block, with
// L = in-block cumulative decay (L_C at the block end) and dSL = dS diag(L_C):
//   Gd    = B~ dSL^T + P_rb^T dY                  dG = T^T Gd        (row t of dG is dS_t b_t)
//   dV    = K~ dSL^T + P_rk^T dY + A_ak^T dG
//   W     = [V; sa] [dY; dG]^T                    upper-triangular Gram blocks
//   dK~'  = W_v,dG A~ + W_v,dy R~ + V  dSL        dk = dK~' / L_t
//   dB~'  = W_sa,dG A~ + W_sa,dy R~ + sa dSL      db = dB~' / L_t
//   dR~'  = dY S0 + W_sa,dy^T B~ + W_v,dy^T K~    dr = dR~' * L_t
//   dA~'  = dG S0 + W_sa,dG^T B~ + W_v,dG^T K~    da = dA~' * L_{t-1}
// The decay gradient uses D_t = sum_i dS_t[i,:] S_t[i,:]: with u_t = r dr - b db - k dk + a da the recurrence
// D_{t-1} = D_t + u_t holds and d(log decay)_t = D_{t-1} - a_t da_t; D at the block end comes exactly from dS
// and the state leaving the block (the next block's saved S0, or the state at `length`).
//
// Shared memory holds every operand as an unpadded slab (8 column blocks of [rows][16 bytes]); the thread
// that scales a token's operands owns one token and two column blocks, so that its 16-byte stores and the
// 128-byte-swizzled staging rows it reads are both free of bank conflicts.  The raw rows of the next block
// arrive by tiled bulk copies (cp.async.bulk.tensor, no multicast) while this block's last epilogue runs.
// The decay factors 1/L_t, L_t, L_{t-1} and the log-decay, computed where the operands are scaled, wait in a
// per-CTA scratch in global memory (32 KB that stays in L2) for the last epilogue, whose threads own other
// (token, channel) pairs: shared memory has no room for them and recomputing them costs more than the round trip.
//
// Semantics: reverse-mode derivative of BaseRWKV.inner_loop of jaxrwkv (src/jaxrwkv/rwkv7.py:199-220).
#include "common.cuh"
#include "tc05.cuh"
#include "chunk_common.cuh"
#include "tmap.cuh"

namespace b200wkv {

namespace {

constexpr int T64 = 8192, T128 = 16384;     // bytes of a 64-row / 128-row slab
constexpr int P64 = 1024, P128 = 2048;      // their column-block pitches
constexpr int OFF_AR = 0;                   // [A~ ; R~]   128-row
constexpr int OFF_BK = OFF_AR + T128;       // [B~ ; K~]   128-row
constexpr int OFF_VSA = OFF_BK + T128;      // [V ; sa]    128-row
constexpr int OFF_DD = OFF_VSA + T128;      // [dY ; dG]   128-row
constexpr int OFF_W = OFF_DD + T128;        // T | A_ak | dSL | P_rb (64-row each), later the two 128-row slabs of W
constexpr int OFF_TINV = OFF_W, OFF_DSL = OFF_W + 2 * T64, OFF_PRB = OFF_W + 3 * T64;
constexpr int OFF_WY = OFF_W, OFF_WSA = OFF_W + T128;
constexpr int OFF_X1 = OFF_W + 4 * T64;     // P_rk (adjacent to P_rb), then Gd, then S0
constexpr int OFF_X2 = OFF_X1 + T64;        // 8 KB used only by the last epilogue
constexpr int OFF_SMALL = OFF_X2 + T64;
// transient tenants
constexpr int OFF_STG = OFF_AR;             // 7 raw tiles (w r k v a b dy) of 64 rows x 128 bytes, 128-byte swizzle
constexpr int OFF_CUMF = OFF_W;             // fp32 cumulative log2-decay while it is scanned (16 KB, swizzled rows)
constexpr int OFF_LF = OFF_W;               // last epilogue: fp32 r dr - k dk per token, then D_{t-1} (16 KB, swizzled rows)
constexpr int OFF_P3 = OFF_W + T128;        // last epilogue: fp32 a da (16 KB, swizzled rows)
constexpr int OFF_UB = OFF_X1;              // last epilogue: fp32 a da - b db (16 KB over X1 | X2, swizzled rows)
// Gradient tiles on their way out: [64 tokens][128 bytes] with the 128-byte swizzle of the tiled copies (piece index
// XOR token mod 8).  dk, db, dr, da are written by the last epilogue over [V ; sa] and [dY ; dG], whose products are
// done, and must have been read before the next block's staging tiles 4..6 land on them; dv, and at the very end of
// the block the decay gradient, use the 8 KB that only the last epilogue's fp32 buffer shares.
constexpr int OFF_TK = OFF_VSA, OFF_TB = OFF_VSA + T64, OFF_TR = OFF_DD, OFF_TA = OFF_DD + T64;
constexpr int OFF_TV = OFF_X2;
struct Small {
    uint64_t bar[8];     // 0..3 product rounds, 4 staging, 5 P_rb|P_rk|sa, 6 T|A_ak, 7 S0
    uint32_t tmem;
    uint32_t pad[3];
    float lam[kN];       // 2^(block total)
    float d_end[kN];     // D at the block end
    float seg_tail[kN];  // with lam and d_end (both dead by then): per-16-token totals of the decay-gradient scan, [3][64]
};
constexpr int SMEM_BYTES = OFF_SMALL + 1024;
static_assert(sizeof(Small) <= 1024, "small state must fit its kilobyte");
static_assert(2 * (SMEM_BYTES + 1024) <= 228 * 1024, "two CTAs per SM");
static_assert(7 * T64 <= 4 * T128, "staging tiles must fit over the four operand slabs");

// factor tiles in the per-CTA global scratch, each in the slab layout [column block][token][8 channels] of bf16
constexpr int F_INV = 0, F_L = 1, F_LPREV = 2, F_LOGW = 3;   // 1/L_t, L_t, L_{t-1}, ln(decay_t)

// TMEM columns (256 allocated)
constexpr uint32_t T_W = 0;       // 128: W ; afterwards [dR~' ; dA~'] in its first 64
constexpr uint32_t T_RA = 0;
constexpr uint32_t T_GD = 128;    // 64 : [Gd ; dV]
constexpr uint32_t T_X = 192;     // 64 : dG, afterwards [dK~' ; dB~']
constexpr uint32_t T_KB = 192;

__device__ __forceinline__ void mma_k64(uint32_t d, Op a, Op b, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) tc::mma(d, op_desc(a, ks), op_desc(b, ks), idesc, accumulate || ks > 0);
}
// operand walks over unpadded slabs
__device__ __forceinline__ Op kmaj128u(uint32_t a) { return make_op(a, 2 * P128, P128, 128); }
__device__ __forceinline__ Op kmaj64u(uint32_t a) { return make_op(a, 2 * P64, P64, 128); }
__device__ __forceinline__ Op mnmaj128u(uint32_t a) { return make_op(a, 256, 128, P128); }
__device__ __forceinline__ Op mnmaj64u(uint32_t a) { return make_op(a, 256, 128, P64); }

// fp32 [64][64] buffers whose rows are read by lanes that own consecutive rows (float4) and by lanes that own
// consecutive columns (scalar): the float4 index inside a row is XORed with the row's low bits
__device__ __forceinline__ int swz4(int row, int c4) { return row * 64 + ((c4 ^ (row & 7)) << 2); }
__device__ __forceinline__ int swz1(int row, int c) { return row * 64 + ((((c >> 2) ^ (row & 7)) << 2) | (c & 3)); }

// eight bf16 values times eight bf16 factors, as four packed products
__device__ __forceinline__ uint4 mul8(uint4 a, uint4 b) {
    const __nv_bfloat162* x = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* y = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 out;
    uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __hmul2(x[i], y[i]);
        o[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return out;
}

__global__ void __launch_bounds__(256, 2)
wkv7_grad_bwd_kernel(int Tlen, int H, int BH, const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                     const __nv_bfloat16* __restrict__ ds_state, const float* __restrict__ s_at_len,
                     const unsigned char* __restrict__ saved, const int* __restrict__ fast, const int* __restrict__ residual_mark,
                     __nv_bfloat16* __restrict__ dw, __nv_bfloat16* __restrict__ dr, __nv_bfloat16* __restrict__ dk,
                     __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ da, __nv_bfloat16* __restrict__ db,
                     int* __restrict__ status, int has_dy, unsigned char* __restrict__ fscr_all,
                     const __grid_constant__ StreamMaps maps, const __grid_constant__ StreamMaps out_maps) {
    if (*residual_mark != 0) return;            // the forward fell back to the sequential kernels
    extern __shared__ __align__(1024) unsigned char smem[];
    Small& sm = *reinterpret_cast<Small*>(smem + OFF_SMALL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hsel = warp >> 2;     // TMEM lane quadrant / column half handled by this warp
    const int row = quad * 32 + lane;                // TMEM lane == tile row
    const int nBlk = Tlen / kC;
    const int n_items = BH * nBlk;   // (the launcher refuses shapes whose block count overflows an int)
    unsigned char* const fscr = fscr_all + (size_t)blockIdx.x * 4 * GTILE;
    // the 128-byte swizzle of the staging tiles is a function of the shared-memory address
    if ((tc::smem_u32(smem) & 1023u) != 0) {
        if (tid == 0 && status != nullptr) atomicExch(status, 4);
        return;
    }
    // next item of the flat (sequence, block) list that belongs to a sequence this kernel handles
    auto next_item = [&](int it) {
        while (it < n_items && fast[it / nBlk] == 0) it += (int)gridDim.x;
        return it;
    };
    int item = next_item((int)blockIdx.x);
    if (item >= n_items) return;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) tc::mbar_init(&sm.bar[i], (i == 2 || i == 3) ? 2 : 1);   // rounds 3, 4 have two issuing threads
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(&sm.tmem, 256);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tbase = sm.tmem;
    const uint32_t lane_addr = tbase + ((uint32_t)(quad * 32) << 16);
    bool failed = false;

    const uint32_t sAR = tc::smem_u32(smem + OFF_AR), sBK = tc::smem_u32(smem + OFF_BK);
    const uint32_t sVSA = tc::smem_u32(smem + OFF_VSA), sDD = tc::smem_u32(smem + OFF_DD);
    const uint32_t sDSL = tc::smem_u32(smem + OFF_DSL), sTINV = tc::smem_u32(smem + OFF_TINV);
    const uint32_t sPRB = tc::smem_u32(smem + OFF_PRB), sX1 = tc::smem_u32(smem + OFF_X1);
    const uint32_t sWY = tc::smem_u32(smem + OFF_WY), sWSA = tc::smem_u32(smem + OFF_WSA);
    constexpr uint32_t ID_N128_KK = tc::make_idesc(128, 128, false, false);
    constexpr uint32_t ID_KK = tc::make_idesc(128, 64, false, false);
    constexpr uint32_t ID_KM = tc::make_idesc(128, 64, false, true);
    constexpr uint32_t ID_MM = tc::make_idesc(128, 64, true, true);
    constexpr uint32_t HALF = 64 * 16;   // byte offset of row 64 inside a column block of a 128-row slab
    const bool issuer_a = (tid == 64), issuer_b = (tid == 192);
    constexpr int kStageThread = 96, kSavedWarp = 7;

    float* cumf = reinterpret_cast<float*>(smem + OFF_CUMF);
    float* lf = reinterpret_cast<float*>(smem + OFF_LF);
    float* p3buf = reinterpret_cast<float*>(smem + OFF_P3);
    float* ubuf = reinterpret_cast<float*>(smem + OFF_UB);
    float* seg = sm.lam;   // [3][64]: totals of segments 1..3 (see Small)
    enum { OUT_W = 0, OUT_R = 1, OUT_K = 2, OUT_V = 3, OUT_A = 4, OUT_B = 5 };   // tensor maps of the gradients
    uint32_t par = 0;   // every barrier completes one phase per block

    // scaling role: one token, two column blocks (16 channels)
    const int st_t = (warp & 1) * 32 + lane, st_jb = (warp >> 1) * 2;
    // state role: one row, two column blocks
    const int si = tid & 63, sc = (tid >> 6) * 2;

    const int n_streams = has_dy ? 7 : 6;
    // raw tiles m_from..m_to-1 of block `it` (thread kStageThread; the first call of a block announces all of them)
    auto issue_stage = [&](int it, int m_from, int m_to) {
        if (tid == kStageThread) {
            const int bh_ = it / nBlk, blk_ = it % nBlk;
            if (m_from == 0) tc::mbar_expect_tx(&sm.bar[4], (uint32_t)(n_streams * T64));
            const int x = (bh_ % H) * kN, y = (bh_ / H) * Tlen + blk_ * kC;
#pragma unroll
            for (int m = 0; m < 7; ++m)
                if (m >= m_from && m < m_to && m < n_streams) tc::tensor_load_2d(smem + OFF_STG + m * T64, &maps.m[m], x, y, &sm.bar[4]);
        }
    };
    tc::fence_async_smem();
    issue_stage(item, 0, 7);
    bool pend_dw = false;    // the decay-gradient tile of the previous block waits for a CTA barrier
    int pend_x = 0, pend_y = 0;
    // what the loop needs to know about a block before it touches it, fetched one block ahead
    int meta_L = min((int)length[(item / nBlk) / H], Tlen);
    bool meta_reset = new_starts[(size_t)((item / nBlk) / H) * Tlen + (item % nBlk) * kC] != 0;

    while (item < n_items) {
        const int bh = item / nBlk, blk = item % nBlk, bi = bh / H;
        const int L = meta_L;
        const bool reset_here = meta_reset;
        const int p = blk * kC, p1 = p + kC;
        const size_t st_base = (size_t)bh * kN * kN;
        const unsigned char* tiles = saved + ((size_t)bh * nBlk + blk) * kSavedBytes;
        const __nv_bfloat16* dsg = ds_state + ((size_t)bh * nBlk + blk) * kN * kN;

        // the state gradient leaving this block (global memory) is asked for before anything waits
        const uint4 ds_raw0 = *reinterpret_cast<const uint4*>(dsg + sc * (kN * 8) + si * 8);         // column block sc, row si
        const uint4 ds_raw1 = *reinterpret_cast<const uint4*>(dsg + (sc + 1) * (kN * 8) + si * 8);
        // ================= raw rows out of the staging tiles (registers) =================
        uint4 raw[7][2];   // w r k v a b dy ; column blocks st_jb, st_jb + 1
        if (!tc::mbar_wait(&sm.bar[4], par)) failed = true;
#pragma unroll
        for (int m = 0; m < 7; ++m)
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
                raw[m][h2] = (m < n_streams) ? *reinterpret_cast<const uint4*>(smem + OFF_STG + m * T64 + st_t * 128 + (((st_jb + h2) ^ (st_t & 7)) << 4))
                                             : make_uint4(0, 0, 0, 0);
        tc::fence_async_smem();
        __syncthreads();   // the staging tiles are empty; the previous block's last epilogue has finished everywhere
        if (issuer_b && pend_dw) {
            tc::tensor_store_2d(&out_maps.m[OUT_W], pend_x, pend_y, smem + OFF_TV);
            tc::bulk_commit();
        }
        // P_rb | P_rk and sa of this block (their hosts are free now); T | A_ak follow once the scan buffer is done with
        if (warp == kSavedWarp) {
            if (lane == 0) tc::mbar_expect_tx(&sm.bar[5], (uint32_t)(3 * T64));
            __syncwarp();
            if (lane == 8) tc::bulk_load(smem + OFF_PRB, tiles + SAVED_PRB * GTILE, 2 * GTILE, &sm.bar[5]);
            if (lane < 8) tc::bulk_load(smem + OFF_VSA + lane * P128 + HALF, tiles + SAVED_SA * GTILE + lane * GCB, 64 * 16, &sm.bar[5]);
        }
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            slab_store(smem + OFF_VSA, P128, st_t, st_jb + h2, raw[3][h2]);
            slab_store(smem + OFF_DD, P128, st_t, st_jb + h2, raw[6][h2]);
        }
        // ================= cumulative decay of the block =================
        float lw[16];   // log2 of the decay: -exp(w) * log2(e)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
            float wf[8];
            unpack8(raw[0][h2], wf);
#pragma unroll
            for (int e = 0; e < 8; ++e) lw[h2 * 8 + e] = -kLog2e * __expf(wf[e]);
        }
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4)
            *reinterpret_cast<float4*>(&cumf[swz4(st_t, st_jb * 2 + c4)]) = make_float4(lw[c4 * 4], lw[c4 * 4 + 1], lw[c4 * 4 + 2], lw[c4 * 4 + 3]);
        __syncthreads();
        if (tid < 128) {   // inclusive scan over tokens, two independent halves of 32 per channel; all loads first
            const int j = tid & 63, half = tid >> 6;
            float vv[32];
#pragma unroll
            for (int tt = 0; tt < 32; ++tt) vv[tt] = cumf[swz1(half * 32 + tt, j)];
#pragma unroll
            for (int tt = 1; tt < 32; ++tt) vv[tt] += vv[tt - 1];
#pragma unroll
            for (int tt = 0; tt < 32; ++tt) cumf[swz1(half * 32 + tt, j)] = vv[tt];
        }
        __syncthreads();
        // (the halves' totals are rows 31 and 63 of the scanned buffer)
        if (tid < 64) sm.lam[tid] = ex2(fmaxf(cumf[swz1(31, tid)] + cumf[swz1(63, tid)], kCumFloor));
        // ================= scaled operands into the slabs; the decay factors to this CTA's scratch =================
        {
            float cc[16];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
                const float4 x4 = *reinterpret_cast<const float4*>(&cumf[swz4(st_t, st_jb * 2 + c4)]);
                cc[c4 * 4] = x4.x; cc[c4 * 4 + 1] = x4.y; cc[c4 * 4 + 2] = x4.z; cc[c4 * 4 + 3] = x4.w;
            }
            if (st_t >= 32) {   // second half: on top of the first half's total
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    const float4 h4 = *reinterpret_cast<const float4*>(&cumf[swz4(31, st_jb * 2 + c4)]);
                    cc[c4 * 4] += h4.x; cc[c4 * 4 + 1] += h4.y; cc[c4 * 4 + 2] += h4.z; cc[c4 * 4 + 3] += h4.w;
                }
            }
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                float eL[8], eI[8], eP[8], lg[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float c = fmaxf(cc[h2 * 8 + e], kCumFloor);
                    const float cp = fminf(c - lw[h2 * 8 + e], 0.f);   // cumulative log2-decay before this token
                    eL[e] = ex2(c); eI[e] = ex2(-c); eP[e] = ex2(cp);
                    lg[e] = kLn2 * lw[h2 * 8 + e];
                }
                const int jb = st_jb + h2;
                const uint4 pI = pack8(eI), pL = pack8(eL), pP = pack8(eP);
                slab_store(smem + OFF_AR, P128, st_t, jb, mul8(raw[4][h2], pP));
                slab_store(smem + OFF_AR, P128, 64 + st_t, jb, mul8(raw[1][h2], pL));
                slab_store(smem + OFF_BK, P128, st_t, jb, mul8(raw[5][h2], pI));
                slab_store(smem + OFF_BK, P128, 64 + st_t, jb, mul8(raw[2][h2], pI));
                unsigned char* f = fscr + jb * GCB + st_t * 16;
                *reinterpret_cast<uint4*>(f + F_INV * GTILE) = pI;
                *reinterpret_cast<uint4*>(f + F_L * GTILE) = pL;
                *reinterpret_cast<uint4*>(f + F_LPREV * GTILE) = pP;
                *reinterpret_cast<uint4*>(f + F_LOGW * GTILE) = pack8(lg);
            }
        }
        __syncthreads();   // lam is set
        // ================= dS diag(L_C) in bf16 =================
        {
            float g[8];
            unpack8(ds_raw0, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] *= sm.lam[sc * 8 + e];
            slab_store(smem + OFF_DSL, P64, si, sc, pack8(g));
            unpack8(ds_raw1, g);
#pragma unroll
            for (int e = 0; e < 8; ++e) g[e] *= sm.lam[(sc + 1) * 8 + e];
            slab_store(smem + OFF_DSL, P64, si, sc + 1, pack8(g));
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (warp == kSavedWarp && lane == 0) {   // the scan buffer over T | A_ak is dead
            tc::mbar_expect_tx(&sm.bar[6], (uint32_t)(2 * T64));
            tc::bulk_load(smem + OFF_TINV, tiles + SAVED_T * GTILE, 2 * GTILE, &sm.bar[6]);
        }
        // ================= R2: [Gd ; dVpart] = [B~;K~] dSL^T + [P_rb|P_rk]^T dY =================
        if (issuer_a) {
            tc::fence_after_sync();
            mma_k64(tbase + T_GD, kmaj128u(sBK), kmaj64u(sDSL), ID_KK, false);
            if (!tc::mbar_wait(&sm.bar[5], par)) failed = true;   // P_rb | P_rk (and sa) have landed
            mma_k64(tbase + T_GD, mnmaj64u(sPRB), mnmaj128u(sDD), ID_MM, true);
            tc::commit(&sm.bar[0]);
        }
        if (quad >= 2) {
            // D at the block end, by the four warps that have no part in the next two epilogues:
            //   D_end[c] = sum_i dS[i][c] S_end[i][c] = (sum_i dSL[i][c] S_end[i][c]) / L_C[c]
            // with dSL read from its slab.  S_end is the state at `length` when the block ends there, else the
            // entering state the forward saved for the next block (zero behind a start flag, where dS is too).
            // Thread (column block cbk, row group ig) adds rows ig, ig + 16, ...; the sixteen row groups of a column
            // block sit in one half of a warp and meet in a butterfly of fixed order.
            const int a_tid = ((quad - 2) * 2 + hsel) * 32 + lane, cbk = a_tid >> 4, ig = a_tid & 15;
            float acc[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = 0.f;
            if (p1 == L || blk + 1 < nBlk) {
                const bool at_len = (p1 == L);
                const float* sf = s_at_len + st_base + cbk * 8;
                const unsigned char* sb = tiles + kSavedBytes + SAVED_S0 * GTILE + cbk * GCB;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    const int i = ig + 16 * m;
                    float se[8], dsl[8];
                    if (at_len) {
                        const float4 s0 = __ldg(reinterpret_cast<const float4*>(sf + i * kN)), s1 = __ldg(reinterpret_cast<const float4*>(sf + i * kN + 4));
                        se[0] = s0.x; se[1] = s0.y; se[2] = s0.z; se[3] = s0.w; se[4] = s1.x; se[5] = s1.y; se[6] = s1.z; se[7] = s1.w;
                    } else {
                        unpack8(__ldg(reinterpret_cast<const uint4*>(sb + i * 16)), se);
                    }
                    unpack8(*reinterpret_cast<const uint4*>(smem + OFF_DSL + cbk * P64 + i * 16), dsl);
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[e] = fmaf(dsl[e], se[e], acc[e]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 4);
                acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 8);
            }
            if (ig == 0) {
#pragma unroll
                for (int e = 0; e < 8; ++e) sm.d_end[cbk * 8 + e] = acc[e] / sm.lam[cbk * 8 + e];
            }
        }
        if (quad < 2) {
            if (!tc::mbar_wait(&sm.bar[0], par)) failed = true;
            tc::fence_after_sync();
            float gd[32];
            tc::tmem_ld32(lane_addr + T_GD + hsel * 32, gd);
            tc::tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) slab_store(smem + OFF_X1, P64, row, hsel * 4 + c, pack8(&gd[c * 8]));   // over P_rk, which is read
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        // ================= R3: dG = T^T Gd =================
        if (issuer_a) {
            tc::fence_after_sync();
            if (!tc::mbar_wait(&sm.bar[6], par)) failed = true;   // T | A_ak have landed
            mma_k64(tbase + T_X, mnmaj64u(sTINV), mnmaj64u(sX1), ID_MM, false);
            tc::commit(&sm.bar[1]);
        }
        if (quad < 2) {
            if (!tc::mbar_wait(&sm.bar[1], par)) failed = true;
            tc::fence_after_sync();
            float z[32];
            tc::tmem_ld32(lane_addr + T_X + hsel * 32, z);
            tc::tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) slab_store(smem + OFF_DD, P128, 64 + row, hsel * 4 + c, pack8(&z[c * 8]));
        }
        if (issuer_b) tc::bulk_wait_read<0>();   // the previous block's decay-gradient tile has left: dV takes its place
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (warp == kSavedWarp && lane == 0) {   // Gd is read: the entering state takes its place (needed in the last round)
            tc::mbar_expect_tx(&sm.bar[7], (uint32_t)T64);
            tc::bulk_load(smem + OFF_X1, tiles + SAVED_S0 * GTILE, GTILE, &sm.bar[7]);
        }
        // ================= R4: W = [V;sa][dY;dG]^T ; dV += A_ak^T dG ; [dK~';dB~'] = [V;sa] dSL =================
        if (issuer_a) {
            tc::fence_after_sync();
            mma_k64(tbase + T_W, kmaj128u(sVSA), kmaj128u(sDD), ID_N128_KK, false);
            mma_k64(tbase + T_GD, mnmaj64u(sTINV), mnmaj128u(sDD + HALF), ID_MM, true);
            tc::commit(&sm.bar[2]);
        } else if (issuer_b) {
            tc::fence_after_sync();
            mma_k64(tbase + T_KB, kmaj128u(sVSA), mnmaj64u(sDSL), ID_KM, false);
            tc::commit(&sm.bar[2]);
        }
        // the next block of this CTA, and what the loop needs to know about it
        const int item_next = next_item(item + (int)gridDim.x);
        if (item_next < n_items) {
            const int bi_n = (item_next / nBlk) / H;
            meta_L = min((int)length[bi_n], Tlen);
            meta_reset = new_starts[(size_t)bi_n * Tlen + (item_next % nBlk) * kC] != 0;
        }
        if (!tc::mbar_wait(&sm.bar[2], par)) failed = true;
        tc::fence_after_sync();
        {
            // keep s >= t for the dY blocks, s > t for the dG blocks.  Rows t < 32 keep all of columns 32..63;
            // rows t >= 32 keep nothing of columns 0..31 (zeros are stored without reading the accumulator).
            const int t = row & 63, lo = t + hsel;
            unsigned char* dst = smem + (hsel == 0 ? OFF_WY : OFF_WSA);   // over T, A_ak, dSL, P_rb: all read by now
            float d[32];
            if ((quad & 1) == 0) {
                tc::tmem_ld32(lane_addr + T_W + hsel * 64, d);
                tc::tmem_wait_ld();
#pragma unroll
                for (int s = 0; s < 32; ++s) d[s] = (s >= lo) ? d[s] : 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(dst, P128, row, c, pack8(&d[c * 8]));
                tc::tmem_ld32(lane_addr + T_W + hsel * 64 + 32, d);
                tc::tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(dst, P128, row, 4 + c, pack8(&d[c * 8]));
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(dst, P128, row, c, make_uint4(0, 0, 0, 0));
                tc::tmem_ld32(lane_addr + T_W + hsel * 64 + 32, d);
                tc::tmem_wait_ld();
#pragma unroll
                for (int s = 0; s < 32; ++s) d[s] = (s + 32 >= lo) ? d[s] : 0.f;
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(dst, P128, row, 4 + c, pack8(&d[c * 8]));
            }
        }
        if (quad >= 2) {   // dV rows
            const int t = row - 64;
            float x[32];
            tc::tmem_ld32(lane_addr + T_GD + hsel * 32, x);
            tc::tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(smem + OFF_TV + t * 128 + (((hsel * 4 + c) ^ (t & 7)) << 4)) = pack8(&x[c * 8]);
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        // ================= R5: [dK~';dB~'] += W . [A~;R~] ; [dR~';dA~'] = [dY;dG] S0 + W^T . [B~;K~] =================
        if (issuer_a) {
            tc::fence_after_sync();
            mma_k64(tbase + T_KB, kmaj128u(sWSA), mnmaj128u(sAR), ID_KM, true);
            mma_k64(tbase + T_KB, kmaj128u(sWY), mnmaj128u(sAR + HALF), ID_KM, true);
            tc::commit(&sm.bar[3]);
        } else if (issuer_b) {
            tc::fence_after_sync();
            tc::tensor_store_2d(&out_maps.m[OUT_V], (bh % H) * kN, bi * Tlen + p, smem + OFF_TV);
            tc::bulk_commit();
            mma_k64(tbase + T_RA, mnmaj128u(sWY + HALF), mnmaj128u(sBK), ID_MM, false);
            mma_k64(tbase + T_RA, mnmaj128u(sWY), mnmaj128u(sBK + HALF), ID_MM, true);
            if (!tc::mbar_wait(&sm.bar[7], par)) failed = true;   // S0 has landed
            mma_k64(tbase + T_RA, kmaj128u(sDD), mnmaj64u(sX1), ID_KM, true);
            tc::bulk_wait_read<0>();   // the dV tile has left before this round is reported done: the last epilogue writes over it
            tc::commit(&sm.bar[3]);
        }
        // ---- while the products run: this row's decay factors from the scratch
        const int t = row & 63;
        uint4 fxr[4], fzr[4];   // 1 / L_t ; L_t (rows 0..63: dr) or L_{t-1} (rows 64..127: da), 32 channels each
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const unsigned char* f = fscr + (hsel * 4 + c) * GCB + t * 16;
            fxr[c] = *reinterpret_cast<const uint4*>(f + F_INV * GTILE);
            fzr[c] = *reinterpret_cast<const uint4*>(f + (row < 64 ? F_L : F_LPREV) * GTILE);
        }
        if (!tc::mbar_wait(&sm.bar[3], par)) failed = true;
        tc::fence_after_sync();
        // ================= last epilogue: unscale, write dk db dr da, decay gradient =================
        unsigned char* const tile_x = smem + ((row < 64) ? OFF_TK : OFF_TB) + t * 128;   // dk | db
        unsigned char* const tile_z = smem + ((row < 64) ? OFF_TR : OFF_TA) + t * 128;   // dr | da
        float* const ubase = (row < 64) ? lf : ubuf;   // r dr - k dk of the token | a da - b db of the token
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float x[16], z[16];
            tc::tmem_ld16(lane_addr + T_KB + hsel * 32 + hh * 16, x);
            tc::tmem_ld16(lane_addr + T_RA + hsel * 32 + hh * 16, z);
            tc::tmem_wait_ld();
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
                const int c = hh * 2 + h2, cb = hsel * 4 + c;
                float s1[8], s2[8], u[8], pz[8];   // R~ / A~ and K~ / B~ of this row
                unpack8(*reinterpret_cast<const uint4*>(smem + OFF_AR + cb * P128 + ((row < 64) ? (64 + t) : t) * 16), s1);
                unpack8(*reinterpret_cast<const uint4*>(smem + OFF_BK + cb * P128 + ((row < 64) ? (64 + t) : t) * 16), s2);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    pz[e] = s1[e] * z[h2 * 8 + e];
                    u[e] = pz[e] - s2[e] * x[h2 * 8 + e];       // rows 0..63: r dr - k dk ; rows 64..127: a da - b db
                }
                *reinterpret_cast<float4*>(&ubase[swz4(t, cb * 2)]) = make_float4(u[0], u[1], u[2], u[3]);
                *reinterpret_cast<float4*>(&ubase[swz4(t, cb * 2 + 1)]) = make_float4(u[4], u[5], u[6], u[7]);
                if (row >= 64) {   // a da, for the decay gradient
                    *reinterpret_cast<float4*>(&p3buf[swz4(t, cb * 2)]) = make_float4(pz[0], pz[1], pz[2], pz[3]);
                    *reinterpret_cast<float4*>(&p3buf[swz4(t, cb * 2 + 1)]) = make_float4(pz[4], pz[5], pz[6], pz[7]);
                }
                const int piece = ((cb ^ (t & 7)) << 4);
                *reinterpret_cast<uint4*>(tile_x + piece) = mul8(pack8(&x[h2 * 8]), fxr[c]);
                *reinterpret_cast<uint4*>(tile_z + piece) = mul8(pack8(&z[h2 * 8]), fzr[c]);
            }
        }
        // log-decay of this token (rows 64..127 write the decay gradient): asked for ahead of the scan
        uint4 lgr[4];
        if (row >= 64) {
#pragma unroll
            for (int c = 0; c < 4; ++c) lgr[c] = *reinterpret_cast<const uint4*>(fscr + F_LOGW * GTILE + (hsel * 4 + c) * GCB + t * 16);
        }
        const float d_end_c = sm.d_end[tid & 63];   // (its storage serves the scan below)
        tc::fence_async_smem();   // the gradient tiles are read by bulk copies
        tc::fence_before_sync();
        __syncthreads();   // every operand slab has been read for the last time: the next block's rows may arrive
        if (tid == kStageThread) {
            const int x = (bh % H) * kN, y = bi * Tlen + p;
            tc::tensor_store_2d(&out_maps.m[OUT_K], x, y, smem + OFF_TK);
            tc::tensor_store_2d(&out_maps.m[OUT_B], x, y, smem + OFF_TB);
            tc::tensor_store_2d(&out_maps.m[OUT_R], x, y, smem + OFF_TR);
            tc::tensor_store_2d(&out_maps.m[OUT_A], x, y, smem + OFF_TA);
            tc::bulk_commit();
        }
        if (item_next < n_items) issue_stage(item_next, 0, 4);   // tiles 0..3 land on [A~;R~], [B~;K~]
        if (tid == kStageThread) tc::bulk_wait_read<0>();        // tiles 4..6 on the gradient tiles, once those are read
        if (item_next < n_items) issue_stage(item_next, 4, 7);
        {   // D_{t-1} = D_t + u_t from D at the block end: suffix sums over 4 segments of 16 tokens, all loads first
            const int c = tid & 63, sg = tid >> 6;
            float vv[16];
#pragma unroll
            for (int tt = 0; tt < 16; ++tt) vv[tt] = lf[swz1(sg * 16 + tt, c)] + ubuf[swz1(sg * 16 + tt, c)];
#pragma unroll
            for (int tt = 14; tt >= 0; --tt) vv[tt] += vv[tt + 1];
            if (sg > 0) seg[(sg - 1) * 64 + c] = vv[0];
            __syncthreads();
            float off = d_end_c;
            for (int s2 = 3; s2 > sg; --s2) off += seg[(s2 - 1) * 64 + c];
#pragma unroll
            for (int tt = 0; tt < 16; ++tt) lf[swz1(sg * 16 + tt, c)] = vv[tt] + off;
        }
        __syncthreads();
        if (row >= 64) {
            float o[32];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int cb = hsel * 4 + c;
                const float4 d0 = *reinterpret_cast<const float4*>(&lf[swz4(t, cb * 2)]), d1 = *reinterpret_cast<const float4*>(&lf[swz4(t, cb * 2 + 1)]);
                const float4 q0 = *reinterpret_cast<const float4*>(&p3buf[swz4(t, cb * 2)]), q1 = *reinterpret_cast<const float4*>(&p3buf[swz4(t, cb * 2 + 1)]);
                float lg[8];
                unpack8(lgr[c], lg);
                o[c * 8 + 0] = (d0.x - q0.x) * lg[0]; o[c * 8 + 1] = (d0.y - q0.y) * lg[1];
                o[c * 8 + 2] = (d0.z - q0.z) * lg[2]; o[c * 8 + 3] = (d0.w - q0.w) * lg[3];
                o[c * 8 + 4] = (d1.x - q1.x) * lg[4]; o[c * 8 + 5] = (d1.y - q1.y) * lg[5];
                o[c * 8 + 6] = (d1.z - q1.z) * lg[6]; o[c * 8 + 7] = (d1.w - q1.w) * lg[7];
            }
            if (reset_here && t == 0) {   // the state entering a start token is zero: no decay gradient
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = 0.f;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4*>(smem + OFF_TV + t * 128 + (((hsel * 4 + c) ^ (t & 7)) << 4)) = pack8(&o[c * 8]);
        }
        pend_dw = true;
        pend_x = (bh % H) * kN;
        pend_y = bi * Tlen + p;
        tc::fence_async_smem();   // the scan buffers are rewritten by bulk copies early in the next block; the tile is read by one
        tc::fence_before_sync();
        par ^= 1u;
        item = item_next;
    }
    if (failed && status != nullptr) atomicExch(status, 2);
    tc::fence_before_sync();
    __syncthreads();
    if (issuer_b) {
        if (pend_dw) {
            tc::tensor_store_2d(&out_maps.m[OUT_W], pend_x, pend_y, smem + OFF_TV);
            tc::bulk_commit();
        }
        tc::bulk_wait_all<0>();   // shared memory stays this CTA's until every tile has been read
    }
    if (tid == kStageThread) tc::bulk_wait_all<0>();
    if (warp == 0) tc::tmem_dealloc(tbase, 256);
}

}  // namespace

int* wkv7_chunk_status_word();

int wkv7_grad_bwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                  const void* a, const void* b, const uint32_t* length, const uint8_t* ns, const void* dy, void* residual,
                  const int* residual_mark, void* dw, void* dr, void* dk, void* dv, void* da, void* db) {
    typedef __nv_bfloat16 bf;
    static DeviceOnce smem_attr;
    if (!smem_attr.ok([]() { return cudaFuncSetAttribute(wkv7_grad_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); }))
        return B200WKV_ELAUNCH;
    const CarryLayout lay = carry_layout(B, T, H);
    char* base = static_cast<char*>(residual);
    const int nBlk = T / kC, BH = B * H;
    const float* s_at_len = (const float*)residual + (size_t)BH * nBlk * kN * kN;
    const unsigned char* saved = reinterpret_cast<const unsigned char*>((const float*)residual + chunk_saved_offset_floats(B, T, H));
    StreamMaps maps;
    const void* bases[7] = {w, r, k, v, a, b, dy};
    if (!make_stream_maps(&maps, bases, dy != nullptr ? 7 : 6, B, T, H, /*swizzle128=*/true)) return B200WKV_ELAUNCH;
    StreamMaps out_maps;
    const void* out_bases[6] = {dw, dr, dk, dv, da, db};
    if (!make_stream_maps(&out_maps, out_bases, 6, B, T, H, /*swizzle128=*/true)) return B200WKV_ELAUNCH;
    const long long items = (long long)BH * nBlk;
    if (items > 2147483647LL) return B200WKV_ESHAPE;
    long long slots = 2LL * sm_count_of_current_device();
    if (slots > kGradCtas) slots = kGradCtas;        // every CTA owns a set of factor tiles in the residual
    const int grid = (int)(items < slots ? items : slots);
    wkv7_grad_bwd_kernel<<<grid, 256, SMEM_BYTES, st>>>(T, H, BH, length, ns, (const bf*)(base + lay.dstate), s_at_len, saved,
                                                        (const int*)(base + lay.fast), residual_mark, (bf*)dw, (bf*)dr, (bf*)dk,
                                                        (bf*)dv, (bf*)da, (bf*)db, wkv7_chunk_status_word(), dy != nullptr ? 1 : 0,
                                                        (unsigned char*)(base + lay.fscr), maps, out_maps);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace b200wkv

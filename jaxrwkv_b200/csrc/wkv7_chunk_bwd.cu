// RWKV-7 WKV backward, chunked along T on the Blackwell tensor cores (bf16 I/O, fp32 carries).
//
// One persistent CTA (256 threads) per SM walks sequences, or runs of blocks of sequences, in reverse
// (see RunPlan in chunk_common.cuh).  A chunk is re-entered from the forward's saved state S0; its
// forward quantities (the four triangular Gram blocks, T = (I - A_ab)^-1, sa) are copied in from the
// residual when the forward walked the block as one full chunk, and recomputed otherwise; the scaled
// operands are always rebuilt from the raw rows, which arrive by tiled bulk copies one chunk ahead.
// Then with dS = gradient of the state leaving
// the chunk, L = in-chunk cumulative decay (L_C at the chunk end) and dSL = dS diag(L_C):
//   dsa   = T^T (B~ dSL^T + P_rb^T dY)                           row t is dS_t b_t
//   dV    = K~ dSL^T + P_rk^T dY + A_ak^T dsa
//   W     = [V; sa] [dY; dsa]^T                                  upper-triangular Gram blocks
//   dK~'  = W_v,dsa A~ + W_v,dy R~ + V  dSL      dk = dK~' / L_t
//   dB~'  = W_sa,dsa A~ + W_sa,dy R~ + sa dSL    db = dB~' / L_t
//   dR~'  = dY  S0 + W_sa,dy^T B~ + W_v,dy^T K~  dr = dR~' * L_t
//   dA~'  = dsa S0 + W_sa,dsa^T B~ + W_v,dsa^T K~  da = dA~' * L_{t-1}
//   dS0   = dSL + dsa^T A~ + dY^T R~                             carried to the previous chunk
// The decay gradient uses D_t = sum_i dS_t[i,:] S_t[i,:]:  with u_t = r dr - b db - k dk + a da the
// recurrence D_{t-1} = D_t + u_t holds, d(log decay)_t = D_{t-1} - a_t da_t, and D is re-anchored
// exactly at every chunk start from dS0 and S0, so rounding never accumulates across chunks.
// All products are tcgen05.mma (M=128, bf16 operands in shared memory, fp32 accumulators in TMEM).
//
// Semantics: reverse-mode derivative of BaseRWKV.inner_loop of jaxrwkv (src/jaxrwkv/rwkv7.py:199-220).
#include "common.cuh"
#include "tc05.cuh"
#include "chunk_common.cuh"
#include "tmap.cuh"

namespace b200wkv {

namespace {

// shared-memory map (bytes); one CTA per SM
constexpr int OFF_AR = 0;                         // [A~ ; R~]          128-row slab
constexpr int OFF_BK = OFF_AR + SLAB128;          // [B~ ; K~]          128-row slab
constexpr int OFF_VSA = OFF_BK + SLAB128;         // [V ; sa]           128-row slab
constexpr int OFF_DD = OFF_VSA + SLAB128;         // [dY ; dsa]         128-row slab
constexpr int OFF_S0 = OFF_DD + SLAB128;          // S0 bf16 [i][j]     64-row slab
constexpr int OFF_DSL = OFF_S0 + SLAB64;          // dS diag(L_C) bf16  64-row slab
constexpr int OFF_TINV = OFF_DSL + SLAB64;        // T                  64-row slab  } adjacent
constexpr int OFF_AAK = OFF_TINV + SLAB64;        // A_ak               64-row slab  }
constexpr int OFF_X = OFF_AAK + SLAB64;           // P_rb | P_rk | G | Gd  (4 x 64-row slabs), later W
constexpr int OFF_PRB = OFF_X;
constexpr int OFF_PRK = OFF_PRB + SLAB64;
constexpr int OFF_G = OFF_PRK + SLAB64;
constexpr int OFF_GD = OFF_G + SLAB64;
constexpr int OFF_WY = OFF_X;                     // [V ; sa] . dY^T    128-row slab  } adjacent, alias X
constexpr int OFF_WSA = OFF_WY + SLAB128;         // [V ; sa] . dsa^T   128-row slab  }
constexpr int OFF_LF = OFF_X + 4 * SLAB64;        // fp32 A_ab for the inverse; later the decay-gradient scan
constexpr int OFF_CUM = OFF_LF + LF_PITCH * 64 * 4;   // fp32 cumulative log-decay [64][LF_PITCH]
constexpr int OFF_DSF = OFF_CUM + LF_PITCH * 64 * 4;   // fp32 dS carried across chunks [64][LF_PITCH]
constexpr int OFF_XINV = OFF_DSF + LF_PITCH * 64 * 4; // fp32 (I - A_ab)^-1
constexpr int OFF_SCR = OFF_XINV + LF_PITCH * 64 * 4;    // scratch of the inverse
// Staging tiles for the raw rows of the NEXT chunk (7 streams x 64 tokens x 128 bytes), filled by bulk
// asynchronous copies while the current chunk finishes.  Tiles 0..4 lie over XINV, SCR and a tail kept
// for them (all idle once the inverse has been converted), tiles 5..6 over TINV + A_ak (idle once the
// fourth round of products has completed).
constexpr int STG_TILE = kC * kN * 2;
constexpr int OFF_STG = OFF_XINV;
constexpr int STG_TAIL = 5 * STG_TILE - (LF_PITCH * 64 * 4 + TRI_SCR_FLOATS * 4);
constexpr int OFF_SMALL = OFF_SCR + TRI_SCR_FLOATS * 4 + STG_TAIL;
static_assert(STG_TAIL >= 0 && 2 * STG_TILE <= 2 * SLAB64, "staging tiles must fit their hosts");
__device__ __forceinline__ int stage_off(int m) { return m < 5 ? OFF_STG + m * STG_TILE : OFF_TINV + (m - 5) * STG_TILE; }
static_assert(2 * SLAB128 <= 4 * SLAB64, "W must fit over the X region");
struct Small {
    float h1[kN];
    float tot[kN];
    float lam[kN];
    float d_in[kN];        // D carried from the chunk processed before (later in time)
    float d_part[4][kN];   // partial column sums of the new anchor (16 rows each)
    float seg[4][kN];      // per-16-token totals of the decay-gradient scan
    uint64_t bar[7];       // 0..4 product rounds, 5 staging tiles, 6 operand slabs saved by the forward
    uint32_t nsm[2];       // chunk starts inside the current 64-token block
    uint32_t nsf[2];       // start flags inside the current block
    uint32_t tmem;
};
constexpr int SMEM_BYTES = OFF_SMALL + (int)sizeof(Small);
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

// TMEM columns
constexpr uint32_t T_D1 = 0;      // 128: Gram blocks of the forward recompute, later W
constexpr uint32_t T_G = 128;     // 64 : G, later [dR~' ; dA~']
constexpr uint32_t T_GD = 192;    // 64 : [Gd ; dV]
constexpr uint32_t T_SA = 256;    // 64 : sa
constexpr uint32_t T_DSA = 320;   // 64 : dsa
constexpr uint32_t T_TMP = 384;   // 64 : dsa^T A~ + dY^T R~
constexpr uint32_t T_KB = 448;    // 64 : [dK~' ; dB~']


// four K=16 steps (64 deep) of D (+)= A B
__device__ __forceinline__ void mma_k64(uint32_t d, Op a, Op b, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) tc::mma(d, op_desc(a, ks), op_desc(b, ks), idesc, accumulate || ks > 0);
}

__global__ void __launch_bounds__(256, 1)
wkv7_chunk_bwd_kernel(int Tlen, int H, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ r,
                      const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                      const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                      const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                      const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ ds_out,
                      const float* __restrict__ ckpt, const float* __restrict__ s_at_len,
                      __nv_bfloat16* __restrict__ dw, __nv_bfloat16* __restrict__ dr, __nv_bfloat16* __restrict__ dk,
                      __nv_bfloat16* __restrict__ dv, __nv_bfloat16* __restrict__ da, __nv_bfloat16* __restrict__ db,
                      __nv_bfloat16* __restrict__ ds0, int* __restrict__ status, int BH, int SEG,
                      float* __restrict__ carry, int* __restrict__ carry_flag, const __grid_constant__ StreamMaps maps,
                      const unsigned char* __restrict__ saved, const int* __restrict__ residual_mark,
                      const int* __restrict__ fast) {
    // the forward call fell back to the token-sequential kernel (a decay outside the chunked kernels' range):
    // the residual is in that kernel's format and its backward, launched behind this one, does the work
    if (*residual_mark != 0) return;
    // sequences walked in full saved blocks belong to the carry + gradient kernels; leave at once (before any
    // barrier or TMEM allocation) when nothing else lies in this CTA's range
    {
        const long long lo = (long long)BH * SEG * blockIdx.x / gridDim.x, hi = (long long)BH * SEG * (blockIdx.x + 1) / gridDim.x;
        bool mine = false;
        for (long long c = lo / SEG; c <= (hi - 1) / SEG && hi > lo; ++c) mine = mine || (fast[c] == 0);
        if (!mine) return;
    }
    extern __shared__ __align__(128) unsigned char smem[];
    Small& sm = *reinterpret_cast<Small*>(smem + OFF_SMALL);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hsel = warp >> 2;     // TMEM lane quadrant / column half handled by this warp
    const int row = quad * 32 + lane;                // TMEM lane == tile row
    // Two threads issue the products of every round, each its own accumulators, so that issue (a serial
    // instruction stream per thread) takes half as long; they sit in the warps with the least epilogue work.
    // Both commit to the round's mbarrier (count 2).  The copy engines are driven from two other idle warps.
    const bool issuer_a = (tid == 64), issuer_b = (tid == 192);
    constexpr int kStageThread = 96, kSavedThread = 224;
    const size_t tok_stride = (size_t)H * kN;
    const int nBlk = (Tlen + kC - 1) / kC;
    // the sequence this CTA currently walks (set per run)
    int bh = 0, bi = 0, L = 0;
    size_t seq_base = 0, st_base = 0;
    // units [unit_lo, unit_hi) of the (sequence, segment) list belong to this CTA
    const long long unit_lo = (long long)BH * SEG * blockIdx.x / gridDim.x;
    const long long unit_hi = (long long)BH * SEG * (blockIdx.x + 1) / gridDim.x;
    const int n_runs = run_count(unit_lo, unit_hi, SEG);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 7; ++i) tc::mbar_init(&sm.bar[i], i < 5 ? 2 : 1);   // product rounds: one arrival per issuing thread
        tc::mbar_init_fence();
    }
    if (warp == 0) tc::tmem_alloc(&sm.tmem, 512);
    float* dsf = reinterpret_cast<float*>(smem + OFF_DSF);   // [64][LF_PITCH]
    float* cum = reinterpret_cast<float*>(smem + OFF_CUM);   // [64][LF_PITCH]
    float* lf = reinterpret_cast<float*>(smem + OFF_LF);     // [64][LF_PITCH]
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tbase = sm.tmem;
    const uint32_t lane_addr = tbase + ((uint32_t)(quad * 32) << 16);
    bool failed = false;

    const uint32_t sAR = tc::smem_u32(smem + OFF_AR), sBK = tc::smem_u32(smem + OFF_BK);
    const uint32_t sVSA = tc::smem_u32(smem + OFF_VSA), sDD = tc::smem_u32(smem + OFF_DD);
    const uint32_t sS0 = tc::smem_u32(smem + OFF_S0), sDSL = tc::smem_u32(smem + OFF_DSL);
    const uint32_t sTINV = tc::smem_u32(smem + OFF_TINV), sAAK = tc::smem_u32(smem + OFF_AAK);
    const uint32_t sPRB = tc::smem_u32(smem + OFF_PRB), sG = tc::smem_u32(smem + OFF_G), sGD = tc::smem_u32(smem + OFF_GD);
    const uint32_t sWY = tc::smem_u32(smem + OFF_WY), sWSA = tc::smem_u32(smem + OFF_WSA);
    constexpr uint32_t ID_N128_KK = tc::make_idesc(128, 128, false, false);
    constexpr uint32_t ID_KK = tc::make_idesc(128, 64, false, false);
    constexpr uint32_t ID_KM = tc::make_idesc(128, 64, false, true);
    constexpr uint32_t ID_MM = tc::make_idesc(128, 64, true, true);
    constexpr uint32_t HALF = 64 * 16;   // byte offset of row 64 inside a 128-row slab column block

    const int tsub = tid >> 3, jb = tid & 7;   // staging unit: tokens 32q + tsub (q = 0,1), channels 8jb..8jb+7
    const int si = tid & 63, scq = tid >> 6;   // state element ownership: row si, columns 16scq..16scq+15
    // phase parities: product rounds 1..4 (every chunk), round 0 (recomputing chunks only), staging tiles, saved slabs
    uint32_t par = 0, par0 = 0, spar = 0, lpar = 0;

    // ---- chunk schedule, walked in reverse.  The extent and the global loads of the next chunk are
    // issued while the tail of the current one (decay-gradient scan) still runs.
    int blk = nBlk - 1, bs = 0, be = 0, p1 = 0, p = 0, n = 0;
    uint64_t cmask = 0, fmask = 0;
    bool reset_here = false;
    uint4 raw[2][6];   // r, k, v, a, b, dy
    uint4 wraw[2];     // raw log-log decay
    uint8_t flag_ahead = 0;   // threads 0..63: the start flag of their token in the block planned next
    auto fetch_flags = [&](int b) {
        if (tid < 64 && b >= 0 && b * kC + tid < Tlen) flag_ahead = new_starts[(size_t)bi * Tlen + b * kC + tid];
    };
    auto plan_block = [&](int b) {
        // chunk starts inside block b: its first token, every start flag, and `length`.  The flag bytes
        // were requested one block earlier (fetch_flags), so no global load sits in front of the ballots.
        bs = b * kC;
        be = min(bs + kC, Tlen);
        __syncthreads();
        if (tid < 64) {
            const int pos = bs + tid;
            const bool flag = (pos < be) && (flag_ahead != 0);
            const bool f = (pos < be) && (tid == 0 || flag || pos == L);
            const uint32_t m = __ballot_sync(0xffffffffu, f), mf = __ballot_sync(0xffffffffu, flag);
            if (lane == 0) { sm.nsm[warp] = m; sm.nsf[warp] = mf; }
        }
        fetch_flags(b - 1);
        __syncthreads();
        cmask = (uint64_t)sm.nsm[0] | ((uint64_t)sm.nsm[1] << 32);
        fmask = (uint64_t)sm.nsf[0] | ((uint64_t)sm.nsf[1] << 32);
    };
    auto plan_chunk = [&](int end) {   // the chunk [p, end) of the current block, bs < end <= be
        const int rel = end - bs;      // 1..64
        const uint64_t below = (rel >= 64) ? cmask : (cmask & ((1ull << rel) - 1ull));
        p = bs + 63 - __clzll((long long)below);
        n = end - p;
        reset_here = ((fmask >> (p - bs)) & 1ull) != 0;
    };
    // the 64 token rows from cp on of the seven streams into the staging tiles: one tiled copy of
    // 64 x 128 bytes per stream, all issued by one thread.  Rows past the chunk arrive too and are ignored.
    const int n_streams = (dy != nullptr) ? 7 : 6;
    auto issue_stage = [&](int cp) {
        if (tid == kStageThread) {
            tc::mbar_expect_tx(&sm.bar[5], (uint32_t)(n_streams * STG_TILE));
            const int x = (bh % H) * kN, y = bi * Tlen + cp;
#pragma unroll
            for (int m = 0; m < 7; ++m)
                if (m < n_streams) tc::tensor_load_2d(smem + stage_off(m), &maps.m[m], x, y, &sm.bar[5]);
        }
    };
    auto take_stage = [&]() {
        if (!tc::mbar_wait(&sm.bar[5], spar)) failed = true;
        spar ^= 1u;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int t = q * 32 + tsub;
            if (t < n) {
                const int o = t * (kN * 2) + jb * 16;
                wraw[q] = *reinterpret_cast<const uint4*>(smem + stage_off(0) + o);
#pragma unroll
                for (int m = 0; m < 5; ++m) raw[q][m] = *reinterpret_cast<const uint4*>(smem + stage_off(m + 1) + o);
                raw[q][5] = (dy != nullptr) ? *reinterpret_cast<const uint4*>(smem + stage_off(6) + o) : make_uint4(0, 0, 0, 0);
            } else {
                wraw[q] = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int m = 0; m < 6; ++m) raw[q][m] = make_uint4(0, 0, 0, 0);
            }
        }
    };
    // A 64-token block that the forward walked as one chunk has its operand slabs T, A_ak, P_rb, P_rk and sa
    // in the residual: the backward copies them in instead of recomputing them (no Gram product, no inverse).
    // P_rb|P_rk and sa can start as soon as the fifth product round of the chunk before has completed;
    // T|A_ak lie under staging tiles and follow once take_stage has emptied those.
    auto is_saved = [&](int cp, int cn) { return cn == kC && (cp & (kC - 1)) == 0; };
    // Tiles in global memory are unpadded (8 column blocks of 1 KB); the slabs here are padded, so every tile
    // arrives as 8 copies, one per column block, issued by the lanes of one warp.
    auto issue_saved_late = [&](int cp) {
        if (warp == (kSavedThread >> 5)) {
            const unsigned char* src = saved + ((size_t)bh * nBlk + (cp >> 6)) * kSavedBytes;
            if (lane == 0) {
                tc::mbar_expect_tx(&sm.bar[6], (uint32_t)(6 * GTILE));
                tc::bulk_prefetch_l2(src + SAVED_T * GTILE, 2 * GTILE);   // copied in later, from L2 then
            }
            __syncwarp();
            const int c = lane & 7, which = lane >> 3;   // 0: P_rb, 1: P_rk, 2: S0, 3: sa
            const int tile = which == 0 ? SAVED_PRB : (which == 1 ? SAVED_PRK : (which == 2 ? SAVED_S0 : SAVED_SA));
            unsigned char* dst = which == 0 ? smem + OFF_PRB + c * CB64
                               : which == 1 ? smem + OFF_PRK + c * CB64
                               : which == 2 ? smem + OFF_S0 + c * CB64
                                            : smem + OFF_VSA + c * CB128 + 64 * 16;
            tc::bulk_load(dst, src + (size_t)tile * GTILE + c * GCB, 64 * 16, &sm.bar[6]);
        }
    };
    auto issue_saved_early = [&](int cp) {
        if (warp == (kSavedThread >> 5) && lane < 16) {
            const unsigned char* src = saved + ((size_t)bh * nBlk + (cp >> 6)) * kSavedBytes;
            const int c = lane & 7, which = lane >> 3;   // 0: T, 1: A_ak
            tc::bulk_load(smem + (which == 0 ? OFF_TINV : OFF_AAK) + c * CB64, src + (size_t)(which == 0 ? SAVED_T : SAVED_AAK) * GTILE + c * GCB,
                          64 * 16, &sm.bar[6]);
        }
    };
    bool loaded_next = false;
    for (int order = 0; order < n_runs; ++order) {
    const RunPlan run = run_at(unit_lo, unit_hi, SEG, order);
    bh = run.chain;
    if (fast[bh] != 0) continue;
    bi = bh / H;
    L = min((int)length[bi], Tlen);
    seq_base = (size_t)bi * Tlen * tok_stride + (size_t)(bh % H) * kN;
    st_base = (size_t)bh * kN * kN;
    // segments are counted from the end of the sequence: segment j covers blocks
    // [nBlk (SEG-1-j) / SEG, nBlk (SEG-j) / SEG)
    const int blk_hi = (int)((long long)nBlk * (SEG - run.seg_from) / SEG);
    const int blk_lo = (int)((long long)nBlk * (SEG - run.seg_to) / SEG);
    const int tok_lo = blk_lo * kC;
    __syncthreads();   // the previous run has finished with dsf and d_in
    if (run.seg_from == 0) {
        for (int idx = tid; idx < 64 * LF_PITCH; idx += 256) dsf[idx] = 0.f;
        if (tid < 64) sm.d_in[tid] = 0.f;
    } else {
        // the later part of this sequence was walked by the previous CTA: take over its carry
        const int slot = (int)blockIdx.x - 1;
        if (tid == 0) {
            bool ready = false;
            for (uint32_t it = 0; it < (1u << 24) && !ready; ++it) {
                int f;
                asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(f) : "l"(carry_flag + slot) : "memory");
                ready = f != 0;
                if (!ready) __nanosleep(64);
            }
            sm.nsm[0] = ready ? 1u : 0u;
        }
        __syncthreads();
        if (sm.nsm[0] == 0u) failed = true;
        const float* src = carry + (size_t)slot * kHandoffFloats;
        for (int idx = tid; idx < 64 * 16; idx += 256) {
            const int rr = idx >> 4, c4 = (idx & 15) * 4;
            *reinterpret_cast<float4*>(&dsf[rr * LF_PITCH + c4]) = __ldcg(reinterpret_cast<const float4*>(src + rr * kN + c4));
        }
        if (tid < 64) sm.d_in[tid] = __ldcg(src + kN * kN + tid);
    }
    blk = blk_hi - 1;
    fetch_flags(blk);
    plan_block(blk);   // begins and ends with a barrier: dsf and d_in are in place afterwards
    p1 = be;
    plan_chunk(p1);
    tc::fence_async_smem();   // the tiles' hosts were last written by ordinary stores
    __syncthreads();
    issue_stage(p);
    loaded_next = is_saved(p, n);
    if (loaded_next) issue_saved_late(p);
    while (true) {
        {
            const bool cur_loaded = loaded_next;
            take_stage();
            // ---------------- cotangent of the returned state enters at position `length` ----------------
            if (p1 == L && ds_out != nullptr) {
                float g[16];
                unpack8(*reinterpret_cast<const uint4*>(ds_out + st_base + si * kN + scq * 16), g);
                unpack8(*reinterpret_cast<const uint4*>(ds_out + st_base + si * kN + scq * 16 + 8), g + 8);
#pragma unroll
                for (int e = 0; e < 16; ++e) dsf[si * LF_PITCH + scq * 16 + e] += g[e];
                if (tid < 64) {
                    float acc = 0.f;
                    for (int i = 0; i < 64; ++i)
                        acc += __bfloat162float(ds_out[st_base + i * kN + tid]) * s_at_len[st_base + i * kN + tid];
                    sm.d_in[tid] += acc;
                }
            }
            // ---------------- cumulative decay of the chunk ----------------
            float lw[2][8];
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int t = q * 32 + tsub;
                float wf[8];
                unpack8(wraw[q], wf);
#pragma unroll
                for (int e = 0; e < 8; ++e) lw[q][e] = (t < n) ? -kLog2e * __expf(wf[e]) : 0.f;   // log2 of the decay
                *reinterpret_cast<float4*>(&cum[t * LF_PITCH + jb * 8]) = make_float4(lw[q][0], lw[q][1], lw[q][2], lw[q][3]);
                *reinterpret_cast<float4*>(&cum[t * LF_PITCH + jb * 8 + 4]) = make_float4(lw[q][4], lw[q][5], lw[q][6], lw[q][7]);
            }
            __syncthreads();
            if (cur_loaded) issue_saved_early(p);   // every thread has emptied the staging tiles over T | A_ak
            if (tid < 128) {
                const int j = tid & 63, half = tid >> 6;
                float run = 0.f;
#pragma unroll 8
                for (int tt = 0; tt < 32; ++tt) {
                    const int t = half * 32 + tt;
                    run += cum[t * LF_PITCH + j];
                    cum[t * LF_PITCH + j] = run;
                }
                if (half == 0) sm.h1[j] = run;
                else sm.tot[j] = run;
            }
            __syncthreads();
            if (tid < 64) {
                const float t2 = fmaxf(sm.h1[tid] + sm.tot[tid], kCumFloor);
                sm.tot[tid] = t2;
                sm.lam[tid] = ex2(t2);
            }
            __syncthreads();
            {
                float h1v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) h1v[e] = sm.h1[jb * 8 + e];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                    const int t = q * 32 + tsub;
                    float c[8];
                    *reinterpret_cast<float4*>(&c[0]) = *reinterpret_cast<const float4*>(&cum[t * LF_PITCH + jb * 8]);
                    *reinterpret_cast<float4*>(&c[4]) = *reinterpret_cast<const float4*>(&cum[t * LF_PITCH + jb * 8 + 4]);
                    float eL[8], eI[8], eP[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float cc = fmaxf(c[e] + (q == 1 ? h1v[e] : 0.f), kCumFloor);
                        const float cp = fminf(fmaxf(cc - lw[q][e], kCumFloor), 0.f);
                        eL[e] = ex2(cc); eI[e] = ex2(-cc); eP[e] = ex2(cp);
                    }
                    // raw: r, k, v, a, b, dy
                    slab_store(smem + OFF_AR, CB128, t, jb, scale8(raw[q][3], eP));
                    slab_store(smem + OFF_AR, CB128, 64 + t, jb, scale8(raw[q][0], eL));
                    slab_store(smem + OFF_BK, CB128, t, jb, scale8(raw[q][4], eI));
                    slab_store(smem + OFF_BK, CB128, 64 + t, jb, scale8(raw[q][1], eI));
                    slab_store(smem + OFF_VSA, CB128, t, jb, raw[q][2]);
                    slab_store(smem + OFF_DD, CB128, t, jb, raw[q][5]);
                }
            }
            // ---------------- entering state (bf16) and decayed incoming state gradient (bf16) ----------------
            const float* s0src = reset_here ? nullptr : ((p % kC == 0) ? ckpt + ((size_t)bh * nBlk + p / kC) * kN * kN
                                                                        : s_at_len + st_base);
            {
                float g[16];
                if (!cur_loaded) {   // (a loaded chunk gets the forward's own bf16 S0 slab by bulk copy)
                    float s[16];
                    if (s0src != nullptr) {
#pragma unroll
                        for (int c4 = 0; c4 < 4; ++c4) {
                            const float4 x = *reinterpret_cast<const float4*>(s0src + si * kN + scq * 16 + c4 * 4);
                            s[c4 * 4] = x.x; s[c4 * 4 + 1] = x.y; s[c4 * 4 + 2] = x.z; s[c4 * 4 + 3] = x.w;
                        }
                    } else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) s[e] = 0.f;
                    }
                    slab_store(smem + OFF_S0, CB64, si, scq * 2, pack8(s));
                    slab_store(smem + OFF_S0, CB64, si, scq * 2 + 1, pack8(s + 8));
                }
#pragma unroll
                for (int e = 0; e < 16; ++e) g[e] = dsf[si * LF_PITCH + scq * 16 + e] * sm.lam[scq * 16 + e];
                slab_store(smem + OFF_DSL, CB64, si, scq * 2, pack8(g));
                slab_store(smem + OFF_DSL, CB64, si, scq * 2 + 1, pack8(g + 8));
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            if (cur_loaded) {
                // T, A_ak, P_rb, P_rk and sa of this chunk come from the forward
                if (!tc::mbar_wait(&sm.bar[6], lpar)) failed = true;
                lpar ^= 1u;
            } else {
            // ================= R1: Gram blocks, A~ S0^T =================
            if (issuer_a) {
                tc::fence_after_sync();
                mma_k64(tbase + T_D1, kmaj128(sAR), kmaj128(sBK), ID_N128_KK, false);
                tc::commit(&sm.bar[0]);
            } else if (issuer_b) {
                tc::fence_after_sync();
                mma_k64(tbase + T_G, kmaj128(sAR), kmaj64(sS0), ID_KK, false);
                tc::commit(&sm.bar[0]);
            }
            if (!tc::mbar_wait(&sm.bar[0], par0)) failed = true;
            par0 ^= 1u;
            tc::fence_after_sync();
            {
                const int t = row & 63;
                float d[64];
                tc::tmem_ld32(lane_addr + T_D1 + hsel * 64, d);
                tc::tmem_ld32(lane_addr + T_D1 + hsel * 64 + 32, d + 32);
                tc::tmem_wait_ld();
                if (row < 64 && hsel == 0) {          // A_ab, strictly lower, fp32 for the inverse
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        *reinterpret_cast<float4*>(&lf[t * LF_PITCH + c * 4]) =
                            make_float4(c * 4 + 0 < t ? d[c * 4 + 0] : 0.f, c * 4 + 1 < t ? d[c * 4 + 1] : 0.f,
                                        c * 4 + 2 < t ? d[c * 4 + 2] : 0.f, c * 4 + 3 < t ? d[c * 4 + 3] : 0.f);
                } else {
                    const int lim = (row < 64) ? t : t + 1;   // A_ak strict; P_rb, P_rk inclusive
#pragma unroll
                    for (int s = 0; s < 64; ++s) d[s] = (s < lim) ? d[s] : 0.f;
                    unsigned char* dst = smem + ((row < 64) ? OFF_AAK : (hsel == 0 ? OFF_PRB : OFF_PRK));
#pragma unroll
                    for (int c = 0; c < 8; ++c) slab_store(dst, CB64, t, c, pack8(&d[c * 8]));
                }
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            }   // recomputing chunk
            // ================= R2: G += A_ak V ; [Gd ; dVpart] = [B~;K~] dSL^T + [P_rb|P_rk]^T dY ; inverse =================
            if (issuer_a) {
                tc::fence_after_sync();
                mma_k64(tbase + T_GD, kmaj128(sBK), kmaj64(sDSL), ID_KK, false);
                mma_k64(tbase + T_GD, mnmaj64(sPRB), mnmaj128(sDD), ID_MM, true);
                tc::commit(&sm.bar[1]);
            } else if (issuer_b) {
                tc::fence_after_sync();
                if (!cur_loaded) mma_k64(tbase + T_G, kmaj64(sAAK), mnmaj128(sVSA), ID_KM, true);
                tc::commit(&sm.bar[1]);
            }
            if (!cur_loaded) {
                tri_inverse_64<256>(lf, reinterpret_cast<float*>(smem + OFF_XINV), reinterpret_cast<float*>(smem + OFF_SCR), tid);
                fp32_to_slab64<256>(reinterpret_cast<const float*>(smem + OFF_XINV), smem + OFF_TINV, CB64, tid);
            }
            if (quad < 2) {
                if (!tc::mbar_wait(&sm.bar[1], par)) failed = true;
                tc::fence_after_sync();
                float gd[32];
                tc::tmem_ld32(lane_addr + T_GD + hsel * 32, gd);
                if (!cur_loaded) {
                    float g[32];
                    tc::tmem_ld32(lane_addr + T_G + hsel * 32, g);
                    tc::tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 4; ++c) slab_store(smem + OFF_G, CB64, row, hsel * 4 + c, pack8(&g[c * 8]));
                } else {
                    tc::tmem_wait_ld();
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(smem + OFF_GD, CB64, row, hsel * 4 + c, pack8(&gd[c * 8]));
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            // ================= R3: sa = T G ; dsa = T^T Gd =================
            if (issuer_a) {
                tc::fence_after_sync();
                mma_k64(tbase + T_DSA, mnmaj64(sTINV), mnmaj64(sGD), ID_MM, false);
                tc::commit(&sm.bar[2]);
            } else if (issuer_b) {
                tc::fence_after_sync();
                if (!cur_loaded) mma_k64(tbase + T_SA, kmaj64(sTINV), mnmaj64(sG), ID_KM, false);
                tc::commit(&sm.bar[2]);
            }
            if (quad < 2) {
                if (!tc::mbar_wait(&sm.bar[2], par)) failed = true;
                tc::fence_after_sync();
                float z[32];
                tc::tmem_ld32(lane_addr + T_DSA + hsel * 32, z);
                if (!cur_loaded) {
                    float x[32];
                    tc::tmem_ld32(lane_addr + T_SA + hsel * 32, x);
                    tc::tmem_wait_ld();
#pragma unroll
                    for (int c = 0; c < 4; ++c) slab_store(smem + OFF_VSA, CB128, 64 + row, hsel * 4 + c, pack8(&x[c * 8]));
                } else {
                    tc::tmem_wait_ld();
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(smem + OFF_DD, CB128, 64 + row, hsel * 4 + c, pack8(&z[c * 8]));
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            // ================= R4: dV += A_ak^T dsa ; W = [V;sa][dY;dsa]^T ; tmp = dY^T R~ + dsa^T A~ =================
            if (issuer_a) {
                tc::fence_after_sync();
                mma_k64(tbase + T_D1, kmaj128(sVSA), kmaj128(sDD), ID_N128_KK, false);
                mma_k64(tbase + T_GD, mnmaj64(sTINV), mnmaj128(sDD + HALF), ID_MM, true);
                tc::commit(&sm.bar[3]);
            } else if (issuer_b) {
                tc::fence_after_sync();
                mma_k64(tbase + T_TMP, mnmaj128(sDD), mnmaj128(sAR + HALF), ID_MM, false);
                mma_k64(tbase + T_TMP, mnmaj128(sDD + HALF), mnmaj128(sAR), ID_MM, true);
                tc::commit(&sm.bar[3]);
            }
            if (!tc::mbar_wait(&sm.bar[3], par)) failed = true;
            tc::fence_after_sync();
            // ---------------- plan the next chunk (earlier in time) ----------------
            const int cur_p = p, cur_n = n;
            const bool cur_reset = reset_here;
            const bool has_next = cur_p > tok_lo;
            if (has_next) {
                if (cur_p == bs) plan_block(--blk);
                plan_chunk(cur_p);
            }
            loaded_next = has_next && is_saved(p, n);
            {
                const int t = row & 63;
                float d[64];
                tc::tmem_ld32(lane_addr + T_D1 + hsel * 64, d);
                tc::tmem_ld32(lane_addr + T_D1 + hsel * 64 + 32, d + 32);
                tc::tmem_wait_ld();
                const int lo = t + hsel;   // keep s >= t for the dY blocks, s > t for the dsa blocks
#pragma unroll
                for (int s = 0; s < 64; ++s) d[s] = (s >= lo) ? d[s] : 0.f;
                unsigned char* dst = smem + (hsel == 0 ? OFF_WY : OFF_WSA);
#pragma unroll
                for (int c = 0; c < 8; ++c) slab_store(dst, CB128, row, c, pack8(&d[c * 8]));
            }
            if (quad >= 2) {   // dV rows
                const int t = row - 64;
                float x[32];
                tc::tmem_ld32(lane_addr + T_GD + hsel * 32, x);
                tc::tmem_wait_ld();
                if (t < cur_n) {
                    __nv_bfloat16* dst = dv + seq_base + (size_t)(cur_p + t) * tok_stride + hsel * 32;
#pragma unroll
                    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = pack8(&x[c * 8]);
                }
            } else {           // state-gradient carry (fp32, shared memory): dS0 = dS diag(L_C) + dsa^T A~ + dY^T R~
                float x[32];
                tc::tmem_ld32(lane_addr + T_TMP + hsel * 32, x);
                tc::tmem_wait_ld();
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const int c = hsel * 32 + c4 * 4;
                    float4 old = *reinterpret_cast<const float4*>(&dsf[row * LF_PITCH + c]);
                    const float4 l4 = *reinterpret_cast<const float4*>(&sm.lam[c]);
                    old.x = fmaf(old.x, l4.x, x[c4 * 4 + 0]); old.y = fmaf(old.y, l4.y, x[c4 * 4 + 1]);
                    old.z = fmaf(old.z, l4.z, x[c4 * 4 + 2]); old.w = fmaf(old.w, l4.w, x[c4 * 4 + 3]);
                    *reinterpret_cast<float4*>(&dsf[row * LF_PITCH + c]) = old;
                }
            }
            tc::fence_async_smem();
            tc::fence_before_sync();
            __syncthreads();
            // ================= R5: [dK~';dB~'] and [dR~';dA~'] =================
            if (issuer_a) {
                tc::fence_after_sync();
                mma_k64(tbase + T_KB, kmaj128(sWSA), mnmaj128(sAR), ID_KM, false);
                mma_k64(tbase + T_KB, kmaj128(sWY), mnmaj128(sAR + HALF), ID_KM, true);
                mma_k64(tbase + T_KB, kmaj128(sVSA), mnmaj64(sDSL), ID_KM, true);
                tc::commit(&sm.bar[4]);
            } else if (issuer_b) {
                tc::fence_after_sync();
                mma_k64(tbase + T_G, kmaj128(sDD), mnmaj64(sS0), ID_KM, false);
                mma_k64(tbase + T_G, mnmaj128(sWY + HALF), mnmaj128(sBK), ID_MM, true);
                mma_k64(tbase + T_G, mnmaj128(sWY), mnmaj128(sBK + HALF), ID_MM, true);
                tc::commit(&sm.bar[4]);
            }
            // the rows of the next chunk (earlier in time) start travelling while the products run: their
            // tiles lie over buffers that the fourth round was the last to read
            if (has_next) issue_stage(p);
            // exact anchor of the decay gradient for the chunk before: D = column sums of dS0 * S0 in fp32 (16 rows
            // per thread) while the products run; the order of the additions is fixed
            {
                const int c = tid & 63, rq = tid >> 6;
                float acc = 0.f;
                if (cur_loaded) {
                    // a loaded chunk has no fp32 copy of its entering state: the bf16 slab the products use, read
                    // from the residual (in L2 since the bulk copy) rather than from shared memory, whose bandwidth
                    // the running products need for their operands
                    const __nv_bfloat16* s0b = reinterpret_cast<const __nv_bfloat16*>(
                                                   saved + ((size_t)bh * nBlk + (cur_p >> 6)) * kSavedBytes + SAVED_S0 * GTILE + (c >> 3) * GCB) + (c & 7);
                    __nv_bfloat16 sv[16];   // all loads in flight at once
#pragma unroll
                    for (int rr = 0; rr < 16; ++rr) sv[rr] = __ldg(s0b + (rq * 16 + rr) * 8);
#pragma unroll
                    for (int rr = 0; rr < 16; ++rr) acc = fmaf(dsf[(rq * 16 + rr) * LF_PITCH + c], __bfloat162float(sv[rr]), acc);
                } else if (s0src != nullptr) {
                    float sv[16];   // all 16 loads in flight at once: their latency is paid once
#pragma unroll
                    for (int rr = 0; rr < 16; ++rr) sv[rr] = __ldg(s0src + (rq * 16 + rr) * kN + c);
#pragma unroll
                    for (int rr = 0; rr < 16; ++rr) acc = fmaf(dsf[(rq * 16 + rr) * LF_PITCH + c], sv[rr], acc);
                }
                sm.d_part[rq][c] = acc;
            }
            // everything of the epilogue that does not depend on the products runs while they execute:
            // decay factors of this row and the operand rows it pairs with (kept packed)
            float fx[32], fz[32], lwt[32];
            uint4 s1raw[4], s2raw[4];
            {
                const int t = row & 63;
                const unsigned char* slab1 = smem + OFF_AR + ((row < 64) ? (64 + t) * 16 : t * 16);   // R~ / A~
                const unsigned char* slab2 = smem + OFF_BK + ((row < 64) ? (64 + t) * 16 : t * 16);   // K~ / B~
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    s1raw[c8] = *reinterpret_cast<const uint4*>(slab1 + (hsel * 4 + c8) * CB128);
                    s2raw[c8] = *reinterpret_cast<const uint4*>(slab2 + (hsel * 4 + c8) * CB128);
                }
#pragma unroll
                for (int c4 = 0; c4 < 8; ++c4) {
                    const int c = hsel * 32 + c4 * 4;
                    const float4 cr4 = *reinterpret_cast<const float4*>(&cum[t * LF_PITCH + c]);
                    const float4 cp4 = (t & 31) ? *reinterpret_cast<const float4*>(&cum[(t - 1) * LF_PITCH + c])
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float4 h4 = (t >= 32) ? *reinterpret_cast<const float4*>(&sm.h1[c]) : make_float4(0.f, 0.f, 0.f, 0.f);
                    const float cr[4] = {cr4.x, cr4.y, cr4.z, cr4.w}, cp[4] = {cp4.x, cp4.y, cp4.z, cp4.w};
                    const float hh[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
                    for (int e4 = 0; e4 < 4; ++e4) {
                        const int e = c4 * 4 + e4;
                        const float cc = fmaxf(cr[e4] + hh[e4], kCumFloor);
                        lwt[e] = cr[e4] - cp[e4];
                        fx[e] = ex2(-cc);                                                     // dk, db: 1 / L_t
                        fz[e] = (row < 64) ? ex2(cc)                                            // dr: L_t
                                           : ex2(fminf(fmaxf(cc - lwt[e], kCumFloor), 0.f));    // da: L_{t-1}
                    }
                }
            }
            if (!tc::mbar_wait(&sm.bar[4], par)) failed = true;
            tc::fence_after_sync();
            if (loaded_next) issue_saved_late(p);   // P_rb | P_rk and sa of the next chunk: their hosts are idle now
            float p3[32];   // a_t da_t for the rows that own da
            {
                const int t = row & 63;
                float x[32], z[32];
                tc::tmem_ld32(lane_addr + T_KB + hsel * 32, x);
                tc::tmem_ld32(lane_addr + T_G + hsel * 32, z);
                tc::tmem_wait_ld();
                float u[32];
#pragma unroll
                for (int c8 = 0; c8 < 4; ++c8) {
                    float s1[8], s2[8];
                    unpack8(s1raw[c8], s1);
                    unpack8(s2raw[c8], s2);
#pragma unroll
                    for (int e8 = 0; e8 < 8; ++e8) {
                        const int e = c8 * 8 + e8;
                        if (row < 64) {          // dk, dr ; u = r dr - k dk
                            u[e] = s1[e8] * z[e] - s2[e8] * x[e];
                        } else {                 // db, da ; u = a da - b db
                            p3[e] = s1[e8] * z[e];
                            u[e] = p3[e] - s2[e8] * x[e];
                        }
                        x[e] *= fx[e];
                        z[e] *= fz[e];
                    }
                }
                if (t < cur_n) {
                    const size_t g = seq_base + (size_t)(cur_p + t) * tok_stride + hsel * 32;
                    __nv_bfloat16* dx = (row < 64) ? dk : db;
                    __nv_bfloat16* dz = (row < 64) ? dr : da;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        *reinterpret_cast<uint4*>(dx + g + c * 8) = pack8(&x[c * 8]);
                        *reinterpret_cast<uint4*>(dz + g + c * 8) = pack8(&z[c * 8]);
                    }
                }
                // u_t = (r dr - k dk) + (a da - b db): first the dk/dr rows write, then the db/da rows add
                if (row < 64) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4)
                        *reinterpret_cast<float4*>(&lf[t * LF_PITCH + hsel * 32 + c4 * 4]) =
                            make_float4(u[c4 * 4], u[c4 * 4 + 1], u[c4 * 4 + 2], u[c4 * 4 + 3]);
                }
                __syncthreads();
                if (row >= 64) {
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        float4 o = *reinterpret_cast<const float4*>(&lf[t * LF_PITCH + hsel * 32 + c4 * 4]);
                        o.x += u[c4 * 4]; o.y += u[c4 * 4 + 1]; o.z += u[c4 * 4 + 2]; o.w += u[c4 * 4 + 3];
                        *reinterpret_cast<float4*>(&lf[t * LF_PITCH + hsel * 32 + c4 * 4]) = o;
                    }
                }
                __syncthreads();
                {   // D_{t-1} = D_t + u_t from the carried D at the chunk end: suffix sums, 4 segments of 16 tokens
                    const int c = tid & 63, sg = tid >> 6;
                    float run = 0.f;
#pragma unroll 4
                    for (int tt = 15; tt >= 0; --tt) {
                        run += lf[(sg * 16 + tt) * LF_PITCH + c];
                        lf[(sg * 16 + tt) * LF_PITCH + c] = run;
                    }
                    sm.seg[sg][c] = run;
                }
                __syncthreads();
                {
                    const int c = tid & 63, sg = tid >> 6;
                    float off = sm.d_in[c];
                    for (int s2 = 3; s2 > sg; --s2) off += sm.seg[s2][c];
#pragma unroll 4
                    for (int tt = 0; tt < 16; ++tt) lf[(sg * 16 + tt) * LF_PITCH + c] += off;
                }
                __syncthreads();
                // carry for the previous chunk: the exact anchor, or zero across a start flag
                if (tid < 64) sm.d_in[tid] = cur_reset ? 0.f : ((sm.d_part[0][tid] + sm.d_part[1][tid]) + (sm.d_part[2][tid] + sm.d_part[3][tid]));
                __syncthreads();
                if (row >= 64 && t < cur_n) {
                    float o[32];
#pragma unroll
                    for (int c4 = 0; c4 < 8; ++c4) {
                        const float4 d4 = *reinterpret_cast<const float4*>(&lf[t * LF_PITCH + hsel * 32 + c4 * 4]);
                        o[c4 * 4 + 0] = (d4.x - p3[c4 * 4 + 0]) * (kLn2 * lwt[c4 * 4 + 0]);
                        o[c4 * 4 + 1] = (d4.y - p3[c4 * 4 + 1]) * (kLn2 * lwt[c4 * 4 + 1]);
                        o[c4 * 4 + 2] = (d4.z - p3[c4 * 4 + 2]) * (kLn2 * lwt[c4 * 4 + 2]);
                        o[c4 * 4 + 3] = (d4.w - p3[c4 * 4 + 3]) * (kLn2 * lwt[c4 * 4 + 3]);
                    }
                    if (cur_reset && t == 0) {   // the state entering a start token is zero: no decay gradient
#pragma unroll
                        for (int e = 0; e < 32; ++e) o[e] = 0.f;
                    }
                    __nv_bfloat16* dst = dw + seq_base + (size_t)(cur_p + t) * tok_stride + hsel * 32;
#pragma unroll
                    for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = pack8(&o[c * 8]);
                }
            }
            if (cur_reset) {
                __syncthreads();
#pragma unroll
                for (int e = 0; e < 16; ++e) dsf[si * LF_PITCH + scq * 16 + e] = 0.f;
            }
            tc::fence_before_sync();
            par ^= 1u;
            if (!has_next) break;
            p1 = cur_p;
        }
    }
    __syncthreads();
    if (run.seg_to == SEG) {   // the sequence is complete: gradient with respect to the initial state
        float g[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) g[e] = dsf[si * LF_PITCH + scq * 16 + e];
        if (L == 0 && ds_out != nullptr) {
            float o[16];
            unpack8(*reinterpret_cast<const uint4*>(ds_out + st_base + si * kN + scq * 16), o);
            unpack8(*reinterpret_cast<const uint4*>(ds_out + st_base + si * kN + scq * 16 + 8), o + 8);
#pragma unroll
            for (int e = 0; e < 16; ++e) g[e] += o[e];
        }
        *reinterpret_cast<uint4*>(ds0 + st_base + si * kN + scq * 16) = pack8(g);
        *reinterpret_cast<uint4*>(ds0 + st_base + si * kN + scq * 16 + 8) = pack8(g + 8);
    } else {                   // the next CTA walks the earlier part: hand the carry over
        float* dst = carry + (size_t)blockIdx.x * kHandoffFloats;
        for (int idx = tid; idx < 64 * 16; idx += 256) {
            const int rr = idx >> 4, c4 = (idx & 15) * 4;
            __stcg(reinterpret_cast<float4*>(dst + rr * kN + c4), *reinterpret_cast<const float4*>(&dsf[rr * LF_PITCH + c4]));
        }
        if (tid < 64) __stcg(dst + kN * kN + tid, sm.d_in[tid]);
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const int one = 1;
            asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(carry_flag + blockIdx.x), "r"(one) : "memory");
        }
    }
    }   // runs
    if (failed && status != nullptr) atomicExch(status, 2);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tbase, 512);
}

}  // namespace

int* wkv7_chunk_status_word();


int wkv7_chunk_bwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                   const void* a, const void* b, const uint32_t* length, const uint8_t* ns, const void* dy,
                   const void* ds_out, void* residual, const int* residual_mark, const int* fast, void* dw, void* dr,
                   void* dk, void* dv, void* da, void* db, void* ds0) {
    typedef __nv_bfloat16 bf;
    static DeviceOnce smem_attr;   // the opt-in to large dynamic shared memory is a per-device function attribute
    if (!smem_attr.ok([]() { return cudaFuncSetAttribute(wkv7_chunk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); }))
        return B200WKV_ELAUNCH;
    const float* ck = (const float*)residual;
    const int nBlk = (T + kC - 1) / kC;
    const float* sl = ck + (size_t)B * H * nBlk * kN * kN;
    // the tail of the buffer is scratch for carries between CTAs (see chunk_residual_floats)
    float* carry = (float*)residual + chunk_states_floats(B, T, H);
    int* carry_flag = reinterpret_cast<int*>(carry + (size_t)kHandoffSlots * kHandoffFloats);
    const unsigned char* saved = reinterpret_cast<const unsigned char*>(ck + chunk_saved_offset_floats(B, T, H));
    const bf *pw = (const bf*)w, *pr = (const bf*)r, *pk = (const bf*)k, *pv = (const bf*)v, *pa = (const bf*)a, *pb = (const bf*)b;
    const bf *pdy = (const bf*)dy, *pds = (const bf*)ds_out;
    bf *gw = (bf*)dw, *gr = (bf*)dr, *gk = (bf*)dk, *gv = (bf*)dv, *ga = (bf*)da, *gb = (bf*)db, *gs = (bf*)ds0;
    int* status = wkv7_chunk_status_word();
    int BH = B * H;
    StreamMaps maps;
    const void* bases[7] = {w, r, k, v, a, b, dy};   // maps[m]: the seven streams as [B*T tokens][H*64 channels]
    if (!make_stream_maps(&maps, bases, dy != nullptr ? 7 : 6, B, T, H)) return B200WKV_ELAUNCH;
    // One CTA per SM (shared memory).  With more sequences than SMs the CTAs are persistent; when
    // the sequences do not divide evenly, each is cut into `seg` runs of blocks so that every CTA
    // gets the same number of units, and neighbouring CTAs pass the carry through global memory.
    const SplitPlan plan = plan_split(BH, nBlk, 1, sm_count_of_current_device());
    if (plan.seg > 1) {
        if (cudaMemsetAsync(carry_flag, 0, (size_t)kHandoffSlots * sizeof(int), st) != cudaSuccess) return B200WKV_ELAUNCH;
        int Tl = T, Hl = H, seg = plan.seg;
        void* args[] = {&Tl, &Hl, &pw, &pr, &pk, &pv, &pa, &pb, &length, &ns, &pdy, &pds, &ck, &sl, &gw, &gr, &gk, &gv, &ga,
                        &gb, &gs, &status, &BH, &seg, &carry, &carry_flag, &maps, &saved, &residual_mark, &fast};
        // cooperative launch: the runtime guarantees that all CTAs are resident at once, which the
        // carry hand-over relies on; if it refuses, fall through to one CTA per sequence
        if (cudaLaunchCooperativeKernel((const void*)wkv7_chunk_bwd_kernel, dim3(plan.grid), dim3(256), args, SMEM_BYTES, st) ==
            cudaSuccess)
            return B200WKV_OK;
        (void)cudaGetLastError();
    }
    wkv7_chunk_bwd_kernel<<<plan.seg > 1 ? BH : plan.grid, 256, SMEM_BYTES, st>>>(T, H, pw, pr, pk, pv, pa, pb, length, ns, pdy, pds, ck,
                                                                               sl, gw, gr, gk, gv, ga, gb, gs, status, BH, 1,
                                                                               carry, carry_flag, maps, saved, residual_mark, fast);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace b200wkv

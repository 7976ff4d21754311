// RWKV-7 WKV forward, chunked along T on the Blackwell tensor cores (bf16 I/O, fp32 state).
//
// One CTA (256 threads) per (batch, head) walks the sequence in chunks of up to 64 tokens.  With
// L_t = prod_{s<=t} decay_s (per key channel, inside the chunk) and the scaled operands
//   A~_t = a_t * L_{t-1}   R~_t = r_t * L_t   B~_t = b_t / L_t   K~_t = k_t / L_t
//   B^_t = b_t * L_C / L_t K^_t = k_t * L_C / L_t                (L_C = decay over the whole chunk)
// the recurrence  S <- S diag(decay) + (S a) b^T + v k^T,  y = S r  becomes, for a chunk entered
// with state S0 (row = value index, column = key index):
//   [A_ab A_ak; P_rb P_rk] = [A~; R~] [B~; K~]^T            strictly / inclusively lower triangular
//   G   = A_ak V + A~ S0^T                                  (token x value)
//   sa  = (I - A_ab)^-1 G                                   row t is S_{t-1} a_t
//   Y   = P_rk V + R~ S0^T + P_rb sa
//   S_C = S0 diag(L_C) + sa^T B^ + V^T K^
// All products are tcgen05.mma (M=128, bf16 operands from shared memory, fp32 accumulators in
// TMEM); the unit-triangular inverse is an fp32 forward substitution on CUDA cores; the state
// stays in TMEM in fp32 for the whole sequence.  Start flags and `length` never need masks:
// a chunk simply ends early in front of a start position and at `length`, and the rows of a
// short chunk are zero-filled.
//
// Data movement: the raw rows of the next chunk arrive in shared memory by tiled bulk copies
// (cp.async.bulk.tensor) while the current chunk finishes.  When a residual is requested, every block
// walked as one full chunk leaves bf16 operand slabs for the backward (T, A_ak, P_rb, P_rk, sa, S0; most
// of them by bulk stores out of shared memory) so that the backward need not recompute them; the fp32
// state entering a block is written only when the block's first chunk is short.
//
// Semantics: BaseRWKV.inner_loop of jaxrwkv (src/jaxrwkv/rwkv7.py:199-220).
#include "common.cuh"
#include "tc05.cuh"
#include "chunk_common.cuh"
#include "tmap.cuh"

#include <atomic>

namespace b200wkv {

namespace {

// shared-memory map (bytes); two CTAs per SM
constexpr int OFF_AR = 0;                        // [A~ ; R~]           128-row slab  } dead once the first
constexpr int OFF_BK = OFF_AR + SLAB128;         // [B~ ; K~]           128-row slab  } products are done:
constexpr int OFF_S0 = OFF_BK + SLAB128;         // S0 in bf16          64-row slab   } LF, X, SCR alias them
constexpr int OFF_BH = OFF_S0 + SLAB64;          // B^                  64-row slab
constexpr int OFF_KH = OFF_BH + SLAB64;          // K^                  64-row slab
constexpr int OFF_SA = OFF_KH + SLAB64;          // sa                  64-row slab   } consecutive: the MN-major
constexpr int OFF_V = OFF_SA + SLAB64;           // V                   64-row slab   } A operands of the state
constexpr int OFF_M2A = OFF_V + SLAB64;          // [A_ak ; P_rk]       128-row slab  } update span two slabs
constexpr int OFF_G = OFF_M2A;                   // G (aliases M2A once the A_ak/P_rk product is done)
constexpr int OFF_TP = OFF_M2A + SLAB128;        // [Tinv ; P_rb]       128-row slab   (CUM aliases TP)
constexpr int OFF_SMALL = OFF_TP + LF_PITCH * 64 * 4;   // TP is 16512 B; the scan buffer that aliases it needs 17408
constexpr int OFF_LF = OFF_AR;                           // fp32 A_ab
constexpr int OFF_X = OFF_LF + LF_PITCH * 64 * 4;        // fp32 (I - A_ab)^-1
constexpr int OFF_SCR = OFF_X + LF_PITCH * 64 * 4;       // scratch of the inverse
constexpr int OFF_CUM = OFF_TP;
// Result tiles of a chunk, written by the last epilogue over slabs whose products are done and that no copy to the
// residual reads (V, and G = W~), and sent to global memory by bulk copies: the 64 output rows as [64][128 bytes]
// with the 128-byte swizzle of the tiled copy (piece index XOR row mod 8), and M' as 8 column blocks of [64 rows]
// [16 bytes], the layout of the saved tiles.
constexpr int OFF_YT = (OFF_V + 1023) / 1024 * 1024;
constexpr int OFF_MT = OFF_YT + kC * kN * 2;
constexpr int OFF_RT = (OFF_BH + 1023) / 1024 * 1024;   // P_rb W~ (token rows, swizzled like the outputs) over B^, K^
static_assert(OFF_RT + kC * kN * 2 <= OFF_SA, "the P_rb W~ tile must lie over B^ and K^");
static_assert(OFF_MT + GTILE <= OFF_M2A + SLAB64, "result tiles must lie over V and G");
// Staging tiles for the raw rows of the NEXT chunk (6 streams x 64 tokens x 128 bytes), filled by tiled
// bulk copies once the inverse is done: tiles 0..4 over AR + BK + S0, tile 5 over the P_rk half of M2A.
constexpr int STG_TILE = kC * kN * 2;
static_assert(5 * STG_TILE <= 2 * SLAB128 + SLAB64 && STG_TILE <= SLAB128 - SLAB64, "staging tiles must fit their hosts");
__device__ __forceinline__ int stage_off(int m) { return m < 5 ? OFF_AR + m * STG_TILE : OFF_M2A + SLAB64; }
struct Small {
    float h1[kN];        // cumulative log-decay of tokens 0..31, stored [e][jb] for channel 8 jb + e
    float tot[kN];       // ... of the whole chunk
    float lam[kN];       // exp(tot)
    float lamt[kN];      // the same, stored [e][jb]
    uint64_t bar[5];   // 0..3 product rounds, 4 staging tiles
    uint32_t nsm[2];
    uint32_t tmem;
};
constexpr int SMEM_BYTES = OFF_SMALL + (int)sizeof(Small);
static_assert(OFF_SCR + TRI_SCR_FLOATS * 4 <= OFF_BH, "inverse work space must fit over AR+BK+S0");
static_assert(2 * (SMEM_BYTES + 1024) <= 228 * 1024, "two CTAs per SM");

// four K=16 steps (64 deep) of D (+)= A B
__device__ __forceinline__ void mma_k64(uint32_t d, Op a, Op b, uint32_t idesc, bool accumulate) {
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) tc::mma(d, op_desc(a, ks), op_desc(b, ks), idesc, accumulate || ks > 0);
}

__device__ int g_status;  // last device-side error (0 = none); see wkv7_chunk_status()


// 256 threads: warp = (quad, hsel); quad selects the 32 TMEM lanes (tile rows) the warp may access,
// hsel the column half it works on, so every accumulator tile is shared by two warps per row group.
__global__ void __launch_bounds__(256, 2)
wkv7_chunk_fwd_kernel(int Tlen, int H, const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ r,
                      const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                      const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                      const __nv_bfloat16* __restrict__ s0, const uint32_t* __restrict__ length,
                      const uint8_t* __restrict__ new_starts, __nv_bfloat16* __restrict__ y,
                      __nv_bfloat16* __restrict__ s_out, float* __restrict__ ckpt, float* __restrict__ s_at_len,
                      const __grid_constant__ StreamMaps maps, const __grid_constant__ CUtensorMap y_map, const __grid_constant__ CUtensorMap rbar_map,
                      unsigned char* __restrict__ saved,
                      int* __restrict__ range_flag, int range_ticket, int* __restrict__ residual_mark,
                      __nv_bfloat16* __restrict__ mprime, __nv_bfloat16* __restrict__ rbar, float* __restrict__ lam_out,
                      int* __restrict__ fast_flag, int pieces) {
    extern __shared__ __align__(1024) unsigned char smem[];   // (the swizzle of the output tile is a function of the address)
    Small& sm = *reinterpret_cast<Small*>(smem + OFF_SMALL);
    // (all first pieces come first in the grid: where no cut exists the other pieces' CTAs return at once, and the
    // CTAs that do the work are then spread over the SMs before any SM takes a second one)
    const int n_seq = (int)gridDim.x / pieces;
    const int bh = blockIdx.x % n_seq, piece = blockIdx.x / n_seq, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = warp & 3, hsel = warp >> 2;
    const int row = quad * 32 + lane;
    const int L = min((int)length[bi], Tlen);
    // ---- sequence-parallel mode (pieces > 1, calls without a residual): a start flag cuts every dependence, so a
    // sequence may be walked as independent pieces whose first token carries a start flag.  Cut k, k = 1..pieces-1,
    // is the start flag nearest to k T / pieces within half a piece of it, if there is one; every CTA of the
    // sequence finds the same cuts by itself, a CTA whose own cut does not exist has nothing to do.
    int t_begin = 0, t_end = Tlen;
    if (pieces > 1) {
        const uint8_t* ns_row = new_starts + (size_t)bi * Tlen;
        const int half = Tlen / (2 * pieces);
        auto find_cut = [&](int k) -> int {       // position of cut k, or -1; all threads of the CTA take part
            const int target = (int)((long long)k * Tlen / pieces);
            const int lo = max(target - half, 1), hi = min(target + half, Tlen);
            __syncthreads();
            if (tid == 0) sm.nsm[0] = 0xffffffffu;
            __syncthreads();
            for (int t = lo + tid; t < hi; t += blockDim.x)
                if (ns_row[t] != 0) atomicMin(&sm.nsm[0], (uint32_t)(abs(t - target) * 2 + (t > target ? 1 : 0)) << 16 | (uint32_t)(t - lo));
            __syncthreads();
            const uint32_t best = sm.nsm[0];
            return best == 0xffffffffu ? -1 : lo + (int)(best & 0xffffu);
        };
        if (piece > 0) {
            t_begin = find_cut(piece);
            if (t_begin < 0) return;              // (the decision is the same for every thread)
        }
        for (int k = piece + 1; k < pieces; ++k) {
            const int c = find_cut(k);
            if (c >= 0) { t_end = c; break; }
        }
        __syncthreads();
    }
    const size_t tok_stride = (size_t)H * kN;
    const size_t seq_base = (size_t)bi * Tlen * tok_stride + (size_t)h * kN;
    const size_t st_row = ((size_t)bh * kN + (row & 63)) * kN + hsel * 32;  // this thread's 32 state elements
    const int nBlk = (Tlen + kC - 1) / kC;

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < 5; ++i) tc::mbar_init(&sm.bar[i], (i == 2 || i == 3) ? 2 : 1);   // M3, M4: two issuing threads
        tc::mbar_init_fence();
        if (bh == 0 && residual_mark != nullptr) *residual_mark = 0;   // this residual is in the chunked format (so far)
    }
    if (warp == 0) tc::tmem_alloc(&sm.tmem, 256);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tbase = sm.tmem;
    const uint32_t lane_addr = tbase + ((uint32_t)(quad * 32) << 16);  // this warp's 32 TMEM lanes
    const uint32_t D1 = 0, D2 = 128, DS = 192;                        // TMEM column offsets (D3 aliases D1)
    bool failed = false;

    // ---- state into TMEM (rows 0..63 = S0 in fp32, rows 64..127 are never read) --------------
    {
        float s[32];
        if (row < 64 && t_begin == 0) {
#pragma unroll
            for (int c = 0; c < 4; ++c) unpack8(*reinterpret_cast<const uint4*>(s0 + st_row + c * 8), &s[c * 8]);
        } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) s[c] = 0.f;
        }
        tc::tmem_st32(lane_addr + DS + hsel * 32, s);
        tc::tmem_wait_st();
    }

    const uint32_t sAR = tc::smem_u32(smem + OFF_AR), sBK = tc::smem_u32(smem + OFF_BK);
    const uint32_t sBH = tc::smem_u32(smem + OFF_BH), sKH = tc::smem_u32(smem + OFF_KH);
    const uint32_t sSA = tc::smem_u32(smem + OFF_SA), sV = tc::smem_u32(smem + OFF_V);
    const uint32_t sM2A = tc::smem_u32(smem + OFF_M2A), sG = tc::smem_u32(smem + OFF_G);
    const uint32_t sTP = tc::smem_u32(smem + OFF_TP), sS0 = tc::smem_u32(smem + OFF_S0);
    constexpr uint32_t ID_128x128_KK = tc::make_idesc(128, 128, false, false);
    constexpr uint32_t ID_128x64_KK = tc::make_idesc(128, 64, false, false);
    constexpr uint32_t ID_128x64_KM = tc::make_idesc(128, 64, false, true);
    constexpr uint32_t ID_128x64_MM = tc::make_idesc(128, 64, true, true);

    float* cum = reinterpret_cast<float*>(smem + OFF_CUM);  // [64][LF_PITCH]
    float* lf = reinterpret_cast<float*>(smem + OFF_LF);    // [64][LF_PITCH]
    float* xinv = reinterpret_cast<float*>(smem + OFF_X);   // [64][LF_PITCH]
    float* scr = reinterpret_cast<float*>(smem + OFF_SCR);
    const int tsub = tid >> 3, jb = tid & 7;                // staging unit: tokens 32q+tsub (q=0,1), channels 8jb..8jb+7

    constexpr int kIssuer2 = 96;   // a thread of the warp with the least epilogue work
    int p = t_begin;
    bool all_saved = (saved != nullptr);   // every chunk so far was a full block with its operands saved
    uint32_t par = 0, spar = 0;   // phase parities of the product barriers and of the staging barrier
    // result tiles of the chunk just finished, waiting in shared memory for the next CTA barrier
    bool pend_y = false, pend_m = false;
    int pend_p = 0;
    size_t pend_slot = 0;
    auto send_tiles = [&]() {   // behind a CTA barrier that follows the epilogue's stores
        if (warp == 7 && lane == 0 && (pend_y || pend_m)) {
            if (pend_y) tc::tensor_store_2d(&y_map, h * kN, bi * Tlen + pend_p, smem + OFF_YT);
            if (pend_m) {
                tc::bulk_store(mprime + pend_slot * (kN * kN), smem + OFF_MT, GTILE);
                // R- = R~ + P_rb W~: added in bf16 onto the R~ rows that went to global memory when the operands were scaled
                tc::tensor_reduce_add_2d(&rbar_map, h * kN, bi * Tlen + pend_p, smem + OFF_RT);
            }
            tc::bulk_commit();
        }
        pend_y = pend_m = false;
    };
    uint8_t flag_ahead = (tid < 64 && t_begin + tid < Tlen) ? new_starts[(size_t)bi * Tlen + t_begin + tid] : 0;
    // the 64 token rows from cp on of w, r, k, v, a, b into the staging tiles (thread 0; one tiled copy
    // per stream).  Rows past the chunk arrive too and are ignored.
    auto issue_stage = [&](int cp) {
        if (tid == 0) {
            tc::mbar_expect_tx(&sm.bar[4], (uint32_t)(6 * STG_TILE));
#pragma unroll
            for (int m = 0; m < 6; ++m) tc::tensor_load_2d(smem + stage_off(m), &maps.m[m], h * kN, bi * Tlen + cp, &sm.bar[4]);
        }
    };
    issue_stage(t_begin);
    while (true) {
        // ================= boundary at position p: TMEM holds the state after token p-1 =================
        // (of the pieces of a sequence, the one that has walked token L - 1 holds it; L == 0: the first)
        const bool want_out = (p == L) && (p > t_begin || t_begin == 0);
        if (quad < 2 && want_out) {
            float s[32];
            tc::tmem_ld32(lane_addr + DS + hsel * 32, s);
            tc::tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(s_out + st_row + c * 8) = pack8(&s[c * 8]);
            if (s_at_len != nullptr) {
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<float4*>(s_at_len + st_row + c * 4) = make_float4(s[c * 4], s[c * 4 + 1], s[c * 4 + 2], s[c * 4 + 3]);
            }
        }
        if (p >= t_end) break;
        // ================= extent of this chunk =================
        const int be = min(((p >> 6) + 1) << 6, t_end);
        if (tid < 64) {
            // the flag byte of position p + tid was requested while the previous chunk's products ran
            const bool f = (p + tid < be) && (flag_ahead != 0);
            const uint32_t m = __ballot_sync(0xffffffffu, f);
            if (lane == 0) sm.nsm[warp] = m;
        }
        __syncthreads();   // nsm visible; previous chunk's shared-memory readers are done
        send_tiles();
        const uint64_t mask = (uint64_t)sm.nsm[0] | ((uint64_t)sm.nsm[1] << 32);
        const bool reset_here = (mask & 1ull) != 0;
        int p1 = be;
        if ((mask >> 1) != 0) p1 = p + __ffsll((long long)(mask >> 1));
        if (L > p && L < p1) p1 = L;
        const int n = p1 - p;
        // a block walked as one full chunk leaves its operand slabs T, A_ak, P_rb, P_rk, sa for the backward
        unsigned char* const keep = (saved != nullptr && n == kC && (p & (kC - 1)) == 0)
                                        ? saved + ((size_t)bh * nBlk + (p >> 6)) * kSavedBytes : nullptr;
        all_saved = all_saved && (keep != nullptr);
        const size_t blk_slot = (size_t)bh * nBlk + (p >> 6);
        // the fp32 state entering a block is only needed by a backward that recomputes the block's first chunk,
        // i.e. when that chunk is short; a full chunk passes its bf16 entering state with the saved slabs
        if (quad < 2 && ckpt != nullptr && (p & (kC - 1)) == 0 && n < kC) {
            float s[32];
            tc::tmem_ld32(lane_addr + DS + hsel * 32, s);
            tc::tmem_wait_ld();
            float* dst = ckpt + (((size_t)bh * nBlk + p / kC) * kN + row) * kN + hsel * 32;
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<float4*>(dst + c * 4) = make_float4(s[c * 4], s[c * 4 + 1], s[c * 4 + 2], s[c * 4 + 3]);
        }
        // ================= stage inputs (registers), log-decay into the scan buffer =================
        uint4 raw[2][5];   // r, k, v, a, b
        float lw[2][8];    // log2 of the decay: -exp(w) * log2(e)
        if (!tc::mbar_wait(&sm.bar[4], spar)) failed = true;   // the rows of this chunk have landed
        spar ^= 1u;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int t = q * 32 + tsub;
            if (t < n) {
                const int o = t * (kN * 2) + jb * 16;
                float wf[8];
                unpack8(*reinterpret_cast<const uint4*>(smem + stage_off(0) + o), wf);
#pragma unroll
                for (int m = 0; m < 5; ++m) raw[q][m] = *reinterpret_cast<const uint4*>(smem + stage_off(m + 1) + o);
#pragma unroll
                for (int e = 0; e < 8; ++e) lw[q][e] = -kLog2e * __expf(wf[e]);   // log2 of the decay
            } else {
#pragma unroll
                for (int m = 0; m < 5; ++m) raw[q][m] = make_uint4(0, 0, 0, 0);
#pragma unroll
                for (int e = 0; e < 8; ++e) lw[q][e] = 0.f;
            }
            // (column 4 jb + e holds channel 8 jb + e, column 32 + 4 jb + e channel 8 jb + 4 + e: the eight lanes of a
            // token then write, and later read, 128 contiguous bytes)
            *reinterpret_cast<float4*>(&cum[t * LF_PITCH + jb * 4]) = make_float4(lw[q][0], lw[q][1], lw[q][2], lw[q][3]);
            *reinterpret_cast<float4*>(&cum[t * LF_PITCH + 32 + jb * 4]) = make_float4(lw[q][4], lw[q][5], lw[q][6], lw[q][7]);
        }
        __syncthreads();
        if (tid < 128) {   // inclusive scan over tokens, two independent halves of 32 per channel
            const int j = tid & 63, half = tid >> 6;
            float run = 0.f;
#pragma unroll 8
            for (int tt = 0; tt < 32; ++tt) {
                const int t = half * 32 + tt;
                run += cum[t * LF_PITCH + j];
                cum[t * LF_PITCH + j] = run;
            }
            // column j of the scan buffer is channel ch = 8 jb + e
            const int cjb = (j & 31) >> 2, ce = (j & 3) + ((j >> 5) << 2), ch = cjb * 8 + ce;
            if (half == 0) sm.h1[ce * 8 + cjb] = run;
            else sm.tot[ch] = run;   // second-half sum for now
        }
        __syncthreads();
        if (tid < 64) {
            const float total = sm.h1[(tid & 7) * 8 + (tid >> 3)] + sm.tot[tid];
            // A decay so strong that 1 / L leaves the range the products can carry (never reached by decays
            // of the model's own parametrisation): the chunked form cannot represent this chunk.  Record it;
            // the token-sequential kernel launched behind this one redoes the call when it finds the mark.
            if (total < kCumFloor) atomicExch(range_flag, range_ticket);
            const float t2 = fmaxf(total, kCumFloor);
            sm.tot[tid] = t2;
            const float lam_c = ex2(t2);
            sm.lam[tid] = lam_c;
            sm.lamt[(tid & 7) * 8 + (tid >> 3)] = lam_c;
        }
        if (warp == 7) tc::bulk_wait_read<0>();   // the result tiles have left the slabs that are written next
        __syncthreads();
        // ================= scaled operands into the slabs =================
        {
            float h1v[8], lamv[8];   // first-half totals; 2^(chunk total) per channel
#pragma unroll
            for (int e = 0; e < 8; ++e) { h1v[e] = sm.h1[e * 8 + jb]; lamv[e] = sm.lamt[e * 8 + jb]; }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int t = q * 32 + tsub;
                float c[8];
                *reinterpret_cast<float4*>(&c[0]) = *reinterpret_cast<const float4*>(&cum[t * LF_PITCH + jb * 4]);
                *reinterpret_cast<float4*>(&c[4]) = *reinterpret_cast<const float4*>(&cum[t * LF_PITCH + 32 + jb * 4]);
                float eL[8], eI[8], eP[8], eE[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float cc = fmaxf(c[e] + (q == 1 ? h1v[e] : 0.f), kCumFloor);
                    const float cp = fminf(fmaxf(cc - lw[q][e], kCumFloor), 0.f);   // cumulative log2-decay before this token
                    eL[e] = ex2(cc); eI[e] = ex2(-cc); eP[e] = ex2(cp);
                    eE[e] = lamv[e] * eI[e];   // 2^(total - cc) without a fourth trip to the special-function unit
                }
                // raw: r, k, v, a, b
                const uint4 a_t = scale8(raw[q][3], eP), r_t = scale8(raw[q][0], eL);
                slab_store(smem + OFF_AR, CB128, t, jb, a_t);
                slab_store(smem + OFF_AR, CB128, 64 + t, jb, r_t);
                if (keep != nullptr) {
                    // W~ = T A~ is formed after the inverse, when the [A~ ; R~] slab has long been written over:
                    // a second copy of A~ waits in the sa slab, which is idle until sa itself is stored; R~ goes
                    // to the R- rows in global memory, where P_rb W~ is added at the end of the chunk
                    slab_store(smem + OFF_SA, CB64, t, jb, a_t);
                    *reinterpret_cast<uint4*>(rbar + seq_base + (size_t)(p + t) * tok_stride + jb * 8) = r_t;
                    tc::fence_async_global();   // a bulk copy adds onto these rows at the end of the chunk
                }
                slab_store(smem + OFF_BK, CB128, t, jb, scale8(raw[q][4], eI));
                slab_store(smem + OFF_BK, CB128, 64 + t, jb, scale8(raw[q][1], eI));
                slab_store(smem + OFF_BH, CB64, t, jb, scale8(raw[q][4], eE));
                slab_store(smem + OFF_KH, CB64, t, jb, scale8(raw[q][1], eE));
                slab_store(smem + OFF_V, CB64, t, jb, raw[q][2]);
            }
        }
        // ================= entering state: bf16 copy for the products, decayed fp32 copy back to TMEM =====
        if (quad < 2) {
            float s[32];
            if (reset_here) {
#pragma unroll
                for (int c = 0; c < 32; ++c) s[c] = 0.f;
            } else {
                tc::tmem_ld32(lane_addr + DS + hsel * 32, s);
                tc::tmem_wait_ld();
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) slab_store(smem + OFF_S0, CB64, row, hsel * 4 + c, pack8(&s[c * 8]));
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 l4 = *reinterpret_cast<const float4*>(&sm.lam[hsel * 32 + c * 4]);
                s[c * 4] *= l4.x; s[c * 4 + 1] *= l4.y; s[c * 4 + 2] *= l4.z; s[c * 4 + 3] *= l4.w;
            }
            tc::tmem_st32(lane_addr + DS + hsel * 32, s);
            tc::tmem_wait_st();
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        // ================= M1: pairwise products and the S0 products =================
        if (tid == 0) {
            tc::fence_after_sync();
            mma_k64(tbase + D1, kmaj128(sAR), kmaj128(sBK), ID_128x128_KK, false);
            mma_k64(tbase + D2, kmaj128(sAR), kmaj64(sS0), ID_128x64_KK, false);
            tc::commit(&sm.bar[0]);
        }
        if (keep != nullptr && warp == 7 && lane < 8) {   // the bf16 entering state goes to the residual as it is
            tc::bulk_store(keep + (size_t)SAVED_S0 * GTILE + lane * GCB, smem + OFF_S0 + lane * CB64, 64 * 16);
            tc::bulk_commit();
        }
        if (keep != nullptr && tid < 64) lam_out[blk_slot * kN + tid] = sm.lam[tid];
        if (!tc::mbar_wait(&sm.bar[0], par)) failed = true;
        tc::fence_after_sync();
        // ================= E1: triangular masks, operands of the next products =================
        {
            const int t = row & 63;
            float d[64];
            tc::tmem_ld32(lane_addr + D1 + hsel * 64, d);
            tc::tmem_ld32(lane_addr + D1 + hsel * 64 + 32, d + 32);
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
                // A_ak -> M2A rows 0..63, P_rk -> M2A rows 64..127, P_rb -> TP rows 64..127
                unsigned char* dst = smem + ((hsel == 1) ? OFF_M2A : OFF_TP);
#pragma unroll
                for (int c = 0; c < 8; ++c) slab_store(dst, CB128, row, c, pack8(&d[c * 8]));
            }
        }
        if (warp == 7) tc::bulk_wait_read<0>();   // the S0 slab has been read: the inverse writes over part of it next
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        // ================= M2: G += A_ak V, Ypart += P_rk V ; meanwhile the triangular inverse =================
        if (tid == 0) {
            tc::fence_after_sync();
            mma_k64(tbase + D2, kmaj128(sM2A), mnmaj64(sV), ID_128x64_KM, true);
            tc::commit(&sm.bar[1]);
        }
        // A_ak, P_rk and P_rb leave for the residual as bulk copies out of their slabs (one 64-row column
        // block of 1 KB per lane of the last warp); the copies must have read M2A before G is written over it,
        // which the hook in front of the inverse's last barrier guarantees
        if (keep != nullptr && warp == 7 && lane < 24) {
            const int which = lane >> 3, c = lane & 7;   // 0: A_ak, 1: P_rk, 2: P_rb
            const unsigned char* src = smem + (which == 2 ? OFF_TP : OFF_M2A) + c * CB128 + (which == 0 ? 0 : 64 * 16);
            unsigned char* dst = keep + (size_t)(which == 0 ? SAVED_AAK : (which == 1 ? SAVED_PRK : SAVED_PRB)) * GTILE + c * GCB;
            tc::bulk_store(dst, src, 64 * 16);
            tc::bulk_commit();
        }
        tri_inverse_64<256>(lf, xinv, scr, tid, [&]() { if (warp == 7) tc::bulk_wait_read<0>(); });
        fp32_to_slab64<256>(xinv, smem + OFF_TP, CB128, tid);
        if (quad < 2) {
            if (!tc::mbar_wait(&sm.bar[1], par)) failed = true;
            tc::fence_after_sync();
            float g[32];
            tc::tmem_ld32(lane_addr + D2 + hsel * 32, g);
            tc::tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) slab_store(smem + OFF_G, CB64, row, hsel * 4 + c, pack8(&g[c * 8]));
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (keep != nullptr && warp == 7 && lane < 8) {   // T: rows 0..63 of the [Tinv ; P_rb] slab
            tc::bulk_store(keep + (size_t)SAVED_T * GTILE + lane * GCB, smem + OFF_TP + lane * CB128, 64 * 16);
            tc::bulk_commit();
        }
        // ================= M3: sa = Tinv G =================
        if (tid == 0) {
            tc::fence_after_sync();
            mma_k64(tbase + D1, kmaj128(sTP), mnmaj64(sG), ID_128x64_KM, false);
            tc::commit(&sm.bar[2]);
        } else if (tid == kIssuer2) {   // what only the backward's carry needs is issued by a second thread
            tc::fence_after_sync();
            if (keep != nullptr) mma_k64(tbase + D1 + 64, kmaj128(sTP), mnmaj64(sSA), ID_128x64_KM, false);   // W~ = Tinv A~
            tc::commit(&sm.bar[2]);
        }
        // the rows of the next chunk start travelling: their tiles lie over buffers that are idle from
        // here to the next chunk's operand stores (the inverse and the A_ak / P_rk product are done)
        if (p1 < t_end) issue_stage(p1);
        if (quad < 2) {
            if (!tc::mbar_wait(&sm.bar[2], par)) failed = true;
            tc::fence_after_sync();
            float sa[32];
            tc::tmem_ld32(lane_addr + D1 + hsel * 32, sa);
            tc::tmem_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) slab_store(smem + OFF_SA, CB64, row, hsel * 4 + c, pack8(&sa[c * 8]));
            if (keep != nullptr) {
                tc::tmem_ld32(lane_addr + D1 + 64 + hsel * 32, sa);
                tc::tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(smem + OFF_G, CB64, row, hsel * 4 + c, pack8(&sa[c * 8]));
            }
        }
        tc::fence_async_smem();
        tc::fence_before_sync();
        __syncthreads();
        if (keep != nullptr && warp == 7 && lane < 8) {   // sa
            tc::bulk_store(keep + (size_t)SAVED_SA * GTILE + lane * GCB, smem + OFF_SA + lane * CB64, 64 * 16);
            tc::bulk_commit();
        }
        // ================= M4: Y += P_rb sa ; S += sa^T B^ + V^T K^ =================
        if (tid == 0) {
            tc::fence_after_sync();
            mma_k64(tbase + D2, kmaj128(sTP), mnmaj64(sSA), ID_128x64_KM, true);
            mma_k64(tbase + DS, mnmaj64(sSA), mnmaj64(sBH), ID_128x64_MM, true);
            mma_k64(tbase + DS, mnmaj64(sV), mnmaj64(sKH), ID_128x64_MM, true);
            tc::commit(&sm.bar[3]);
        } else if (tid == kIssuer2) {
            tc::fence_after_sync();
            if (keep != nullptr) {
                // the transition's off-diagonal part M' = W~^T B^ (rows 0..63 of the accumulator are used) and
                // the state-dependent part of the outputs, P_rb W~ (rows 64..127)
                mma_k64(tbase + D1, mnmaj64(sG), mnmaj64(sBH), ID_128x64_MM, false);
                mma_k64(tbase + D1 + 64, kmaj128(sTP), mnmaj64(sG), ID_128x64_KM, false);
            }
            tc::commit(&sm.bar[3]);
        }
        if (tid < 64) flag_ahead = (p1 + tid < Tlen) ? new_starts[(size_t)bi * Tlen + p1 + tid] : 0;   // next chunk's start flags
        if (!tc::mbar_wait(&sm.bar[3], par)) failed = true;
        tc::fence_after_sync();
        if (quad >= 2) {
            const int t = row - 64;
            float yv[32];
            tc::tmem_ld32(lane_addr + D2 + hsel * 32, yv);
            tc::tmem_wait_ld();
            if (n == kC) {        // a full block leaves as one tiled copy out of shared memory
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(smem + OFF_YT + t * 128 + (((hsel * 4 + c) ^ (t & 7)) << 4)) = pack8(&yv[c * 8]);
            } else if (t < n) {
                __nv_bfloat16* dst = y + seq_base + (size_t)(p + t) * tok_stride + hsel * 32;
#pragma unroll
                for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = pack8(&yv[c * 8]);
            }
        }
        pend_y = (n == kC);
        pend_p = p;
        pend_m = (keep != nullptr);
        pend_slot = blk_slot;
        if (keep != nullptr) {
            float m[32];
            if (quad < 2) {       // M'[j][j'], row j = this thread's lane
                tc::tmem_ld32(lane_addr + D1 + hsel * 32, m);
                tc::tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c) slab_store(smem + OFF_MT, GCB, row, hsel * 4 + c, pack8(&m[c * 8]));
            } else {              // R-_t = R~_t + (P_rb W~)_t on top of the R~ row stored at the start of the chunk
                const int t = row - 64;
                tc::tmem_ld32(lane_addr + D1 + 64 + hsel * 32, m);
                tc::tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4*>(smem + OFF_RT + t * 128 + (((hsel * 4 + c) ^ (t & 7)) << 4)) = pack8(&m[c * 8]);
            }
        }
        tc::fence_async_smem();   // the result tiles are read by bulk copies
        tc::fence_before_sync();
        if (warp == 7) tc::bulk_wait_read<0>();   // the slabs copied out may be rewritten after the next barrier
        p = p1;
        par ^= 1u;
    }
    __syncthreads();
    send_tiles();   // of the last chunk
    if (fast_flag != nullptr && tid == 0) fast_flag[bh] = all_saved ? 1 : 0;
    if (warp == 7) tc::bulk_wait_all<0>();   // every copy to the residual has landed before the CTA retires
    if (failed) atomicExch(&g_status, 1);
    tc::fence_before_sync();
    __syncthreads();
    if (warp == 0) tc::tmem_dealloc(tbase, 256);
}

}  // namespace

size_t wkv7_chunk_residual_bytes(int B, int T, int H) { return chunk_residual_floats(B, T, H) * sizeof(float); }

// A forward call that meets a decay outside the chunked kernels' range tells the fallback launched behind
// it through one int of device memory.  Calls may be in flight on several streams, so each call takes the
// next slot of a small ring and a ticket that no earlier call used: a slot never needs clearing.
__device__ int g_range_flags[64];

static int* range_flag_ring() {
    static DeviceOnce once;
    static int* addr[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return nullptr;
    if (!once.ok([dev]() {
            int* ptr = nullptr;
            const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_range_flags);
            addr[dev] = (e == cudaSuccess) ? ptr : nullptr;
            return e;
        }))
        return nullptr;
    return addr[dev];
}

// A slot of the ring and a ticket no earlier call used (never 0, so untouched memory cannot match); NULL on failure.
int* wkv_call_flag(int* ticket) {
    static std::atomic<unsigned> tickets{1};
    int* ring = range_flag_ring();
    if (ring == nullptr) return nullptr;
    const unsigned t = tickets.fetch_add(1);
    *ticket = (int)(t | 0x40000000u);
    return ring + (t & 63u);
}

int wkv7_chunk_fwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                   const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                   void* s_out, void* residual, int* residual_mark, int** range_flag, int* range_ticket) {
    typedef __nv_bfloat16 bf;
    static DeviceOnce smem_attr;   // the opt-in to large dynamic shared memory is a per-device function attribute
    if (!smem_attr.ok([]() { return cudaFuncSetAttribute(wkv7_chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); }))
        return B200WKV_ELAUNCH;
    *range_flag = wkv_call_flag(range_ticket);
    if (*range_flag == nullptr) return B200WKV_ELAUNCH;
    const CarryLayout lay = carry_layout(B, T, H);
    StreamMaps maps;
    const void* bases[6] = {w, r, k, v, a, b};   // maps[m]: the six streams as [B*T tokens][H*64 channels]
    if (!make_stream_maps(&maps, bases, 6, B, T, H)) return B200WKV_ELAUNCH;
    StreamMaps out_maps;                         // m[0]: the outputs, with the 128-byte swizzle of the kernel's output tile
    const void* out_bases[2] = {y, residual ? (const void*)((char*)residual + lay.rbar) : y};   // m[1]: the R- rows
    if (!make_stream_maps(&out_maps, out_bases, 2, B, T, H, /*swizzle128=*/true)) return B200WKV_ELAUNCH;
    // Without a residual (inference) and with fewer sequences than CTA slots, every sequence is offered to several
    // CTAs, which cut it at start flags where there are any (see the kernel): at most 8 pieces of at least 128 tokens.
    int pieces = 1;
    if (residual == nullptr) {
        const long long slots = 2LL * sm_count_of_current_device();
        const long long seqs = (long long)B * H;
        if (seqs < slots) pieces = (int)((2 * slots + seqs - 1) / seqs);
        if (pieces > 8) pieces = 8;
        if (pieces > T / 128) pieces = T / 128;
        if (pieces < 1 || T / pieces >= 32768) pieces = 1;
    }
    wkv7_chunk_fwd_kernel<<<B * H * pieces, 256, SMEM_BYTES, st>>>(T, H, (const bf*)w, (const bf*)r, (const bf*)k, (const bf*)v,
                                                          (const bf*)a, (const bf*)b, (const bf*)s0, length, ns,
                                                          (bf*)y, (bf*)s_out, (float*)residual,
                                                          residual ? (float*)residual + (size_t)B * H * ((T + kC - 1) / kC) * kN * kN : nullptr,
                                                          maps, out_maps.m[0], out_maps.m[1],
                                                          residual ? (unsigned char*)((float*)residual + chunk_saved_offset_floats(B, T, H)) : nullptr,
                                                          *range_flag, *range_ticket, residual_mark,
                                                          residual ? (bf*)((char*)residual + lay.mprime) : nullptr,
                                                          residual ? (bf*)((char*)residual + lay.rbar) : nullptr,
                                                          residual ? (float*)((char*)residual + lay.lam) : nullptr,
                                                          residual ? (int*)((char*)residual + lay.fast) : nullptr, pieces);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

// Device address of the status word on the current device (resolved once per device).
int* wkv7_chunk_status_word() {
    static DeviceOnce once;
    static int* addr[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return nullptr;
    if (!once.ok([dev]() {
            int* ptr = nullptr;
            const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_status);
            addr[dev] = (e == cudaSuccess) ? ptr : nullptr;
            return e;
        }))
        return nullptr;
    return addr[dev];
}

// Reads and clears the device-side error word (synchronises the device; diagnostics only).
int wkv7_chunk_status() {
    int h = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&h, g_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return h;
}

}  // namespace b200wkv

// Constants and small helpers shared by the chunked (tcgen05) forward and backward kernels.
#pragma once
#include "common.cuh"
#include "device_once.cuh"

namespace b200wkv {

constexpr int kC = 64;                 // tokens per full chunk == checkpoint spacing
constexpr int CB64 = 1040;             // column-block pitch of a 64-row operand slab (64*16 + 16 pad)
constexpr int CB128 = 2064;            // ... of a 128-row slab
constexpr int SLAB64 = 8 * CB64;       // 8320
constexpr int SLAB128 = 8 * CB128;     // 16512
constexpr int LF_PITCH = 68;           // floats per row of fp32 matrices kept in shared memory
constexpr float kCumFloor = -86.56f;   // floor of the in-chunk cumulative log2-decay (= -60 in natural log; keeps 1/L finite)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// Residual written by the chunked forward for the chunked backward (all fp32):
//   [B*H][ceil(T/64)][64][64]  state entering every 64-token block (before a start flag is applied)
//   [B*H][64][64]              state at position `length` (what the forward returns as s_out)
//   [kHandoffSlots][64*64 + 64] carries passed between CTAs that share one (batch, head) sequence
//   [kHandoffSlots]             their ready flags (int)
// The last two are scratch of whichever kernel runs: a sequence may be cut at 64-token block
// boundaries into runs owned by neighbouring CTAs, so that B*H sequences spread evenly over the SMs.
constexpr int kHandoffSlots = 512;
constexpr int kHandoffFloats = kN * kN + kN;
inline size_t chunk_states_floats(int B, int T, int H) {
    return (size_t)B * H * ((size_t)((T + kC - 1) / kC) + 1) * kN * kN;
}
//   [B*H][ceil(T/64)][6 tiles]  for every 64-token block that the forward walked as ONE chunk: the bf16
//                               operands T = (I - A_ab)^-1, A_ak, P_rb, P_rk, sa and the entering state S0
//                               exactly as the forward used them, so the backward loads them instead of
//                               recomputing them.  A tile is 8 column blocks of [64 rows][16 bytes] (the
//                               operand slab layout without the shared-memory padding), 8 KB.
constexpr int kSavedSlabs = 6;   // order: T, A_ak, P_rb, P_rk, sa, S0
constexpr int SAVED_T = 0, SAVED_AAK = 1, SAVED_PRB = 2, SAVED_PRK = 3, SAVED_SA = 4, SAVED_S0 = 5;
constexpr int GCB = kC * 16;          // column-block pitch of a tile in global memory (1024)
constexpr int GTILE = 8 * GCB;        // 8192
constexpr size_t kSavedBytes = (size_t)kSavedSlabs * GTILE;
inline size_t chunk_saved_offset_floats(int B, int T, int H) {
    return chunk_states_floats(B, T, H) + (size_t)kHandoffSlots * (kHandoffFloats + 1);
}
// What the carry / gradient split of the backward adds behind the saved tiles (see wkv7_carry.cu, wkv7_grad.cu):
//   [B*H][ceil(T/64)][64][64] bf16  M' = W~^T B^ of every saved block: S_C = S0 diag(L_C) + S0 M' + (terms without S0)
//                                   (8 column blocks of [64 rows][16 bytes], like the saved tiles)
//   [B*T][H*64]               bf16  R- = R~ + P_rb W~ (token rows, laid out like the streams): y_t = R-_t S0^T + ...
//   [B*H][ceil(T/64)][64]     fp32  L_C, the decay over the whole block
//   [B*H][ceil(T/64)][64][64] bf16  scratch of the backward: the state gradient leaving every block (column blocks, as M')
//   [B*H]                     int   1 if the forward walked the whole sequence as full, saved blocks
//   [kGradCtas][4][64][64]    bf16  scratch of the gradient kernel, one set per CTA: the decay factors 1/L_t, L_t,
//                                   L_{t-1} and the log-decay of the block in hand (written when the operands are
//                                   scaled, read back by the last epilogue; it lives in L2)
constexpr int kGradCtas = 512;
struct CarryLayout {
    size_t mprime, rbar, lam, dstate, fast, fscr, end;   // byte offsets from the start of the residual
};
inline CarryLayout carry_layout(int B, int T, int H) {
    const size_t nBlk = (size_t)((T + kC - 1) / kC), BH = (size_t)B * H;
    CarryLayout l;
    l.mprime = (chunk_saved_offset_floats(B, T, H)) * sizeof(float) + BH * nBlk * kSavedBytes;
    l.rbar = l.mprime + BH * nBlk * GTILE;
    l.lam = l.rbar + (size_t)B * nBlk * kC * H * kN * 2;      // token rows padded to whole blocks
    l.dstate = l.lam + BH * nBlk * kN * sizeof(float);
    l.fast = l.dstate + BH * nBlk * GTILE;
    l.fscr = (l.fast + BH * sizeof(int) + 255) / 256 * 256;
    const size_t ctas = BH * nBlk < (size_t)kGradCtas ? BH * nBlk : (size_t)kGradCtas;
    l.end = l.fscr + ctas * 4 * GTILE;
    return l;
}
inline size_t chunk_residual_floats(int B, int T, int H) { return carry_layout(B, T, H).end / sizeof(float); }

// Host side of the split: grid size and segments per sequence for `chains` sequences of `n_blk`
// blocks with `per_sm` resident CTAs per SM on a device of `sm_count` SMs (the launchers pass the
// count of the device that is current, looked up once per device).
struct SplitPlan {
    int grid;
    int seg;
};
inline SplitPlan plan_split(int chains, int n_blk, int per_sm, int sm_count) {
    const int slots = sm_count * per_sm;
    SplitPlan p{chains, 1};
    if (chains <= slots) return p;            // every sequence gets its own resident CTA
    p.grid = slots;
    if (chains % slots == 0 || slots > kHandoffSlots) return p;
    // makespan in sequence lengths is ceil(chains * seg / slots) / seg: take the smallest seg that helps
    double best = (double)((chains + slots - 1) / slots);
    for (int seg = 2; seg <= 8 && seg <= n_blk; seg *= 2) {
        const double m = (double)(((long long)chains * seg + slots - 1) / slots) / seg;
        if (m < best * 0.98) {
            best = m;
            p.seg = seg;
        }
    }
    return p;
}

// Work split of U = (sequences x segments) units over G CTAs: CTA c owns units [U c / G, U (c+1) / G).
// Units are numbered sequence-major; the consecutive units of one sequence inside a CTA's range form
// a run that the CTA walks as one piece.  A CTA whose range ends inside a sequence walks that run
// FIRST and hands its carry to the next CTA (slot c); the run at the start of its range that begins
// inside a sequence comes LAST and takes the carry of slot c - 1.  No CTA waits before it has
// produced what its neighbour needs, so the waits cannot form a cycle.
struct RunPlan {
    int chain;      // sequence index (batch * H + head)
    int seg_from;   // first segment of the run, in walking order
    int seg_to;     // one past the last segment
};
__host__ __device__ __forceinline__ int run_count(long long lo, long long hi, int seg) { return (int)((hi - 1) / seg - lo / seg) + 1; }
__host__ __device__ __forceinline__ RunPlan run_at(long long lo, long long hi, int seg, int order) {
    const int first = (int)(lo / seg), n = run_count(lo, hi, seg);
    // walking order: the last run of the range, the middle runs, the first run of the range
    const int ri = (n == 1) ? 0 : (order == 0 ? n - 1 : (order == n - 1 ? 0 : order));
    RunPlan r;
    r.chain = first + ri;
    r.seg_from = (ri == 0) ? (int)(lo % seg) : 0;
    r.seg_to = (ri == n - 1) ? (int)((hi - 1) % seg) + 1 : seg;
    return r;
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


// One warp: C(16x8) = A(16xK) B(Kx8), all fp32 row-major in shared memory; only k in [k_from, k_to) (multiples
// of 8) is walked, for operands that are known to be zero outside that range.
__device__ __forceinline__ void tile_mma_tf32(const float* A, int lda, const float* B, int ldb, float* C, int ldc,
                                              int k_from, int k_to, int lane) {
    const int g = lane >> 2, t = lane & 3;
    float c0 = 0.f, c1 = 0.f, c2 = 0.f, c3 = 0.f;
    for (int k0 = k_from; k0 < k_to; k0 += 8) {
        const uint32_t a0 = __float_as_uint(A[g * lda + k0 + t]), a1 = __float_as_uint(A[(g + 8) * lda + k0 + t]);
        const uint32_t a2 = __float_as_uint(A[g * lda + k0 + t + 4]), a3 = __float_as_uint(A[(g + 8) * lda + k0 + t + 4]);
        const uint32_t b0 = __float_as_uint(B[(k0 + t) * ldb + g]), b1 = __float_as_uint(B[(k0 + t + 4) * ldb + g]);
        asm volatile(
            "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
    *reinterpret_cast<float2*>(&C[g * ldc + 2 * t]) = make_float2(c0, c1);
    *reinterpret_cast<float2*>(&C[(g + 8) * ldc + 2 * t]) = make_float2(c2, c3);
}

// ---------------------------------------------------------------------------------------------
// X = (I - L)^-1 for a 64x64 strictly lower triangular L, by all NT threads of the CTA, in fp32.
// L and X are row-major with LF_PITCH floats per row; scr holds 32 x TRI_SCR_PITCH floats.
// Recursive blocking: the four 16x16 diagonal blocks by forward substitution, then
// X21 = X22 (L21 X11) for the two 32x32 blocks and once more for the whole matrix (these products
// on the warp-level tensor path in tf32).
// Every thread must call it (it synchronises the CTA); X is complete when it returns.
constexpr int TRI_SCR_PITCH = 36;
constexpr int TRI_SCR_FLOATS = 32 * TRI_SCR_PITCH;

struct NoHook {
    __device__ __forceinline__ void operator()() const {}
};
// `before_last_barrier` runs in every thread just ahead of the final CTA barrier (a place to retire
// asynchronous work that must be ordered before what the caller does next).
template <int NT, typename Hook = NoHook>
__device__ __forceinline__ void tri_inverse_64(const float* __restrict__ L, float* __restrict__ X,
                                               float* __restrict__ scr, int tid, Hook before_last_barrier = Hook()) {
    // The 16- and 32-wide stages involve only the first four warps, which meet at a named barrier of their
    // own; the other warps go straight to the CTA barrier in front of the 64-wide merge, so whatever they
    // still have to do (issuing bulk copies, say) does not hold the first stages up.
    // ---- diagonal blocks (threads 0..63) and zero fill of the blocks above the diagonal (threads 64..127)
    if (tid < 64) {
        const int d = tid >> 4, c = tid & 15, o = d * 16;
        float x[16];
#pragma unroll
        for (int t = 0; t < 16; ++t) x[t] = 0.f;
        // L is strictly lower: row t needs its first t entries only (whole groups of four are loaded or left out;
        // x[m] is still zero for m >= t).  The loads do not depend on x and can be issued ahead.
#pragma unroll
        for (int t = 0; t < 16; ++t) {
            const float4* lr = reinterpret_cast<const float4*>(&L[(o + t) * LF_PITCH + o]);
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            const float4 l0 = (t > 0) ? lr[0] : zero4, l1 = (t > 4) ? lr[1] : zero4, l2 = (t > 8) ? lr[2] : zero4, l3 = (t > 12) ? lr[3] : zero4;
            float a0 = (t == c) ? 1.f : 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
            a0 = fmaf(l0.x, x[0], a0); a1 = fmaf(l0.y, x[1], a1); a2 = fmaf(l0.z, x[2], a2); a3 = fmaf(l0.w, x[3], a3);
            a0 = fmaf(l1.x, x[4], a0); a1 = fmaf(l1.y, x[5], a1); a2 = fmaf(l1.z, x[6], a2); a3 = fmaf(l1.w, x[7], a3);
            a0 = fmaf(l2.x, x[8], a0); a1 = fmaf(l2.y, x[9], a1); a2 = fmaf(l2.z, x[10], a2); a3 = fmaf(l2.w, x[11], a3);
            a0 = fmaf(l3.x, x[12], a0); a1 = fmaf(l3.y, x[13], a1); a2 = fmaf(l3.z, x[14], a2); a3 = fmaf(l3.w, x[15], a3);
            x[t] = (a0 + a1) + (a2 + a3);
        }
#pragma unroll
        for (int t = 0; t < 16; ++t) X[(o + t) * LF_PITCH + o + c] = x[t];
    } else if (tid < 128) {
        for (int idx = tid - 64; idx < 6 * 256; idx += 64) {
            const int blk = idx >> 8, e = idx & 255;
            // blocks (bi, bj) with bj > bi: (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
            const int bi = (blk < 3) ? 0 : (blk < 5 ? 1 : 2);
            const int bj = (blk < 3) ? blk + 1 : (blk < 5 ? blk - 1 : 3);
            X[(bi * 16 + (e >> 4)) * LF_PITCH + bj * 16 + (e & 15)] = 0.f;
        }
    }
    // ---- merges on the warp-level tensor path (m16n8k8, tf32 operands, fp32 accumulate): the result is
    // rounded to bf16 afterwards, so tf32's 11-bit mantissa costs nothing.  One 16x8 output tile per warp.
    const int warp = tid >> 5, lane = tid & 31;
    // 16 -> 32: W_q = L21 X11 for q = 0,1 (two 16x16 products = four tiles), then X21 = X22 W_q
    if (warp < 4) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int q = warp >> 1, n0 = (warp & 1) * 8, o = q * 32;
        // (X11 is lower triangular: its rows above n0 are zero in this column tile)
        tile_mma_tf32(L + (o + 16) * LF_PITCH + o, LF_PITCH, X + o * LF_PITCH + o + n0, LF_PITCH,
                      scr + (q * 16) * TRI_SCR_PITCH + n0, TRI_SCR_PITCH, n0, 16, lane);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        tile_mma_tf32(X + (o + 16) * LF_PITCH + o + 16, LF_PITCH, scr + (q * 16) * TRI_SCR_PITCH + n0, TRI_SCR_PITCH,
                      X + (o + 16) * LF_PITCH + o + n0, LF_PITCH, 0, 16, lane);
    }
    __syncthreads();
    // 32 -> 64: W = L21 X11 (32x32x32 = eight tiles), then X21 = X22 W
    static_assert(NT == 256, "the merges are laid out for eight warps");
    {
        const int m0 = (warp >> 2) * 16, n0 = (warp & 3) * 8;
        tile_mma_tf32(L + (32 + m0) * LF_PITCH, LF_PITCH, X + n0, LF_PITCH, scr + m0 * TRI_SCR_PITCH + n0, TRI_SCR_PITCH,
                      n0, 32, lane);
        __syncthreads();
        // (X22 is lower triangular: the rows of this tile end at column m0 + 15)
        tile_mma_tf32(X + (32 + m0) * LF_PITCH + 32, LF_PITCH, scr + n0, TRI_SCR_PITCH, X + (32 + m0) * LF_PITCH + n0,
                      LF_PITCH, 0, m0 + 16, lane);
    }
    before_last_barrier();
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

// 2^x on the special-function unit (the cumulative decays are kept in log2 units so that no
// multiply is needed in front of it)
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// eight bf16 values (one 16-byte slab entry) times eight fp32 factors, as four packed bf16x2 products
__device__ __forceinline__ uint4 scale8(uint4 raw, const float* f) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    uint4 out;
    uint32_t* o = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __nv_bfloat162 p = __hmul2(h[i], __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]));
        o[i] = *reinterpret_cast<const uint32_t*>(&p);
    }
    return out;
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// ---------------------------------------------------------------------------------------------
// Operand walks for tcgen05.mma over the slab layout.  A descriptor is 64 bits: the low word holds
// (address >> 4) and the leading-dimension offset, the high word the stride offset and the version,
// so stepping along K is one 32-bit add on the low word.
struct Op { uint32_t lo, hi, step16; };
__device__ __forceinline__ Op make_op(uint32_t addr, uint32_t step, uint32_t lbo, uint32_t sbo) {
    return {(addr >> 4) | ((lbo >> 4) << 16), (sbo >> 4) | (1u << 14), step >> 4};
}
__device__ __forceinline__ Op kmaj128(uint32_t a) { return make_op(a, 2 * CB128, CB128, 128); }   // rows = M/N, cols = K
__device__ __forceinline__ Op kmaj64(uint32_t a) { return make_op(a, 2 * CB64, CB64, 128); }
__device__ __forceinline__ Op mnmaj128(uint32_t a) { return make_op(a, 256, 128, CB128); }       // cols = M/N, rows = K
__device__ __forceinline__ Op mnmaj64(uint32_t a) { return make_op(a, 256, 128, CB64); }
__device__ __forceinline__ uint64_t op_desc(Op o, int ks) {
    return ((uint64_t)o.hi << 32) | (uint64_t)(o.lo + (uint32_t)ks * o.step16);
}

}  // namespace b200wkv

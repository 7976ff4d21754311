// RWKV-5 / 5.2 / 6 WKV recurrence in chunks of 16 tokens on the tensor cores (bf16 I/O, fp32 state).
//
// State S[key i][value j];  y_t = r_t (S_{t-1} + diag(u) k_t^T v_t),  S_t = diag(d_t) S_{t-1} + k_t^T v_t  with the decay
// d_t = exp(lw_t) per key channel (lw_t = w_t for RWKV-6, log of the head's constant for RWKV-5 / 5.2).  With the
// inclusive cumulative log-decay c_t inside a chunk (c_{-1} = 0, c_m at the chunk's middle, c_C at its end):
//     R0_t = r_t exp(c_{t-1})            K^_s = k_s exp(c_C - c_s)
//     R~_t = r_t exp(c_{t-1} - c_m)      K~_s = k_s exp(c_m - c_s)         (referenced to the middle: |exponent| <= 8 tokens)
//     A_ts = R~_t . K~_s  (s < t),  A_tt = sum_i r u k
//     Y = R0 S0 + A V                    S_C = diag(exp(c_C)) S0 + K^^T V
// A start flag on token p cuts every dependence of tokens >= p on tokens < p and on S0: masks on A, on the rows
// of R0 and of K^, and on the carried state.  The state is held transposed, S^T[j][i], as mma.sync accumulator
// tiles (fp32, each of the four warps 16 value rows): a tile is already in the register layout of the next
// product's left operand, and the 16x16 score block A, computed by every warp for itself, is already in the
// layout of a right operand, so nothing but the scaled operands passes through shared memory.  The chunk is 16
// tokens because the per-channel decay is unbounded: referenced to the chunk's middle the scaling factors stay
// below exp(8 |lw|), which fp32 / bf16 hold for |lw| <= 10 per token (decay >= 4.5e-5); a chunk beyond that, or a
// decay above 1, makes the kernel leave its ticket in a flag and the token-sequential kernels (wkv6_seq.cu) redo the
// call.  A `length` inside a chunk splits that chunk in two parts that are walked like two chunks.  tcgen05 does not
// apply: its smallest tile is 64 tokens.
//
// Semantics: BaseRWKV.inner_loop of jaxrwkv, src/jaxrwkv/rwkv6.py:174-191, rwkv5_2.py:164-180, rwkv5.py:161-177.
#include <type_traits>

#include "common.cuh"
#include "device_once.cuh"

namespace b200wkv {

int* wkv_call_flag(int* ticket);   // wkv7_chunk.cu: a slot of the per-device flag ring and a fresh ticket

namespace {

typedef __nv_bfloat16 bf;
constexpr int kC6 = 16;          // tokens per chunk
constexpr int kRunLen6 = 16;    // chunks per run of the run-parallel backward
constexpr int PITCH = 72;        // bf16 per shared-memory row (144 bytes): 4-byte fragment reads and ldmatrix rows hit 32 banks
constexpr int kStages6 = 3;
constexpr float kMaxHalfDecay = 80.f;   // |sum of lw over half a chunk| the scaling can represent

struct RawStage {
    bf r[kC6][PITCH], k[kC6][PITCH], v[kC6][PITCH], w[kC6][PITCH];
};

__device__ __forceinline__ void cp_async16_zfill(void* dst_smem, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src), "r"(n)
                 : "memory");
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
// One 16-token x 16-channel block of a row-major [token][channel] tile, f[0..3] = (tokens 0-7 | 8-15) x (channels 0-7 |
// 8-15) in the order (0-7, 0-7), (8-15, 0-7), (0-7, 8-15), (8-15, 8-15).  As a LEFT operand (rows = tokens) the four
// are a0..a3; as a RIGHT operand (n = token, k = channel) tokens 0-7 take (f[0], f[2]) and tokens 8-15 (f[1], f[3]).
struct Frag {
    uint32_t f[4];
};
__device__ __forceinline__ Frag load_frag(const bf (*tile)[72], int ks, int lane) {
    Frag x;
    const int mi = lane >> 3, r8 = lane & 7;
    ldmatrix_x4(x.f[0], x.f[1], x.f[2], x.f[3], &tile[(mi & 1) * 8 + r8][16 * ks + (mi >> 1) * 8]);
    return x;
}
__device__ __forceinline__ void mma_ab(float* d, const Frag& a, const Frag& b, int nt) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a.f[0]), "r"(a.f[1]), "r"(a.f[2]), "r"(a.f[3]), "r"(b.f[nt]), "r"(b.f[nt + 2]));
}
// D(16x8, fp32) += A(16x16, bf16, row) B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Sums each of eight per-lane values over the warp with nine shuffles: three halving steps leave one value per lane,
// two butterflies finish.  Returns the total of v[which] with which = 4 bit4(lane) + 2 bit3(lane) + bit2(lane).
__device__ __forceinline__ float warp_sum8(const float* v, int lane, int* which) {
    const bool b4 = lane & 16, b3 = lane & 8, b2 = lane & 4;
    float a[4], b[2], c;
#pragma unroll
    for (int j = 0; j < 4; ++j) a[j] = (b4 ? v[j + 4] : v[j]) + __shfl_xor_sync(0xffffffffu, b4 ? v[j] : v[j + 4], 16);
#pragma unroll
    for (int j = 0; j < 2; ++j) b[j] = (b3 ? a[j + 2] : a[j]) + __shfl_xor_sync(0xffffffffu, b3 ? a[j] : a[j + 2], 8);
    c = (b2 ? b[1] : b[0]) + __shfl_xor_sync(0xffffffffu, b2 ? b[0] : b[1], 4);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    *which = (b4 ? 4 : 0) + (b3 ? 2 : 0) + (b2 ? 1 : 0);
    return c;
}

// The same for four values with six shuffles: which = 2 bit4(lane) + bit3(lane); every lane ends with the total.
__device__ __forceinline__ float warp_sum4(const float* v, int lane, int* which) {
    const bool b4 = lane & 16, b3 = lane & 8;
    float a[2], c;
#pragma unroll
    for (int j = 0; j < 2; ++j) a[j] = (b4 ? v[j + 2] : v[j]) + __shfl_xor_sync(0xffffffffu, b4 ? v[j] : v[j + 2], 16);
    c = (b3 ? a[1] : a[0]) + __shfl_xor_sync(0xffffffffu, b3 ? a[0] : a[1], 8);
    c += __shfl_xor_sync(0xffffffffu, c, 4);
    c += __shfl_xor_sync(0xffffffffu, c, 2);
    c += __shfl_xor_sync(0xffffffffu, c, 1);
    *which = (b4 ? 2 : 0) + (b3 ? 1 : 0);
    return c;
}

// ------------------------------------------------------------------ forward ---------
struct Fwd6cSmem {
    RawStage raw[kStages6];
    bf rt[kC6][PITCH], kt[kC6][PITCH], r0[kC6][PITCH], kh[kC6][PITCH];   // R~, K~, R0, K^
    bf ys[kC6][PITCH];                                                   // the chunk's outputs, token-major
    float tot[4][kN];        // sum of lw over each quarter of the chunk
    float wc[kN];            // exp(c_C), or 0 when a start flag lies in the chunk
    float dpart[2][kC6];     // sum_i r u k per token, one partial per 32 channels
    int seg[kC6];            // number of start flags at or before the token, inside the chunk
    unsigned startmask;      // bit t: start flag on token t of the chunk
    uint8_t ns[kStages6][kC6];
};

// One CTA of 128 threads per (batch, head).  ckpt: the state entering every chunk, bf16 S^T[value j][key i] in 8 column blocks of [64 j][8 i], for
// the backward (may be NULL).  The kernel gives up (flag := ticket, see the file header) on a decay above 1 and on a
// half-chunk decay beyond exp(-80).
__global__ void __launch_bounds__(128, 4)
wkv6_chunk_fwd_kernel(int Tlen, int H, const bf* __restrict__ r, const bf* __restrict__ k, const bf* __restrict__ v,
                      const bf* __restrict__ w, int w_per_token, const bf* __restrict__ u, const bf* __restrict__ s0,
                      const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts, bf* __restrict__ y,
                      bf* __restrict__ s_out, bf* __restrict__ ckpt, int* __restrict__ flag, int ticket,
                      int* __restrict__ residual_mark) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Fwd6cSmem& sm = *reinterpret_cast<Fwd6cSmem*>(smem_raw);
    const int bh = blockIdx.x, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3;
    const int j0 = warp * 16;                                    // this warp's value rows of S^T
    const size_t tok_stride = (size_t)H * kN;
    const size_t seq_base = (size_t)bi * Tlen * tok_stride + (size_t)h * kN;
    const size_t st_base = (size_t)bh * kN * kN;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kC6 - 1) / kC6;
    if (bh == 0 && tid == 0 && residual_mark != nullptr) *residual_mark = 0;   // chunked format (so far)
    const int c_out = L > 0 ? (L - 1) / kC6 : -1;                // the returned state leaves this chunk ...
    const int p_out = L > 0 ? (L - 1) % kC6 : -1;                // ... behind this token of it
    // A length inside a chunk: that chunk is walked in two parts, tokens 0..p_out and the rest, as if they were
    // two chunks (tokens outside the part at hand are inert: no decay, zero r and k, no output).
    const bool split = L > 0 && L < Tlen && p_out != kC6 - 1;

    // S^T tiles: acc[ni][e] = S[i = 8 ni + 2 q + (e & 1)][j = j0 + g + 8 (e >> 1)]
    float acc[8][4];
#pragma unroll
    for (int ni = 0; ni < 8; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e)
            acc[ni][e] = __bfloat162float(s0[st_base + (size_t)(8 * ni + 2 * q + (e & 1)) * kN + j0 + g + 8 * (e >> 1)]);
    auto write_state = [&](bf* dst) {                             // [key i][value j], as the caller keeps it
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                dst[st_base + (size_t)(8 * ni + 2 * q + (e & 1)) * kN + j0 + g + 8 * (e >> 1)] = __float2bfloat16_rn(acc[ni][e]);
    };
    if (L == 0) write_state(s_out);

    const int srow = tid >> 3, spiece = (tid & 7) * 8;            // staging: one 16-byte piece of one token row per stream
    auto issue = [&](int c) {
        if (c < nC) {
            RawStage& st = sm.raw[c % kStages6];
            const int t = c * kC6 + srow;
            const bool ok = t < Tlen;
            const size_t off = seq_base + (size_t)(ok ? t : 0) * tok_stride + spiece;
            cp_async16_zfill(&st.r[srow][spiece], r + off, ok);
            cp_async16_zfill(&st.k[srow][spiece], k + off, ok);
            cp_async16_zfill(&st.v[srow][spiece], v + off, ok);
            if (w_per_token) cp_async16_zfill(&st.w[srow][spiece], w + off, ok);
        }
        cp_async_commit();
    };
    auto load_ns = [&](int c) -> uint8_t {
        const int t = c * kC6 + tid;
        return (tid < kC6 && c < nC && t < Tlen) ? new_starts[(size_t)bi * Tlen + t] : (uint8_t)0;
    };
    issue(0);
    issue(1);
    if (tid < kC6) {
        sm.ns[0][tid] = load_ns(0);
        sm.ns[1 % kStages6][tid] = load_ns(1);
    }
    uint8_t ns_ahead = load_ns(2);

    // phase A ownership: the channel pair cp, cp + 1 and the four tokens of quarter qt (= the warp, which so holds all 64
    // channels of its tokens)
    const int cp = (tid & 31) * 2, qt = warp;
    const float2 uu = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(u + (size_t)h * kN + cp));
    float2 lw_const = make_float2(0.f, 0.f);
    if (!w_per_token) {
        const float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + (size_t)h * kN + cp));
        lw_const = make_float2(__logf(wv.x), __logf(wv.y));
    }
    bool bad = false;

    // One chunk, or one part of the split chunk.  The two cases are separate instantiations: in the common one the
    // bounds of the part are the constants 0 and 16 and every test against them folds away.
    auto walk = [&](auto split_tag, const int c, const int part_arg) {
        constexpr bool kSplitHere = decltype(split_tag)::value;
        const int part = kSplitHere ? part_arg : 0;
        const int lo = (kSplitHere && part == 1) ? p_out + 1 : 0, hi = (kSplitHere && part == 0) ? p_out + 1 : kC6;
        const RawStage& st = sm.raw[c % kStages6];
        const int t0 = c * kC6;
        if (part == 0) {
            cp_async_wait<1>();
            __syncthreads();          // chunk c has landed for everyone; the tiles of chunk c - 1 are no longer read
            issue(c + 2);
            if (tid < kC6) sm.ns[(c + 2) % kStages6][tid] = ns_ahead;
            ns_ahead = load_ns(c + 3);
            // ---- outputs of the previous chunk to global memory
            if (c > 0 && t0 - kC6 + srow < Tlen)
                *reinterpret_cast<uint4*>(y + seq_base + (size_t)(t0 - kC6 + srow) * tok_stride + spiece) =
                    *reinterpret_cast<const uint4*>(&sm.ys[srow][spiece]);
        } else {
            __syncthreads();          // the first part's products have read the operand tiles
        }
        // ---- the entering state for the backward (of the second part of a split chunk: slot nC)
        if (ckpt != nullptr) {
            bf* dst = ckpt + ((size_t)bh * (nC + 1) + (part == 0 ? c : nC)) * kN * kN;
#pragma unroll
            for (int ni = 0; ni < 8; ++ni) {
                // (8 column blocks of [64 rows j][8 keys i]: the eight row groups of a warp write one 128-byte line)
                *reinterpret_cast<uint32_t*>(dst + ni * (kN * 8) + (j0 + g) * 8 + 2 * q) = pack2(acc[ni][0], acc[ni][1]);
                *reinterpret_cast<uint32_t*>(dst + ni * (kN * 8) + (j0 + g + 8) * 8 + 2 * q) = pack2(acc[ni][2], acc[ni][3]);
            }
        }
        // ---- phase A: cumulative log-decay and scaled operands
        if (warp == 0) {
            const unsigned m = __ballot_sync(0xffffffffu, lane < kC6 && sm.ns[c % kStages6][lane] != 0);
            if (lane == 0) sm.startmask = m;
        }
        float2 lw[4], cl[4];
        float2 run = make_float2(0.f, 0.f);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const int t = 4 * qt + tt;
            const bool ok = t0 + t < Tlen && t >= lo && t < hi;
            lw[tt] = !ok ? make_float2(0.f, 0.f)
                         : (w_per_token ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.w[t][cp])) : lw_const);
            if (!(lw[tt].x <= 0.f) || !(lw[tt].y <= 0.f)) bad = true;      // a decay above 1 (or NaN) is outside what the scaling covers
            run.x += lw[tt].x;
            run.y += lw[tt].y;
            cl[tt] = run;
        }
        *reinterpret_cast<float2*>(&sm.tot[qt][cp]) = run;
        // the operands need the other quarters' totals: a barrier of the whole CTA
        __syncthreads();
        // segments: seg(t) = number of start flags at or before token t
        const unsigned starts = sm.startmask;
        auto seg_of = [&](int t) { return __popc(starts & ((2u << t) - 1u)); };
        const int seg_last = seg_of(hi - 1), seg_base = lo > 0 ? seg_of(lo - 1) : 0;   // of the part's last token; of the state entering it
        if (tid < kC6) sm.seg[tid] = seg_of(tid);
        const float2 tq0 = *reinterpret_cast<const float2*>(&sm.tot[0][cp]), tq1 = *reinterpret_cast<const float2*>(&sm.tot[1][cp]);
        const float2 tq2 = *reinterpret_cast<const float2*>(&sm.tot[2][cp]), tq3 = *reinterpret_cast<const float2*>(&sm.tot[3][cp]);
        const float2 tot0 = make_float2(tq0.x + tq1.x, tq0.y + tq1.y), tot1 = make_float2(tq2.x + tq3.x, tq2.y + tq3.y);
        if (fabsf(tot0.x) > kMaxHalfDecay || fabsf(tot1.x) > kMaxHalfDecay || fabsf(tot0.y) > kMaxHalfDecay || fabsf(tot1.y) > kMaxHalfDecay) bad = true;
        const float2 c_m = make_float2(fmaxf(tot0.x, -kMaxHalfDecay), fmaxf(tot0.y, -kMaxHalfDecay));
        const float2 c_C = make_float2(c_m.x + fmaxf(tot1.x, -kMaxHalfDecay), c_m.y + fmaxf(tot1.y, -kMaxHalfDecay));
        // cumulative log-decay in front of this quarter (the second half counts from the clamped middle, as c_C does)
        const float2 base = qt == 0 ? make_float2(0.f, 0.f) : (qt == 1 ? tq0 : (qt == 2 ? c_m : make_float2(c_m.x + tq2.x, c_m.y + tq2.y)));
        if (qt == 3)
            *reinterpret_cast<float2*>(&sm.wc[cp]) = seg_last == seg_base ? make_float2(__expf(c_C.x), __expf(c_C.y)) : make_float2(0.f, 0.f);
        float dsum[4];
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const int t = 4 * qt + tt;
            const bool in_part = t >= lo && t < hi;
            const int seg_t = seg_of(t);
            const float2 c_t = make_float2(base.x + cl[tt].x, base.y + cl[tt].y), c_prev = make_float2(c_t.x - lw[tt].x, c_t.y - lw[tt].y);
            const float2 zero2 = make_float2(0.f, 0.f);
            const float2 rv = in_part ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.r[t][cp])) : zero2;
            const float2 kv = in_part ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.k[t][cp])) : zero2;
            *reinterpret_cast<uint32_t*>(&sm.rt[t][cp]) = pack2(rv.x * __expf(fminf(c_prev.x - c_m.x, kMaxHalfDecay)), rv.y * __expf(fminf(c_prev.y - c_m.y, kMaxHalfDecay)));
            *reinterpret_cast<uint32_t*>(&sm.kt[t][cp]) = pack2(kv.x * __expf(fminf(c_m.x - c_t.x, kMaxHalfDecay)), kv.y * __expf(fminf(c_m.y - c_t.y, kMaxHalfDecay)));
            const bool first = seg_t == seg_base, last = seg_t == seg_last;
            *reinterpret_cast<uint32_t*>(&sm.r0[t][cp]) = pack2(first ? rv.x * __expf(c_prev.x) : 0.f, first ? rv.y * __expf(c_prev.y) : 0.f);
            *reinterpret_cast<uint32_t*>(&sm.kh[t][cp]) = pack2(last ? kv.x * __expf(c_C.x - c_t.x) : 0.f, last ? kv.y * __expf(c_C.y - c_t.y) : 0.f);
            dsum[tt] = fmaf(rv.x * uu.x, kv.x, rv.y * uu.y * kv.y);
        }
        {
            int which;
            const float total = warp_sum4(dsum, lane, &which);      // over all 64 channels: the warp holds them all
            if ((lane & 7) == 0) {
                sm.dpart[0][4 * qt + which] = total;
                sm.dpart[1][4 * qt + which] = 0.f;
            }
        }
        __syncthreads();

        // ---- phase B: the products
        uint32_t va[4];            // V^T of this warp: A fragments (M = value row, K = token)
        {
            const int mi = lane >> 3, r8 = lane & 7;
            ldmatrix_x4_trans(va[0], va[1], va[2], va[3], &st.v[(mi >> 1) * 8 + r8][j0 + (mi & 1) * 8]);
        }
        float yacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};    // Y^T: rows value j, columns token t
        float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};    // A: rows token t, columns token s
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint32_t s_a0 = pack2(acc[2 * ks][0], acc[2 * ks][1]), s_a1 = pack2(acc[2 * ks][2], acc[2 * ks][3]);
            const uint32_t s_a2 = pack2(acc[2 * ks + 1][0], acc[2 * ks + 1][1]), s_a3 = pack2(acc[2 * ks + 1][2], acc[2 * ks + 1][3]);
            const Frag fr = load_frag(sm.rt, ks, lane), f0 = load_frag(sm.r0, ks, lane), fk = load_frag(sm.kt, ks, lane);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                mma_bf16(yacc[nt], s_a0, s_a1, s_a2, s_a3, f0.f[nt], f0.f[nt + 2]);
                mma_ab(sacc[nt], fr, fk, nt);
            }
        }
        // masks: strictly earlier tokens of the same segment; the diagonal is the u term
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = g + 8 * (e >> 1), s = 8 * nt + 2 * q + (e & 1);
                const bool keep = s < t && sm.seg[s] == sm.seg[t];      // (rows and columns outside the part are zero operands)
                sacc[nt][e] = keep ? sacc[nt][e] : (s == t ? sm.dpart[0][t] + sm.dpart[1][t] : 0.f);
            }
        // Y^T += V^T A^T: the score tiles are the right operand as they are
        mma_bf16(yacc[0], va[0], va[1], va[2], va[3], pack2(sacc[0][0], sacc[0][1]), pack2(sacc[1][0], sacc[1][1]));
        mma_bf16(yacc[1], va[0], va[1], va[2], va[3], pack2(sacc[0][2], sacc[0][3]), pack2(sacc[1][2], sacc[1][3]));
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int t = 8 * nt + 2 * q + (e & 1);
                if (t >= lo && t < hi) sm.ys[t][j0 + g + 8 * (e >> 1)] = __float2bfloat16_rn(yacc[nt][e]);
            }
        // S^T <- S^T diag(exp(c_C)) [no start in the chunk] + V^T K^
        {
            const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const float2 w0 = *reinterpret_cast<const float2*>(&sm.wc[16 * np + 2 * q]);
                const float2 w1 = *reinterpret_cast<const float2*>(&sm.wc[16 * np + 8 + 2 * q]);
                acc[2 * np][0] *= w0.x; acc[2 * np][1] *= w0.y; acc[2 * np][2] *= w0.x; acc[2 * np][3] *= w0.y;
                acc[2 * np + 1][0] *= w1.x; acc[2 * np + 1][1] *= w1.y; acc[2 * np + 1][2] *= w1.x; acc[2 * np + 1][3] *= w1.y;
                uint32_t b0, b1, b2, b3;        // key tiles 2 np (b0, b1) and 2 np + 1 (b2, b3)
                ldmatrix_x4_trans(b0, b1, b2, b3, &sm.kh[(mi & 1) * 8 + r8][(2 * np + (mi >> 1)) * 8]);
                mma_bf16(acc[2 * np], va[0], va[1], va[2], va[3], b0, b1);
                mma_bf16(acc[2 * np + 1], va[0], va[1], va[2], va[3], b2, b3);
            }
        }
        if (c == c_out && part == 0) write_state(s_out);
    };
    for (int c = 0; c < nC; ++c) {
        if (split && c == c_out) {
#pragma unroll 1
            for (int part = 0; part < 2; ++part) walk(std::true_type{}, c, part);
        } else {
            walk(std::false_type{}, c, 0);
        }
    }
    __syncthreads();
    {
        const int t = (nC - 1) * kC6 + srow;
        if (t < Tlen) *reinterpret_cast<uint4*>(y + seq_base + (size_t)t * tok_stride + spiece) = *reinterpret_cast<const uint4*>(&sm.ys[srow][spiece]);
    }
    if (bad) atomicExch(flag, ticket);
}


// ------------------------------------------------------------------ backward --------
// Chunks in reverse order with the gradient of the state, dS^T[j][i], in accumulator tiles.  Per chunk, with the
// forward's operands rebuilt from the raw rows and the entering state S0 read from the forward's checkpoint:
//     dA = mask(dY V^T)                                   dd_t = dy_t . v_t  (its diagonal, the u term)
//     dV  = A^T dY + K^ dS_C
//     dR0 = dY S0^T        dR~ = dA K~        dK~ = dA^T R~        dK^ = V dS_C^T
//     dr = dR0 exp(c_{t-1}) + dR~ exp(c_{t-1} - c_m) + dd u k        dk = dK~ exp(c_m - c_s) + dK^ exp(c_C - c_s) + dd u r
//     dS0^T = dS_C^T diag(exp(c_C)) + dY^T R0
// and the gradient of the log-decay from the positions at which each factor depends on the cumulative sum:
//     dlw_tau = sum_{x >= tau} [ (r dr')_{x+1} - (k dk')_x ] + sum_s k dK^ exp(c_C - c_s) + exp(c_C) sum_j dS_C S0
// (dr', dk' without the u terms; the two references to the middle cancel).  Every warp owns 16 channels of the
// token-by-channel results and 16 value rows of dS^T, and computes the 16x16 score blocks for itself.
struct BwdStage {
    bf r[kC6][PITCH], k[kC6][PITCH], v[kC6][PITCH], w[kC6][PITCH], dy[kC6][PITCH];
    // S0^T[j][i] as it lies in the residual: 8 column blocks of [64 rows j][8 keys i] (a linear copy; the eight rows of an
    // ldmatrix tile are 128 contiguous bytes); once the products have read it, r dr' and k dk' per token and channel
    // (fp32, two tiles of [16][EPITCH], which need the tail)
    bf s0[8][kN][8];
    bf s0_tail[kN * PITCH - 8 * kN * 8];
};
// fp32 [token][channel] tiles that the epilogue's threads address as (row g, column pair 2 q): with 72 floats per row the
// sixteen lanes of a 64-bit access (four rows, four column pairs) fall into 32 different banks
constexpr int EPITCH = 72;
static_assert(sizeof(bf) * kN * PITCH >= 2 * sizeof(float) * kC6 * EPITCH, "the two fp32 tiles must fit over the state tile and its tail");
struct Bwd6cSmem {
    BwdStage st[2];
    bf ops[4][kC6][PITCH];     // R~, K~, R0, K^ while the products run; then dr, dk, dv, dw on their way out
    bf ds[kN][PITCH];          // dS_C^T[j][i] in bf16, for the one product that contracts over j
    float e2[kC6][EPITCH], e3[kC6][EPITCH];   // exp(c_{t-1} - c_m) and exp(c_m - c_t): what turns dR~, dK~ into dr, dk
    float em[kN], ecm[kN];     // exp(c_m) and exp(c_C - c_m): the same for dR0 and dK^
    float tot[4][kN];          // sum of lw over each quarter of the chunk
    float wc[kN];              // exp(c_C), or 0 when a start flag lies in the chunk
    float lump[kN];            // what every token of the chunk receives: the K^ references and the carried state
    float gw[4][kN];           // sum_j dS_C S0 over each warp's value rows
    float dpart[2][kC6];
    int seg[kC6];
    unsigned startmask;
    uint8_t ns[2][kC6];
};

__global__ void __launch_bounds__(128, 3)
wkv6_chunk_bwd_kernel(int Tlen, int H, const bf* __restrict__ r, const bf* __restrict__ k, const bf* __restrict__ v,
                      const bf* __restrict__ w, int w_per_token, const bf* __restrict__ u,
                      const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                      const bf* __restrict__ dy, const bf* __restrict__ ds_out, const bf* __restrict__ ckpt,
                      const int* __restrict__ residual_mark, bf* __restrict__ dr, bf* __restrict__ dk, bf* __restrict__ dv,
                      bf* __restrict__ dw_tok, float* __restrict__ dw_head, float* __restrict__ du_head, bf* __restrict__ ds0,
                      int n_runs, int run_len, const bf* __restrict__ dsck, float* __restrict__ partial) {
    if (*residual_mark != 0) return;          // the forward fell back to the sequential kernels
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Bwd6cSmem& sm = *reinterpret_cast<Bwd6cSmem*>(smem_raw);
    // n_runs > 1: a sequence is walked by n_runs CTAs, run rho = chunks [rho run_len, (rho + 1) run_len), each starting
    // from the state gradient that the carry kernel (wkv6_carry_bwd_kernel) left for the end of its run
    const int bh = blockIdx.x / n_runs, run = blockIdx.x % n_runs, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3, mi = lane >> 3, r8 = lane & 7;
    const int j0 = warp * 16;                 // value rows of dS^T, and key channels of the token-by-channel results
    const size_t tok_stride = (size_t)H * kN;
    const size_t seq_base = (size_t)bi * Tlen * tok_stride + (size_t)h * kN;
    const size_t st_base = (size_t)bh * kN * kN;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kC6 - 1) / kC6;
    const int c_out = L > 0 ? (L - 1) / kC6 : -1, p_out = L > 0 ? (L - 1) % kC6 : -1;
    const bool split = L > 0 && L < Tlen && p_out != kC6 - 1;      // see the forward: that chunk is walked in two parts
    const int c_lo = run * run_len, c_hi = min(nC, c_lo + run_len);
    if (c_lo >= c_hi) return;

    float acc[8][4];
    if (run == n_runs - 1 || c_hi >= nC) {
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[ni][e] = 0.f;
    } else {
        const bf* src = dsck + ((size_t)bh * n_runs + run) * kN * kN;
#pragma unroll
        for (int ni = 0; ni < 8; ++ni) {
            const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (size_t)(j0 + g) * kN + 8 * ni + 2 * q));
            const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (size_t)(j0 + g + 8) * kN + 8 * ni + 2 * q));
            acc[ni][0] = lo2.x; acc[ni][1] = lo2.y; acc[ni][2] = hi2.x; acc[ni][3] = hi2.y;
        }
    }
    auto add_ds_out = [&]() {
        if (ds_out == nullptr) return;
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                acc[ni][e] += __bfloat162float(ds_out[st_base + (size_t)(8 * ni + 2 * q + (e & 1)) * kN + j0 + g + 8 * (e >> 1)]);
    };

    const int srow = tid >> 3, spiece = (tid & 7) * 8;
    auto issue = [&](int c, int stage) {
        if (c >= c_lo) {
            BwdStage& st = sm.st[stage];
            const int t = c * kC6 + srow;
            const bool ok = t < Tlen;
            const size_t off = seq_base + (size_t)(ok ? t : 0) * tok_stride + spiece;
            cp_async16_zfill(&st.r[srow][spiece], r + off, ok);
            cp_async16_zfill(&st.k[srow][spiece], k + off, ok);
            cp_async16_zfill(&st.v[srow][spiece], v + off, ok);
            if (w_per_token) cp_async16_zfill(&st.w[srow][spiece], w + off, ok);
            cp_async16_zfill(&st.dy[srow][spiece], dy != nullptr ? dy + off : r + off, ok && dy != nullptr);
            const bf* src = ckpt + ((size_t)bh * (nC + 1) + c) * kN * kN;
#pragma unroll
            for (int rr = 0; rr < 4; ++rr) {   // piece tid + 128 rr of the tile: row = piece mod 64 of column block piece / 64
                const int pc = tid + 128 * rr;
                cp_async16_zfill(&st.s0[pc >> 6][pc & 63][0], src + (size_t)pc * 8, true);
            }
        }
        cp_async_commit();
    };
    // the state entering a part of the split chunk, fetched on the spot (once or twice per sequence)
    auto fetch_state = [&](int slot, int stage) {
        const bf* src = ckpt + ((size_t)bh * (nC + 1) + slot) * kN * kN;
#pragma unroll
        for (int rr = 0; rr < 4; ++rr)
            cp_async16_zfill(&sm.st[stage].s0[(tid + 128 * rr) >> 6][(tid + 128 * rr) & 63][0], src + (size_t)(tid + 128 * rr) * 8, true);
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
    };
    auto load_ns = [&](int c) -> uint8_t {
        const int t = c * kC6 + tid;
        return (tid < kC6 && c >= 0 && t < Tlen) ? new_starts[(size_t)bi * Tlen + t] : (uint8_t)0;
    };
    issue(c_hi - 1, 0);
    if (tid < kC6) sm.ns[0][tid] = load_ns(c_hi - 1);
    uint8_t ns_ahead = load_ns(c_hi - 2);

    // phase A ownership as in the forward: the channel pair cp, cp + 1 and the four tokens of quarter qt (= the warp)
    const int cp = (tid & 31) * 2, qt = warp;
    const float2 uu_a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(u + (size_t)h * kN + cp));
    float2 lw_const = make_float2(0.f, 0.f);
    if (!w_per_token) {
        const float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + (size_t)h * kN + cp));
        lw_const = make_float2(__logf(wv.x), __logf(wv.y));
    }
    float u_col[2][2];                         // u of this thread's four result columns
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) u_col[nt][e] = __bfloat162float(u[(size_t)h * kN + j0 + 8 * nt + 2 * q + e]);
    float du_acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    float dw_acc = 0.f;                        // constant decay: sum over tokens of the log-decay gradient (thread ch < 64)

    int out_t0 = -1, out_lo = 0, out_hi = 0;     // the chunk (part) whose results wait in the result tiles
    auto flush_results = [&]() {
        const int t = out_t0 + srow;
        if (out_t0 >= 0 && t < Tlen && srow >= out_lo && srow < out_hi) {
            const size_t off = seq_base + (size_t)t * tok_stride + spiece;
            *reinterpret_cast<uint4*>(dr + off) = *reinterpret_cast<const uint4*>(&sm.ops[0][srow][spiece]);
            *reinterpret_cast<uint4*>(dk + off) = *reinterpret_cast<const uint4*>(&sm.ops[1][srow][spiece]);
            *reinterpret_cast<uint4*>(dv + off) = *reinterpret_cast<const uint4*>(&sm.ops[2][srow][spiece]);
            if (w_per_token) *reinterpret_cast<uint4*>(dw_tok + off) = *reinterpret_cast<const uint4*>(&sm.ops[3][srow][spiece]);
        }
    };
    auto walk = [&](auto split_tag, const int c, const int it, const int part_arg) {
        constexpr bool kSplitHere = decltype(split_tag)::value;
        const bool split_here = kSplitHere;
        const int part = kSplitHere ? part_arg : 0;
        const int stage = it & 1;
        const int lo = (kSplitHere && part == 1) ? p_out + 1 : 0, hi = (kSplitHere && part == 0) ? p_out + 1 : kC6;
        if (!split_here || part == 1) {                               // first visit of the chunk
            cp_async_wait<0>();
            __syncthreads();                                          // S1
            issue(c - 1, stage ^ 1);
            if (tid < kC6) sm.ns[stage ^ 1][tid] = ns_ahead;
            ns_ahead = load_ns(c - 2);
            if (split_here) fetch_state(nC, stage);                   // the state behind token p_out
        } else {
            __syncthreads();                                          // the first visit's suffix sums have read the tile refilled here
            fetch_state(c, stage);
        }
        flush_results();                                              // of the walk before this one; phase A rewrites the tiles behind S2
        const BwdStage& st = sm.st[stage];
        const int t0 = c * kC6;
        if (c == c_out && part == 0) add_ds_out();
        // dS_C^T in bf16 for the product that contracts over value rows
#pragma unroll
        for (int ni = 0; ni < 8; ++ni) {
            *reinterpret_cast<uint32_t*>(&sm.ds[j0 + g][8 * ni + 2 * q]) = pack2(acc[ni][0], acc[ni][1]);
            *reinterpret_cast<uint32_t*>(&sm.ds[j0 + g + 8][8 * ni + 2 * q]) = pack2(acc[ni][2], acc[ni][3]);
        }
        // ---- phase A: as in the forward
        if (warp == 0) {
            const unsigned m = __ballot_sync(0xffffffffu, lane < kC6 && sm.ns[stage][lane] != 0);
            if (lane == 0) sm.startmask = m;
        }
        float2 lw[4], cl[4];
        float2 run = make_float2(0.f, 0.f);
#pragma unroll
        for (int tt = 0; tt < 4; ++tt) {
            const int t = 4 * qt + tt;
            const bool ok = t0 + t < Tlen && t >= lo && t < hi;
            lw[tt] = !ok ? make_float2(0.f, 0.f)
                         : (w_per_token ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.w[t][cp])) : lw_const);
            run.x += lw[tt].x;
            run.y += lw[tt].y;
            cl[tt] = run;
        }
        *reinterpret_cast<float2*>(&sm.tot[qt][cp]) = run;
        __syncthreads();                                              // S2
        {
            const unsigned starts = sm.startmask;
            auto seg_of = [&](int t) { return __popc(starts & ((2u << t) - 1u)); };
            const int seg_last = seg_of(hi - 1), seg_base = lo > 0 ? seg_of(lo - 1) : 0;
            if (tid < kC6) sm.seg[tid] = seg_of(tid);
            const float2 tq0 = *reinterpret_cast<const float2*>(&sm.tot[0][cp]), tq1 = *reinterpret_cast<const float2*>(&sm.tot[1][cp]);
            const float2 tq2 = *reinterpret_cast<const float2*>(&sm.tot[2][cp]), tq3 = *reinterpret_cast<const float2*>(&sm.tot[3][cp]);
            const float2 c_m = make_float2(fmaxf(tq0.x + tq1.x, -kMaxHalfDecay), fmaxf(tq0.y + tq1.y, -kMaxHalfDecay));
            const float2 c_C = make_float2(c_m.x + fmaxf(tq2.x + tq3.x, -kMaxHalfDecay), c_m.y + fmaxf(tq2.y + tq3.y, -kMaxHalfDecay));
            const float2 base = qt == 0 ? make_float2(0.f, 0.f) : (qt == 1 ? tq0 : (qt == 2 ? c_m : make_float2(c_m.x + tq2.x, c_m.y + tq2.y)));
            if (qt == 3) {
                const bool carried = seg_last == seg_base;
                *reinterpret_cast<float2*>(&sm.wc[cp]) = carried ? make_float2(__expf(c_C.x), __expf(c_C.y)) : make_float2(0.f, 0.f);
                *reinterpret_cast<float2*>(&sm.em[cp]) = make_float2(__expf(c_m.x), __expf(c_m.y));
                *reinterpret_cast<float2*>(&sm.ecm[cp]) = make_float2(__expf(c_C.x - c_m.x), __expf(c_C.y - c_m.y));
            }
            float dsum[4];
#pragma unroll
            for (int tt = 0; tt < 4; ++tt) {
                const int t = 4 * qt + tt;
                const int seg_t = seg_of(t);
                const float2 c_t = make_float2(base.x + cl[tt].x, base.y + cl[tt].y), c_prev = make_float2(c_t.x - lw[tt].x, c_t.y - lw[tt].y);
                const bool in_part = t >= lo && t < hi;
                const float2 zero2 = make_float2(0.f, 0.f);
                const float2 rv = in_part ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.r[t][cp])) : zero2;
                const float2 kv = in_part ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.k[t][cp])) : zero2;
                const float2 f2 = make_float2(__expf(fminf(c_prev.x - c_m.x, kMaxHalfDecay)), __expf(fminf(c_prev.y - c_m.y, kMaxHalfDecay)));
                const float2 f3 = make_float2(__expf(fminf(c_m.x - c_t.x, kMaxHalfDecay)), __expf(fminf(c_m.y - c_t.y, kMaxHalfDecay)));
                *reinterpret_cast<float2*>(&sm.e2[t][cp]) = f2;
                *reinterpret_cast<float2*>(&sm.e3[t][cp]) = f3;
                const bool first = seg_t == seg_base, last = seg_t == seg_last;
                *reinterpret_cast<uint32_t*>(&sm.ops[0][t][cp]) = pack2(rv.x * f2.x, rv.y * f2.y);
                *reinterpret_cast<uint32_t*>(&sm.ops[1][t][cp]) = pack2(kv.x * f3.x, kv.y * f3.y);
                *reinterpret_cast<uint32_t*>(&sm.ops[2][t][cp]) = pack2(first ? rv.x * __expf(c_prev.x) : 0.f, first ? rv.y * __expf(c_prev.y) : 0.f);
                *reinterpret_cast<uint32_t*>(&sm.ops[3][t][cp]) = pack2(last ? kv.x * __expf(c_C.x - c_t.x) : 0.f, last ? kv.y * __expf(c_C.y - c_t.y) : 0.f);
                dsum[tt] = fmaf(rv.x * uu_a.x, kv.x, rv.y * uu_a.y * kv.y);
            }
            int which;
            const float total = warp_sum4(dsum, lane, &which);       // over all 64 channels: the warp holds them all
            if ((lane & 7) == 0) {
                sm.dpart[0][4 * qt + which] = total;
                sm.dpart[1][4 * qt + which] = 0.f;
            }
        }
        __syncthreads();                                              // S3
        const bf (*Rt)[PITCH] = sm.ops[0];
        const bf (*Kt)[PITCH] = sm.ops[1];
        const bf (*R0)[PITCH] = sm.ops[2];
        const bf (*Kh)[PITCH] = sm.ops[3];

        // ---- the 16x16 blocks: dA (t x s), dA^T (s x t), A^T (s x t)
        float dA[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, dAT[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float AT[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        Frag fdy[4], fv[4];                   // dY and V, all four K steps (left and right operands alike)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            fdy[ks] = load_frag(st.dy, ks, lane);
            fv[ks] = load_frag(st.v, ks, lane);
            const Frag fk = load_frag(Kt, ks, lane), fr = load_frag(Rt, ks, lane);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                mma_ab(dA[nt], fdy[ks], fv[ks], nt);
                mma_ab(dAT[nt], fv[ks], fdy[ks], nt);
                mma_ab(AT[nt], fk, fr, nt);
            }
        }
        // dd of this thread's two token rows: the diagonal of dA sits in lane 4 g + g / 2
        float dd_lo, dd_hi;
        {
            const float cand_lo = (g & 1) ? dA[0][1] : dA[0][0], cand_hi = (g & 1) ? dA[1][3] : dA[1][2];
            const int src = (lane & ~3) | (g >> 1);
            dd_lo = __shfl_sync(0xffffffffu, cand_lo, src);
            dd_hi = __shfl_sync(0xffffffffu, cand_hi, src);
        }
        int seg_r[2] = {sm.seg[g], sm.seg[g + 8]};
        const int seg_end = sm.seg[hi - 1], seg_in = lo > 0 ? sm.seg[lo - 1] : 0;     // as seg_last / seg_base of phase A
        const bool row_in[2] = {g >= lo && g < hi, g + 8 >= lo && g + 8 < hi};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int row = g + 8 * (e >> 1), col = 8 * nt + 2 * q + (e & 1);
                const bool same = sm.seg[col] == seg_r[e >> 1] && row_in[e >> 1] && col >= lo && col < hi;
                dA[nt][e] = (col < row && same) ? dA[nt][e] : 0.f;                       // rows t, columns s < t
                dAT[nt][e] = (row < col && same) ? dAT[nt][e] : 0.f;                     // rows s, columns t > s
                AT[nt][e] = (row < col && same) ? AT[nt][e] : (row == col ? sm.dpart[0][row] + sm.dpart[1][row] : 0.f);
            }
        // ---- dV (s x j of this warp) = A^T dY + K^ dS_C
        float dV[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, &st.dy[(mi & 1) * 8 + r8][j0 + (mi >> 1) * 8]);
            const uint32_t a0 = pack2(AT[0][0], AT[0][1]), a1 = pack2(AT[0][2], AT[0][3]);
            const uint32_t a2 = pack2(AT[1][0], AT[1][1]), a3 = pack2(AT[1][2], AT[1][3]);
            mma_bf16(dV[0], a0, a1, a2, a3, b0, b1);
            mma_bf16(dV[1], a0, a1, a2, a3, b2, b3);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const Frag fh = load_frag(Kh, ks, lane);
                const uint32_t h0 = fh.f[0], h1 = fh.f[1], h2 = fh.f[2], h3 = fh.f[3];
                // dS_C^T tiles as right operand: K = key channel (their columns), n = value row (their rows)
                mma_bf16(dV[0], h0, h1, h2, h3, pack2(acc[2 * ks][0], acc[2 * ks][1]), pack2(acc[2 * ks + 1][0], acc[2 * ks + 1][1]));
                mma_bf16(dV[1], h0, h1, h2, h3, pack2(acc[2 * ks][2], acc[2 * ks][3]), pack2(acc[2 * ks + 1][2], acc[2 * ks + 1][3]));
            }
        }
        // ---- the token x channel results for this warp's 16 key channels
        float dR0[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, dRt[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
        float dKt[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, dKh[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, &st.s0[j0 / 8 + (mi >> 1)][16 * ks + (mi & 1) * 8 + r8][0]);
            mma_bf16(dR0[0], fdy[ks].f[0], fdy[ks].f[1], fdy[ks].f[2], fdy[ks].f[3], b0, b1);
            mma_bf16(dR0[1], fdy[ks].f[0], fdy[ks].f[1], fdy[ks].f[2], fdy[ks].f[3], b2, b3);
            ldmatrix_x4_trans(b0, b1, b2, b3, &sm.ds[16 * ks + (mi & 1) * 8 + r8][j0 + (mi >> 1) * 8]);
            mma_bf16(dKh[0], fv[ks].f[0], fv[ks].f[1], fv[ks].f[2], fv[ks].f[3], b0, b1);
            mma_bf16(dKh[1], fv[ks].f[0], fv[ks].f[1], fv[ks].f[2], fv[ks].f[3], b2, b3);
        }
        {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(b0, b1, b2, b3, &Kt[(mi & 1) * 8 + r8][j0 + (mi >> 1) * 8]);
            uint32_t a0 = pack2(dA[0][0], dA[0][1]), a1 = pack2(dA[0][2], dA[0][3]), a2 = pack2(dA[1][0], dA[1][1]), a3 = pack2(dA[1][2], dA[1][3]);
            mma_bf16(dRt[0], a0, a1, a2, a3, b0, b1);
            mma_bf16(dRt[1], a0, a1, a2, a3, b2, b3);
            ldmatrix_x4_trans(b0, b1, b2, b3, &Rt[(mi & 1) * 8 + r8][j0 + (mi >> 1) * 8]);
            a0 = pack2(dAT[0][0], dAT[0][1]); a1 = pack2(dAT[0][2], dAT[0][3]); a2 = pack2(dAT[1][0], dAT[1][1]); a3 = pack2(dAT[1][2], dAT[1][3]);
            mma_bf16(dKt[0], a0, a1, a2, a3, b0, b1);
            mma_bf16(dKt[1], a0, a1, a2, a3, b2, b3);
        }
        // ---- sum_j dS_C[i][j] S0[i][j] over this warp's value rows
        {
#pragma unroll
            for (int ni = 0; ni < 8; ++ni) {
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.s0[ni][j0 + g][2 * q]));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.s0[ni][j0 + g + 8][2 * q]));
                float p0 = acc[ni][0] * lo.x + acc[ni][2] * hi.x, p1 = acc[ni][1] * lo.y + acc[ni][3] * hi.y;
#pragma unroll
                for (int m = 4; m < 32; m <<= 1) {
                    p0 += __shfl_xor_sync(0xffffffffu, p0, m);
                    p1 += __shfl_xor_sync(0xffffffffu, p1, m);
                }
                if (g == 0) *reinterpret_cast<float2*>(&sm.gw[warp][8 * ni + 2 * q]) = make_float2(p0, p1);
            }
        }
        // ---- dS0^T = dS_C^T diag(exp(c_C)) [no start in the chunk] + dY^T R0
        {
            uint32_t ya[4];
            ldmatrix_x4_trans(ya[0], ya[1], ya[2], ya[3], &st.dy[(mi >> 1) * 8 + r8][j0 + (mi & 1) * 8]);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const float2 w0 = *reinterpret_cast<const float2*>(&sm.wc[16 * np + 2 * q]);
                const float2 w1 = *reinterpret_cast<const float2*>(&sm.wc[16 * np + 8 + 2 * q]);
                acc[2 * np][0] *= w0.x; acc[2 * np][1] *= w0.y; acc[2 * np][2] *= w0.x; acc[2 * np][3] *= w0.y;
                acc[2 * np + 1][0] *= w1.x; acc[2 * np + 1][1] *= w1.y; acc[2 * np + 1][2] *= w1.x; acc[2 * np + 1][3] *= w1.y;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, &R0[(mi & 1) * 8 + r8][(2 * np + (mi >> 1)) * 8]);
                mma_bf16(acc[2 * np], ya[0], ya[1], ya[2], ya[3], b0, b1);
                mma_bf16(acc[2 * np + 1], ya[0], ya[1], ya[2], ya[3], b2, b3);
            }
        }
        __syncthreads();                                              // S4: nobody reads the operand tiles any more
        // ---- epilogue: rows t = g, g + 8; column pairs i = j0 + 8 nt + 2 q, + 1
        float (*ea)[EPITCH] = reinterpret_cast<float (*)[EPITCH]>(&sm.st[stage].s0[0][0][0]);
        float (*eb)[EPITCH] = ea + kC6;
        {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int i = j0 + 8 * nt + 2 * q;
                const float2 em2 = *reinterpret_cast<const float2*>(&sm.em[i]), ecm2 = *reinterpret_cast<const float2*>(&sm.ecm[i]);
                float lump0 = 0.f, lump1 = 0.f;
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {       // the two token rows
                    const int t = g + 8 * hh, e0 = 2 * hh;
                    const float2 f2 = *reinterpret_cast<const float2*>(&sm.e2[t][i]), f3 = *reinterpret_cast<const float2*>(&sm.e3[t][i]);
                    const float2 rv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.r[t][i]));
                    const float2 kv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.k[t][i]));
                    const float dd = hh ? dd_hi : dd_lo;
                    const int sg = seg_r[hh];
                    const float live = row_in[hh] ? 1.f : 0.f;
                    const float m0 = sg == seg_in ? live : 0.f, mE = sg == seg_end ? live : 0.f;
                    // x: column i, y: column i + 1
                    const float drp_x = (m0 * dR0[nt][e0] * em2.x + dRt[nt][e0]) * f2.x, drp_y = (m0 * dR0[nt][e0 + 1] * em2.y + dRt[nt][e0 + 1]) * f2.y;
                    const float khp_x = mE * dKh[nt][e0] * ecm2.x * f3.x, khp_y = mE * dKh[nt][e0 + 1] * ecm2.y * f3.y;
                    const float dkp_x = fmaf(dKt[nt][e0], f3.x, khp_x), dkp_y = fmaf(dKt[nt][e0 + 1], f3.y, khp_y);
                    *reinterpret_cast<uint32_t*>(&sm.ops[0][t][i]) = pack2(fmaf(dd * u_col[nt][0], kv.x, drp_x), fmaf(dd * u_col[nt][1], kv.y, drp_y));
                    *reinterpret_cast<uint32_t*>(&sm.ops[1][t][i]) = pack2(fmaf(dd * u_col[nt][0], rv.x, dkp_x), fmaf(dd * u_col[nt][1], rv.y, dkp_y));
                    *reinterpret_cast<uint32_t*>(&sm.ops[2][t][i]) = pack2(dV[nt][e0], dV[nt][e0 + 1]);   // dV: rows s = t, columns j = i
                    *reinterpret_cast<float2*>(&ea[t][i]) = make_float2(rv.x * drp_x, rv.y * drp_y);
                    *reinterpret_cast<float2*>(&eb[t][i]) = make_float2(kv.x * dkp_x, kv.y * dkp_y);
                    lump0 = fmaf(kv.x, khp_x, lump0);
                    lump1 = fmaf(kv.y, khp_y, lump1);
                    du_acc[nt][0] = fmaf(live * dd * rv.x, kv.x, du_acc[nt][0]);
                    du_acc[nt][1] = fmaf(live * dd * rv.y, kv.y, du_acc[nt][1]);
                }
#pragma unroll
                for (int m = 4; m < 32; m <<= 1) {
                    lump0 += __shfl_xor_sync(0xffffffffu, lump0, m);
                    lump1 += __shfl_xor_sync(0xffffffffu, lump1, m);
                }
                if (g == 0) {
                    const float2 wc2 = *reinterpret_cast<const float2*>(&sm.wc[i]);
                    const float gx = sm.gw[0][i] + sm.gw[1][i] + sm.gw[2][i] + sm.gw[3][i];
                    const float gy = sm.gw[0][i + 1] + sm.gw[1][i + 1] + sm.gw[2][i + 1] + sm.gw[3][i + 1];
                    *reinterpret_cast<float2*>(&sm.lump[i]) = make_float2(fmaf(gx, wc2.x, lump0), fmaf(gy, wc2.y, lump1));
                }
            }
        }
        __syncthreads();                                              // S5
        if (tid < kN) {
            // suffix sums over the chunk's 16 positions: the log-decay of token tau acts on every cumulative sum c_x, x >= tau
            float run2 = sm.lump[tid];
#pragma unroll
            for (int x = kC6 - 1; x >= 0; --x) {
                run2 += (x + 1 < kC6 ? ea[x + 1][tid] : 0.f) - eb[x][tid];
                if (w_per_token) sm.ops[3][x][tid] = __float2bfloat16_rn(run2);
                else if (t0 + x < Tlen && x >= lo && x < hi) dw_acc += run2;
            }
        }
        // the four result tiles leave after the next barrier (the top of the next walk, or the one behind the loop)
        out_t0 = t0;
        out_lo = lo;
        out_hi = hi;
    };
    for (int c = c_hi - 1, it = 0; c >= c_lo; --c, ++it) {
        if (split && c == c_out) {
#pragma unroll 1
            for (int part = 1; part >= 0; --part) walk(std::true_type{}, c, it, part);   // tokens behind `length` first
        } else {
            walk(std::false_type{}, c, it, 0);
        }
    }
    __syncthreads();
    flush_results();
    if (run == 0) {
        if (L == 0) add_ds_out();
#pragma unroll
        for (int ni = 0; ni < 8; ++ni)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                ds0[st_base + (size_t)(8 * ni + 2 * q + (e & 1)) * kN + j0 + g + 8 * (e >> 1)] = __float2bfloat16_rn(acc[ni][e]);
    }
    // per-(batch, head) sums over tokens: directly, or this run's share for the reduction behind the kernel
    float* const du_dst = n_runs == 1 ? du_head + (size_t)bh * kN : partial + ((size_t)bh * n_runs + run) * 2 * kN;
    float* const dw_dst = n_runs == 1 ? (dw_head != nullptr ? dw_head + (size_t)bh * kN : nullptr) : du_dst + kN;
    // du: sum over this thread's token rows, then over the eight row groups of the warp
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float p = du_acc[nt][e];
#pragma unroll
            for (int m = 4; m < 32; m <<= 1) p += __shfl_xor_sync(0xffffffffu, p, m);
            if (g == 0) du_dst[j0 + 8 * nt + 2 * q + e] = p;
        }
    if (!w_per_token && tid < kN && dw_dst != nullptr) dw_dst[tid] = dw_acc / __bfloat162float(w[(size_t)h * kN + tid]);
}

// ------------------------------------------------------------------ the state-gradient carry
// The only part of the backward that is sequential in T, on its own: dS0^T = dS_C^T diag(exp(c_C)) [no start in the
// chunk] + dY^T R0 per chunk (and the cotangent of the returned state where it enters), with dS^T in accumulator
// registers.  It leaves the state gradient at the end of every run of `run_len` chunks, from which the gradient kernel
// above walks the runs in parallel.
// Unlike the other kernels of this file it walks 64 tokens at a time: it uses no factor other than exp(cumulative
// log-decay) <= 1, so nothing limits its chunk, and a quarter of the steps means a quarter of the barriers and waits.
constexpr int kCB = 64;            // tokens per step of the carry
constexpr int kCarryStages = 2;
constexpr int kQT = kCB / 4;       // tokens per thread in phase A
static_assert(kRunLen6 % (kCB / kC6) == 0, "runs must end at a step of the carry");
struct CarryStage6 {
    bf r[kCB][PITCH], w[kCB][PITCH], dy[kCB][PITCH];   // r becomes R0 in place
};
struct Carry6Smem {
    CarryStage6 st[kCarryStages];
    float tot[4][kN];              // sum of the log-decay over each quarter of the step
    float wc[kN];
    unsigned startmask[2];         // bit t of word t / 32: start flag on token t of the step (one word used when kCB == 32)
    uint8_t ns[kCarryStages][kCB];
};
static_assert(4 * (sizeof(Carry6Smem) + 1024) <= 228 * 1024, "four CTAs per SM");

__global__ void __launch_bounds__(128, 4)
wkv6_carry_bwd_kernel(int Tlen, int H, const bf* __restrict__ r, const bf* __restrict__ w, int w_per_token,
                      const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts, const bf* __restrict__ dy,
                      const bf* __restrict__ ds_out, const int* __restrict__ residual_mark, int n_runs, int run_len,
                      bf* __restrict__ dsck) {
    if (*residual_mark != 0) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Carry6Smem& sm = *reinterpret_cast<Carry6Smem*>(smem_raw);
    const int bh = blockIdx.x, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, q = lane & 3, mi = lane >> 3, r8 = lane & 7;
    const int j0 = warp * 16;
    const size_t tok_stride = (size_t)H * kN;
    const size_t seq_base = (size_t)bi * Tlen * tok_stride + (size_t)h * kN;
    const size_t st_base = (size_t)bh * kN * kN;
    const int L = min((int)length[bi], Tlen);
    const int nB = (Tlen + kCB - 1) / kCB;                 // steps of the carry
    const int run_steps = run_len / (kCB / kC6);           // steps per run of the gradient kernel
    const int c_out = L > 0 ? (L - 1) / kCB : -1, p_out = L > 0 ? (L - 1) % kCB : -1;
    const bool split = L > 0 && L < Tlen && p_out != kCB - 1;
    const int c_stop = run_steps;      // nothing below the first run's end is needed: run 0 starts from the state left there

    float acc[8][4];
#pragma unroll
    for (int ni = 0; ni < 8; ++ni)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[ni][e] = 0.f;
    auto issue = [&](int c) {
        if (c >= c_stop) {
            CarryStage6& st = sm.st[c % kCarryStages];
#pragma unroll
            for (int rr = 0; rr < kCB / 16; ++rr) {
                const int row = (tid >> 3) + 16 * rr, piece = (tid & 7) * 8;
                const int t = c * kCB + row;
                const bool ok = t < Tlen;
                const size_t off = seq_base + (size_t)(ok ? t : 0) * tok_stride + piece;
                cp_async16_zfill(&st.r[row][piece], r + off, ok);
                if (w_per_token) cp_async16_zfill(&st.w[row][piece], w + off, ok);
                cp_async16_zfill(&st.dy[row][piece], dy != nullptr ? dy + off : r + off, ok && dy != nullptr);
            }
        }
        cp_async_commit();
    };
    auto load_ns = [&](int c) -> uint8_t {
        const int t = c * kCB + tid;
        return (tid < kCB && c >= 0 && t < Tlen) ? new_starts[(size_t)bi * Tlen + t] : (uint8_t)0;
    };
#pragma unroll
    for (int i = 1; i < kCarryStages; ++i) {
        issue(nB - i);
        if (tid < kCB && nB - i >= 0) sm.ns[(nB - i) % kCarryStages][tid] = load_ns(nB - i);
    }
    uint8_t ns_ahead = load_ns(nB - kCarryStages);
    // phase A ownership: the channel pair cp, cp + 1 and the kQT tokens of quarter qt
    const int cp = (tid & 31) * 2, qt = tid >> 5;
    float2 lw_const = make_float2(0.f, 0.f);
    if (!w_per_token) {
        const float2 wv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(w + (size_t)h * kN + cp));
        lw_const = make_float2(__logf(wv.x), __logf(wv.y));
    }

    auto walk = [&](auto split_tag, const int c, const int part_arg) {
        constexpr bool kSplitHere = decltype(split_tag)::value;
        const int part = kSplitHere ? part_arg : 0;
        const int lo = (kSplitHere && part == 1) ? p_out + 1 : 0, hi = (kSplitHere && part == 0) ? p_out + 1 : kCB;
        CarryStage6& st = sm.st[c % kCarryStages];
        const int t0 = c * kCB;
        if (!kSplitHere || part == 1) {
            cp_async_wait<kCarryStages - 2>();
            __syncthreads();          // step c has landed for everyone; the tiles of step c + 1 are no longer read
            issue(c - (kCarryStages - 1));
            if (tid < kCB && c - (kCarryStages - 1) >= 0) sm.ns[(c - (kCarryStages - 1)) % kCarryStages][tid] = ns_ahead;
            ns_ahead = load_ns(c - kCarryStages);
        } else {
            // the first visit turned r into R0 in place: fetch the rows again for the part in front of `length`
            __syncthreads();
#pragma unroll
            for (int rr = 0; rr < kCB / 16; ++rr) {
                const int row = (tid >> 3) + 16 * rr, piece = (tid & 7) * 8;
                const int t = t0 + row;
                const bool ok = t < Tlen;
                *reinterpret_cast<uint4*>(&st.r[row][piece]) =
                    ok ? *reinterpret_cast<const uint4*>(r + seq_base + (size_t)t * tok_stride + piece) : make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
        }
        if (c == c_out && part == 0 && ds_out != nullptr) {
#pragma unroll
            for (int ni = 0; ni < 8; ++ni)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    acc[ni][e] += __bfloat162float(ds_out[st_base + (size_t)(8 * ni + 2 * q + (e & 1)) * kN + j0 + g + 8 * (e >> 1)]);
        }
        if (warp < kCB / 32) {
            const unsigned m = __ballot_sync(0xffffffffu, sm.ns[c % kCarryStages][32 * warp + lane] != 0);
            if (lane == 0) sm.startmask[warp] = m;
        }
        // the log-decay of this thread's kQT tokens (two channels each), and its sum
        auto lw_of = [&](int tt) -> float2 {
            const int t = kQT * qt + tt;
            const bool ok = t0 + t < Tlen && t >= lo && t < hi;
            return !ok ? make_float2(0.f, 0.f)
                       : (w_per_token ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.w[t][cp])) : lw_const);
        };
        float2 run = make_float2(0.f, 0.f);
#pragma unroll
        for (int tt = 0; tt < kQT; ++tt) {
            const float2 l2 = lw_of(tt);
            run.x += l2.x;
            run.y += l2.y;
        }
        *reinterpret_cast<float2*>(&sm.tot[qt][cp]) = run;
        __syncthreads();
        {
            const unsigned long long starts = (unsigned long long)sm.startmask[0] | (kCB > 32 ? (unsigned long long)sm.startmask[1] << 32 : 0ull);
            auto seg_of = [&](int t) { return __popcll(starts & ((2ull << t) - 1ull)); };
            const int seg_last = seg_of(hi - 1), seg_base = lo > 0 ? seg_of(lo - 1) : 0;
            float2 c_prev = make_float2(0.f, 0.f);         // cumulative log-decay in front of the token
            for (int qq = 0; qq < qt; ++qq) {
                const float2 tq = *reinterpret_cast<const float2*>(&sm.tot[qq][cp]);
                c_prev.x += tq.x;
                c_prev.y += tq.y;
            }
            if (qt == 3)
                *reinterpret_cast<float2*>(&sm.wc[cp]) = seg_last == seg_base ? make_float2(__expf(c_prev.x + run.x), __expf(c_prev.y + run.y))
                                                                               : make_float2(0.f, 0.f);
            int seg = qt > 0 ? seg_of(kQT * qt - 1) : 0;    // number of start flags at or before the token, kept in step
#pragma unroll
            for (int tt = 0; tt < kQT; ++tt) {
                const int t = kQT * qt + tt;
                seg += (int)((starts >> t) & 1ull);
                const bool in_part = t >= lo && t < hi;
                const float2 rv = in_part ? __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&st.r[t][cp])) : make_float2(0.f, 0.f);
                const bool first_seg = seg == seg_base;
                *reinterpret_cast<uint32_t*>(&st.r[t][cp]) =                                   // R0, in place
                    pack2(first_seg ? rv.x * __expf(c_prev.x) : 0.f, first_seg ? rv.y * __expf(c_prev.y) : 0.f);
                const float2 l2 = lw_of(tt);
                c_prev.x += l2.x;
                c_prev.y += l2.y;
            }
        }
        __syncthreads();
        // dS0^T = dS_C^T diag(exp(c_C)) [no start in the step] + dY^T R0
#pragma unroll
        for (int np = 0; np < 4; ++np) {
            const float2 w0 = *reinterpret_cast<const float2*>(&sm.wc[16 * np + 2 * q]);
            const float2 w1 = *reinterpret_cast<const float2*>(&sm.wc[16 * np + 8 + 2 * q]);
            acc[2 * np][0] *= w0.x; acc[2 * np][1] *= w0.y; acc[2 * np][2] *= w0.x; acc[2 * np][3] *= w0.y;
            acc[2 * np + 1][0] *= w1.x; acc[2 * np + 1][1] *= w1.y; acc[2 * np + 1][2] *= w1.x; acc[2 * np + 1][3] *= w1.y;
        }
#pragma unroll
        for (int ks = 0; ks < kCB / 16; ++ks) {
            uint32_t ya[4];
            ldmatrix_x4_trans(ya[0], ya[1], ya[2], ya[3], &st.dy[16 * ks + (mi >> 1) * 8 + r8][j0 + (mi & 1) * 8]);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(b0, b1, b2, b3, &st.r[16 * ks + (mi & 1) * 8 + r8][(2 * np + (mi >> 1)) * 8]);
                mma_bf16(acc[2 * np], ya[0], ya[1], ya[2], ya[3], b0, b1);
                mma_bf16(acc[2 * np + 1], ya[0], ya[1], ya[2], ya[3], b2, b3);
            }
        }
    };
    for (int c = nB - 1; c >= c_stop - 1; --c) {
        // the state gradient behind the last step of a run (before anything of that step is applied), for the CTA of
        // the gradient kernel that walks the run
        if ((c + 1) % run_steps == 0 && c + 1 < nB) {
            bf* dst = dsck + ((size_t)bh * n_runs + c / run_steps) * kN * kN;
#pragma unroll
            for (int ni = 0; ni < 8; ++ni) {
                *reinterpret_cast<uint32_t*>(dst + (size_t)(j0 + g) * kN + 8 * ni + 2 * q) = pack2(acc[ni][0], acc[ni][1]);
                *reinterpret_cast<uint32_t*>(dst + (size_t)(j0 + g + 8) * kN + 8 * ni + 2 * q) = pack2(acc[ni][2], acc[ni][3]);
            }
        }
        if (c < c_stop) break;
        if (split && c == c_out) {
#pragma unroll 1
            for (int part = 1; part >= 0; --part) walk(std::true_type{}, c, part);
        } else {
            walk(std::false_type{}, c, 0);
        }
    }
    cp_async_wait<0>();
}

// du (and the gradient of a constant decay) of a (batch, head): the runs' shares added in a fixed order
__global__ void wkv6_reduce_runs_kernel(int BH, int n_runs, const float* __restrict__ partial, const int* __restrict__ residual_mark,
                                        float* __restrict__ du_head, float* __restrict__ dw_head) {
    if (*residual_mark != 0) return;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= BH * kN) return;
    const int bh = idx / kN, i = idx % kN;
    float su = 0.f, sw = 0.f;
    for (int rho = 0; rho < n_runs; ++rho) {
        su += partial[((size_t)bh * n_runs + rho) * 2 * kN + i];
        if (dw_head != nullptr) sw += partial[((size_t)bh * n_runs + rho) * 2 * kN + kN + i];
    }
    du_head[idx] = su;
    if (dw_head != nullptr) dw_head[idx] = sw;
}

}  // namespace

// How the backward cuts a sequence: runs of 16 chunks (256 tokens) once there are at least two of them.
constexpr int kRunLen = kRunLen6;
static int runs_of(int T) {
    const int nC = (T + kC6 - 1) / kC6;
    return nC >= 2 * kRunLen ? (nC + kRunLen - 1) / kRunLen : 1;
}
struct Layout6 {
    size_t states, dsck, partial, end;
};
static Layout6 layout6(int B, int T, int H) {
    const size_t nC = (size_t)(T + kC6 - 1) / kC6, runs = (size_t)runs_of(T), tile = (size_t)kN * kN * sizeof(bf);
    Layout6 l;
    l.states = 0;                                              // every chunk's entering state, and the second part of a split one
    l.dsck = l.states + (size_t)B * H * (nC + 1) * tile;       // the state gradient at the end of every run (written by the backward)
    l.partial = l.dsck + (size_t)B * H * runs * tile;          // the runs' shares of du and of a constant decay's gradient (fp32)
    l.end = l.partial + (size_t)B * H * runs * 2 * kN * sizeof(float);
    return l;
}

size_t wkv6_chunk_residual_bytes(int B, int T, int H) { return layout6(B, T, H).end; }

int wkv6_chunk_fwd(cudaStream_t st, int B, int T, int H, const void* r, const void* k, const void* v, const void* w,
                   int per_token, const void* u, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                   void* s_out, void* residual, int* residual_mark, int** flag, int* ticket) {
    static DeviceOnce smem_attr;
    if (!smem_attr.ok([]() { return cudaFuncSetAttribute(wkv6_chunk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Fwd6cSmem)); }))
        return B200WKV_ELAUNCH;
    *flag = wkv_call_flag(ticket);
    if (*flag == nullptr) return B200WKV_ELAUNCH;
    wkv6_chunk_fwd_kernel<<<B * H, 128, sizeof(Fwd6cSmem), st>>>(T, H, (const bf*)r, (const bf*)k, (const bf*)v, (const bf*)w, per_token,
                                                                (const bf*)u, (const bf*)s0, length, ns, (bf*)y, (bf*)s_out,
                                                                (bf*)residual, *flag, *ticket, residual_mark);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

int wkv6_chunk_bwd(cudaStream_t st, int B, int T, int H, const void* r, const void* k, const void* v, const void* w,
                   int per_token, const void* u, const uint32_t* length, const uint8_t* ns, const void* dy, const void* ds_out,
                   void* residual, const int* residual_mark, void* dr, void* dk, void* dv, void* dw, void* du, void* ds0) {
    static DeviceOnce smem_attr;
    if (!smem_attr.ok([]() {
            cudaError_t e = cudaFuncSetAttribute(wkv6_chunk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Bwd6cSmem));
            if (e != cudaSuccess) return e;
            return cudaFuncSetAttribute(wkv6_carry_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Carry6Smem));
        }))
        return B200WKV_ELAUNCH;
    const Layout6 lay = layout6(B, T, H);
    char* base = static_cast<char*>(residual);
    const int n_runs = runs_of(T);
    bf* dsck = reinterpret_cast<bf*>(base + lay.dsck);
    float* partial = reinterpret_cast<float*>(base + lay.partial);
    float* dw_head = per_token ? nullptr : (float*)dw;
    if (n_runs > 1) {
        wkv6_carry_bwd_kernel<<<B * H, 128, sizeof(Carry6Smem), st>>>(T, H, (const bf*)r, (const bf*)w, per_token, length, ns, (const bf*)dy,
                                                                     (const bf*)ds_out, residual_mark, n_runs, kRunLen, dsck);
        if (cudaGetLastError() != cudaSuccess) return B200WKV_ELAUNCH;
    }
    wkv6_chunk_bwd_kernel<<<B * H * n_runs, 128, sizeof(Bwd6cSmem), st>>>(
        T, H, (const bf*)r, (const bf*)k, (const bf*)v, (const bf*)w, per_token, (const bf*)u, length, ns, (const bf*)dy,
        (const bf*)ds_out, (const bf*)(base + lay.states), residual_mark, (bf*)dr, (bf*)dk, (bf*)dv, per_token ? (bf*)dw : nullptr,
        dw_head, (float*)du, (bf*)ds0, n_runs, n_runs > 1 ? kRunLen : (T + kC6 - 1) / kC6, dsck, partial);
    if (cudaGetLastError() != cudaSuccess) return B200WKV_ELAUNCH;
    if (n_runs > 1) {
        const int total = B * H * kN;
        wkv6_reduce_runs_kernel<<<(total + 255) / 256, 256, 0, st>>>(B * H, n_runs, partial, residual_mark, (float*)du, dw_head);
        if (cudaGetLastError() != cudaSuccess) return B200WKV_ELAUNCH;
    }
    return B200WKV_OK;
}

}  // namespace b200wkv

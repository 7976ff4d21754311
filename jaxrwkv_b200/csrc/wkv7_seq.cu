// RWKV-7 WKV recurrence, token-sequential CUDA-core kernels (fp32 arithmetic).
//
// These are the exact-arithmetic kernels: one CTA per (batch, head) walks the
// sequence token by token with the 64x64 state held in registers.  They serve the
// fp32 element type (whose 1e-4 tolerance rules out bf16 tensor-core products) and
// are the in-library cross-check for the chunked tensor-core kernels.
//
// Semantics: BaseRWKV.inner_loop of jaxrwkv (src/jaxrwkv/rwkv7.py:199-220); the
// backward is the reverse-time recurrence of the same loop.
#include "common.cuh"
#include "device_once.cuh"

namespace b200wkv {

constexpr int kCk = 16;  // tokens per staged chunk == spacing of the saved state checkpoints

// ------------------------------------------------------------------ forward ---------
// 128 threads per (batch, head).  Warps 0-1 compute: thread i owns the whole row i of S in
// registers, so S.a and S.r are in-thread dot products and every shared-memory read of the
// token vectors is a warp-uniform (broadcast) address.  Warps 2-3 stream: they convert the next
// 16-token chunk into the other shared buffer and write the previous chunk's outputs, so the
// compute warps' instruction stream is only LDS + FMA.
struct FwdSmem {
    float in[2][6][kCk][kN];  // decay, r, k, v, a, b
    float y[2][kCk][kN];
    uint8_t ns[2][kCk];
};

template <typename T>
__global__ void __launch_bounds__(128)
wkv7_seq_fwd_kernel(int Tlen, int H, const T* __restrict__ w, const T* __restrict__ r,
                    const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ a,
                    const T* __restrict__ b, const T* __restrict__ s0,
                    const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                    T* __restrict__ y, T* __restrict__ s_out, float* __restrict__ ckpt,
                    const int* __restrict__ run_if, int run_ticket, int* __restrict__ residual_mark) {
    // As the fallback behind the chunked kernel: run only when that kernel left its ticket in *run_if,
    // and mark the residual as being in this kernel's format.
    if (run_if != nullptr && *run_if != run_ticket) return;
    if (residual_mark != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *residual_mark = 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FwdSmem& sm = *reinterpret_cast<FwdSmem*>(smem_raw);
    const int bh = blockIdx.x, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x;
    const bool streamer = tid >= 64;
    const int i = tid & 63;
    const size_t seq_base = (size_t)bi * Tlen * H * kN + (size_t)h * kN;
    const size_t tok_stride = (size_t)H * kN;
    const T* src[6] = {w, r, k, v, a, b};
    const int L = min((int)length[bi], Tlen);
    const size_t row_base = ((size_t)bh * kN + i) * kN;
    const int nC = (Tlen + kCk - 1) / kCk;

    // streamer: 64 threads move one chunk = 6 streams x 16 tokens x 16 groups of 4 elements
    auto stage = [&](int c, int buf) {
        const int t0 = c * kCk;
#pragma unroll
        for (int m = 0; m < 6; ++m) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int g = i + 64 * u, lt = g >> 4, lc = (g & 15) * 4;
                x[u] = (t0 + lt < Tlen) ? load4(src[m] + seq_base + (size_t)(t0 + lt) * tok_stride + lc)
                                        : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int g = i + 64 * u, lt = g >> 4, lc = (g & 15) * 4;
                if (m == 0) x[u] = make_float4(expf(-expf(x[u].x)), expf(-expf(x[u].y)), expf(-expf(x[u].z)), expf(-expf(x[u].w)));
                *reinterpret_cast<float4*>(&sm.in[buf][m][lt][lc]) = x[u];
            }
        }
        if (i < kCk) sm.ns[buf][i] = (t0 + i < Tlen) ? new_starts[(size_t)bi * Tlen + t0 + i] : 0;
    };
    auto flush_y = [&](int c, int buf) {
        const int t0 = c * kCk;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int g = i + 64 * u, lt = g >> 4, lc = (g & 15) * 4;
            if (t0 + lt < Tlen)
                store4(y + seq_base + (size_t)(t0 + lt) * tok_stride + lc, *reinterpret_cast<const float4*>(&sm.y[buf][lt][lc]));
        }
    };

    float S[kN];
    if (!streamer) {
#pragma unroll
        for (int g = 0; g < 16; ++g) {
            float4 x = load4(s0 + row_base + g * 4);
            S[g * 4 + 0] = x.x; S[g * 4 + 1] = x.y; S[g * 4 + 2] = x.z; S[g * 4 + 3] = x.w;
        }
        if (L == 0) {
#pragma unroll
            for (int g = 0; g < 16; ++g)
                store4(s_out + row_base + g * 4, make_float4(S[g * 4], S[g * 4 + 1], S[g * 4 + 2], S[g * 4 + 3]));
        }
    } else {
        stage(0, 0);
    }
    __syncthreads();

    for (int c = 0; c < nC; ++c) {
        const int buf = c & 1, t0 = c * kCk;
        if (streamer) {
            if (c > 0) flush_y(c - 1, buf ^ 1);
            if (c + 1 < nC) stage(c + 1, buf ^ 1);
        } else {
            if (ckpt != nullptr) {
                float* dst = ckpt + (((size_t)bh * nC + c) * kN + i) * kN;
#pragma unroll
                for (int g = 0; g < 16; ++g)
                    *reinterpret_cast<float4*>(dst + g * 4) = make_float4(S[g * 4], S[g * 4 + 1], S[g * 4 + 2], S[g * 4 + 3]);
            }
            const int nt = min(kCk, Tlen - t0);
            for (int tt = 0; tt < nt; ++tt) {
                if (sm.ns[buf][tt]) {
#pragma unroll
                    for (int j = 0; j < kN; ++j) S[j] = 0.f;
                }
                float sa0 = 0.f, sa1 = 0.f, sa2 = 0.f, sa3 = 0.f;
#pragma unroll
                for (int g = 0; g < 16; ++g) {
                    const float4 av = *reinterpret_cast<const float4*>(&sm.in[buf][4][tt][g * 4]);
                    sa0 = fmaf(S[g * 4 + 0], av.x, sa0); sa1 = fmaf(S[g * 4 + 1], av.y, sa1);
                    sa2 = fmaf(S[g * 4 + 2], av.z, sa2); sa3 = fmaf(S[g * 4 + 3], av.w, sa3);
                }
                const float sa = (sa0 + sa1) + (sa2 + sa3);
                const float vi = sm.in[buf][3][tt][i];
                float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
                for (int g = 0; g < 16; ++g) {
                    const float4 wv = *reinterpret_cast<const float4*>(&sm.in[buf][0][tt][g * 4]);
                    const float4 kv = *reinterpret_cast<const float4*>(&sm.in[buf][2][tt][g * 4]);
                    const float4 bv = *reinterpret_cast<const float4*>(&sm.in[buf][5][tt][g * 4]);
                    const float4 rv = *reinterpret_cast<const float4*>(&sm.in[buf][1][tt][g * 4]);
                    float* s4 = &S[g * 4];
                    s4[0] = fmaf(s4[0], wv.x, fmaf(vi, kv.x, sa * bv.x));
                    s4[1] = fmaf(s4[1], wv.y, fmaf(vi, kv.y, sa * bv.y));
                    s4[2] = fmaf(s4[2], wv.z, fmaf(vi, kv.z, sa * bv.z));
                    s4[3] = fmaf(s4[3], wv.w, fmaf(vi, kv.w, sa * bv.w));
                    y0 = fmaf(s4[0], rv.x, y0); y1 = fmaf(s4[1], rv.y, y1);
                    y2 = fmaf(s4[2], rv.z, y2); y3 = fmaf(s4[3], rv.w, y3);
                }
                sm.y[buf][tt][i] = (y0 + y1) + (y2 + y3);
                if (t0 + tt == L - 1) {
#pragma unroll
                    for (int g = 0; g < 16; ++g)
                        store4(s_out + row_base + g * 4, make_float4(S[g * 4], S[g * 4 + 1], S[g * 4 + 2], S[g * 4 + 3]));
                }
            }
        }
        __syncthreads();
    }
    if (streamer) flush_y(nC - 1, (nC - 1) & 1);
}

// ------------------------------------------------------------------ backward --------
// 256 threads: thread (ti, tj) owns the 4x4 tile rows 4ti.., cols 4tj.. of S and dS, with
// tj = lane%16 and ti = 2*warp + lane/16, so sums over columns stay inside a half-warp and
// sums over rows need one shuffle plus an ordered 8-way add through shared memory.
// Each 16-token chunk is replayed from its checkpoint in two halves of 8 tokens whose
// entering states are kept in registers for the reverse sweep.
struct BwdSmem {
    float in[8][kCk][kN];      // decay, r, k, v, a, b, dy, dwfac (= -exp(w) * decay)
    float sa[kCk][kN];
    float out[6][kCk][kN];     // dw, dr, dk, dv, da, db
    float red[2][8][5][kN];    // per-warp partial column sums: dr, dk, db, dw, da
    uint8_t ns[kCk];
};

template <typename T>
__global__ void __launch_bounds__(256, 1)
wkv7_seq_bwd_kernel(int Tlen, int H, const T* __restrict__ w, const T* __restrict__ r,
                    const T* __restrict__ k, const T* __restrict__ v, const T* __restrict__ a,
                    const T* __restrict__ b, const T* __restrict__ s0,
                    const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                    const T* __restrict__ dy, const T* __restrict__ ds_out,
                    const float* __restrict__ ckpt,
                    T* __restrict__ dw, T* __restrict__ dr, T* __restrict__ dk, T* __restrict__ dv,
                    T* __restrict__ da, T* __restrict__ db, T* __restrict__ ds0, const int* __restrict__ run_if) {
    // as the fallback behind the chunked backward: run only when the forward marked the residual as this kernel's
    if (run_if != nullptr && *run_if == 0) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdSmem& sm = *reinterpret_cast<BwdSmem*>(smem_raw);
    const int bh = blockIdx.x, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tj = lane & 15, ti = warp * 2 + (lane >> 4);
    const size_t seq_base = (size_t)bi * Tlen * H * kN + (size_t)h * kN;
    const size_t tok_stride = (size_t)H * kN;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kCk - 1) / kCk;
    const int lt = tid >> 4, lc = (tid & 15) * 4;
    const T* src[7] = {w, r, k, v, a, b, dy};
    T* dst[6] = {dw, dr, dk, dv, da, db};
    const size_t tile_base = ((size_t)bh * kN + 4 * ti) * kN + 4 * tj;  // + ii*kN + jj

    float dS[4][4];
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) dS[ii][jj] = 0.f;

    int step = 0;  // parity counter for the partial-sum double buffer
    for (int c = nC - 1; c >= 0; --c) {
        const int t0 = c * kCk;
        __syncthreads();
        {   // stage the chunk's inputs
            const int t = t0 + lt;
            float4 x[7];
#pragma unroll
            for (int m = 0; m < 7; ++m) {
                if (t < Tlen && src[m] != nullptr) x[m] = load4(src[m] + seq_base + (size_t)t * tok_stride + lc);
                else x[m] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            const float4 ew = make_float4(expf(x[0].x), expf(x[0].y), expf(x[0].z), expf(x[0].w));
            const float4 dc = make_float4(expf(-ew.x), expf(-ew.y), expf(-ew.z), expf(-ew.w));
            *reinterpret_cast<float4*>(&sm.in[0][lt][lc]) = dc;
            *reinterpret_cast<float4*>(&sm.in[7][lt][lc]) = make_float4(-ew.x * dc.x, -ew.y * dc.y, -ew.z * dc.z, -ew.w * dc.w);
#pragma unroll
            for (int m = 1; m < 7; ++m) *reinterpret_cast<float4*>(&sm.in[m][lt][lc]) = x[m];
            if (tid < kCk) sm.ns[tid] = (t0 + tid < Tlen) ? new_starts[(size_t)bi * Tlen + t0 + tid] : 0;
        }
        __syncthreads();

        for (int hb = 1; hb >= 0; --hb) {
            const int tb = hb * 8;
            if (t0 + tb >= Tlen) continue;
            float S[4][4];
            {
                const float* cp = ckpt + (((size_t)bh * nC + c) * kN + 4 * ti) * kN + 4 * tj;
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    float4 x = *reinterpret_cast<const float4*>(cp + ii * kN);
                    S[ii][0] = x.x; S[ii][1] = x.y; S[ii][2] = x.z; S[ii][3] = x.w;
                }
            }
            auto fwd_step = [&](int t) {  // t = token index inside the chunk; returns with S advanced
                if (sm.ns[t]) {
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) S[ii][jj] = 0.f;
                }
            };
            float hist[8][4][4];
            // forward replay: tokens [0, tb) discarded, tokens [tb, tb+8) recorded
            for (int t = 0; t < tb; ++t) {
                fwd_step(t);
                const float4 a4 = *reinterpret_cast<const float4*>(&sm.in[4][t][4 * tj]);
                const float4 b4 = *reinterpret_cast<const float4*>(&sm.in[5][t][4 * tj]);
                const float4 w4 = *reinterpret_cast<const float4*>(&sm.in[0][t][4 * tj]);
                const float4 k4 = *reinterpret_cast<const float4*>(&sm.in[2][t][4 * tj]);
                const float4 v4 = *reinterpret_cast<const float4*>(&sm.in[3][t][4 * ti]);
                const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    float sa = S[ii][0] * a4.x + S[ii][1] * a4.y + S[ii][2] * a4.z + S[ii][3] * a4.w;
                    sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                    sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                    sa += __shfl_xor_sync(0xffffffffu, sa, 4);
                    sa += __shfl_xor_sync(0xffffffffu, sa, 8);
                    S[ii][0] = fmaf(S[ii][0], w4.x, fmaf(vv[ii], k4.x, sa * b4.x));
                    S[ii][1] = fmaf(S[ii][1], w4.y, fmaf(vv[ii], k4.y, sa * b4.y));
                    S[ii][2] = fmaf(S[ii][2], w4.z, fmaf(vv[ii], k4.z, sa * b4.z));
                    S[ii][3] = fmaf(S[ii][3], w4.w, fmaf(vv[ii], k4.w, sa * b4.w));
                }
            }
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                const int t = tb + tt;
                if (t0 + t < Tlen) {
                    fwd_step(t);
                    const float4 a4 = *reinterpret_cast<const float4*>(&sm.in[4][t][4 * tj]);
                    const float4 b4 = *reinterpret_cast<const float4*>(&sm.in[5][t][4 * tj]);
                    const float4 w4 = *reinterpret_cast<const float4*>(&sm.in[0][t][4 * tj]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&sm.in[2][t][4 * tj]);
                    const float4 v4 = *reinterpret_cast<const float4*>(&sm.in[3][t][4 * ti]);
                    const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) hist[tt][ii][jj] = S[ii][jj];
                        float sa = S[ii][0] * a4.x + S[ii][1] * a4.y + S[ii][2] * a4.z + S[ii][3] * a4.w;
                        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 4);
                        sa += __shfl_xor_sync(0xffffffffu, sa, 8);
                        if (tj == 0) sm.sa[t][4 * ti + ii] = sa;
                        S[ii][0] = fmaf(S[ii][0], w4.x, fmaf(vv[ii], k4.x, sa * b4.x));
                        S[ii][1] = fmaf(S[ii][1], w4.y, fmaf(vv[ii], k4.y, sa * b4.y));
                        S[ii][2] = fmaf(S[ii][2], w4.z, fmaf(vv[ii], k4.z, sa * b4.z));
                        S[ii][3] = fmaf(S[ii][3], w4.w, fmaf(vv[ii], k4.w, sa * b4.w));
                    }
                }
            }
            __syncwarp();
            // reverse sweep over the recorded half
#pragma unroll
            for (int tt = 7; tt >= 0; --tt) {
                const int t = tb + tt;
                if (t0 + t < Tlen) {
                    const float4 w4 = *reinterpret_cast<const float4*>(&sm.in[0][t][4 * tj]);
                    const float4 r4 = *reinterpret_cast<const float4*>(&sm.in[1][t][4 * tj]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&sm.in[2][t][4 * tj]);
                    const float4 a4 = *reinterpret_cast<const float4*>(&sm.in[4][t][4 * tj]);
                    const float4 b4 = *reinterpret_cast<const float4*>(&sm.in[5][t][4 * tj]);
                    const float4 v4 = *reinterpret_cast<const float4*>(&sm.in[3][t][4 * ti]);
                    const float4 g4 = *reinterpret_cast<const float4*>(&sm.in[6][t][4 * ti]);
                    const float4 s4 = *reinterpret_cast<const float4*>(&sm.sa[t][4 * ti]);
                    const float wj[4] = {w4.x, w4.y, w4.z, w4.w}, rj[4] = {r4.x, r4.y, r4.z, r4.w};
                    const float kj[4] = {k4.x, k4.y, k4.z, k4.w}, aj[4] = {a4.x, a4.y, a4.z, a4.w};
                    const float bj[4] = {b4.x, b4.y, b4.z, b4.w}, vi[4] = {v4.x, v4.y, v4.z, v4.w};
                    const float gi[4] = {g4.x, g4.y, g4.z, g4.w}, sai[4] = {s4.x, s4.y, s4.z, s4.w};
                    if (t0 + t == L - 1 && ds_out != nullptr) {
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii) {
                            float4 x = load4(ds_out + tile_base + ii * kN);
                            dS[ii][0] += x.x; dS[ii][1] += x.y; dS[ii][2] += x.z; dS[ii][3] += x.w;
                        }
                    }
                    float pdr[4] = {0, 0, 0, 0}, pdk[4] = {0, 0, 0, 0}, pdb[4] = {0, 0, 0, 0}, pdw[4] = {0, 0, 0, 0};
                    float pdv[4], pdsa[4];
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
                        pdv[ii] = 0.f; pdsa[ii] = 0.f;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const float hs = hist[tt][ii][jj];
                            const float sp = fmaf(hs, wj[jj], fmaf(vi[ii], kj[jj], sai[ii] * bj[jj]));
                            const float d = fmaf(gi[ii], rj[jj], dS[ii][jj]);
                            dS[ii][jj] = d;
                            pdr[jj] = fmaf(sp, gi[ii], pdr[jj]);
                            pdk[jj] = fmaf(d, vi[ii], pdk[jj]);
                            pdb[jj] = fmaf(d, sai[ii], pdb[jj]);
                            pdw[jj] = fmaf(d, hs, pdw[jj]);
                            pdv[ii] = fmaf(d, kj[jj], pdv[ii]);
                            pdsa[ii] = fmaf(d, bj[jj], pdsa[ii]);
                        }
                    }
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
                        for (int m = 1; m < 16; m <<= 1) {
                            pdv[ii] += __shfl_xor_sync(0xffffffffu, pdv[ii], m);
                            pdsa[ii] += __shfl_xor_sync(0xffffffffu, pdsa[ii], m);
                        }
                    }
                    float pda[4] = {0, 0, 0, 0};
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            pda[jj] = fmaf(hist[tt][ii][jj], pdsa[ii], pda[jj]);
                            dS[ii][jj] = fmaf(dS[ii][jj], wj[jj], pdsa[ii] * aj[jj]);
                        }
                    if (sm.ns[t]) {
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) dS[ii][jj] = 0.f;
                    }
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        pdr[jj] += __shfl_xor_sync(0xffffffffu, pdr[jj], 16);
                        pdk[jj] += __shfl_xor_sync(0xffffffffu, pdk[jj], 16);
                        pdb[jj] += __shfl_xor_sync(0xffffffffu, pdb[jj], 16);
                        pdw[jj] += __shfl_xor_sync(0xffffffffu, pdw[jj], 16);
                        pda[jj] += __shfl_xor_sync(0xffffffffu, pda[jj], 16);
                    }
                    const int buf = step & 1;
                    if (lane < 16) {
                        *reinterpret_cast<float4*>(&sm.red[buf][warp][0][4 * tj]) = make_float4(pdr[0], pdr[1], pdr[2], pdr[3]);
                        *reinterpret_cast<float4*>(&sm.red[buf][warp][1][4 * tj]) = make_float4(pdk[0], pdk[1], pdk[2], pdk[3]);
                        *reinterpret_cast<float4*>(&sm.red[buf][warp][2][4 * tj]) = make_float4(pdb[0], pdb[1], pdb[2], pdb[3]);
                        *reinterpret_cast<float4*>(&sm.red[buf][warp][3][4 * tj]) = make_float4(pdw[0], pdw[1], pdw[2], pdw[3]);
                        *reinterpret_cast<float4*>(&sm.red[buf][warp][4][4 * tj]) = make_float4(pda[0], pda[1], pda[2], pda[3]);
                    }
                    if (tj == 0)
                        *reinterpret_cast<float4*>(&sm.out[3][t][4 * ti]) = make_float4(pdv[0], pdv[1], pdv[2], pdv[3]);
                    __syncthreads();
                    ++step;
                    for (int idx = tid; idx < 5 * kN; idx += 256) {
                        const int vec = idx >> 6, col = idx & 63;
                        float s = 0.f;
#pragma unroll
                        for (int wq = 0; wq < 8; ++wq) s += sm.red[buf][wq][vec][col];
                        // red order: dr, dk, db, dw, da  ->  out order: dw, dr, dk, dv, da, db
                        if (vec == 0) sm.out[1][t][col] = s;
                        else if (vec == 1) sm.out[2][t][col] = s;
                        else if (vec == 2) sm.out[5][t][col] = s;
                        else if (vec == 3) sm.out[0][t][col] = s * sm.in[7][t][col];
                        else sm.out[4][t][col] = s;
                    }
                }
            }
        }
        __syncthreads();
        if (t0 + lt < Tlen) {
#pragma unroll
            for (int m = 0; m < 6; ++m)
                store4(dst[m] + seq_base + (size_t)(t0 + lt) * tok_stride + lc,
                       *reinterpret_cast<const float4*>(&sm.out[m][lt][lc]));
        }
    }
    // gradient with respect to the initial state
    if (L == 0 && ds_out != nullptr) {
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
            float4 x = load4(ds_out + tile_base + ii * kN);
            dS[ii][0] += x.x; dS[ii][1] += x.y; dS[ii][2] += x.z; dS[ii][3] += x.w;
        }
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
        store4(ds0 + tile_base + ii * kN, make_float4(dS[ii][0], dS[ii][1], dS[ii][2], dS[ii][3]));
}

// sixteen consecutive state elements of one thread, moved with 16-byte accesses
__device__ __forceinline__ void load16(const float* p, float* f) {
#pragma unroll
    for (int g = 0; g < 4; ++g) *reinterpret_cast<float4*>(f + g * 4) = __ldg(reinterpret_cast<const float4*>(p) + g);
}
__device__ __forceinline__ void load16(const __nv_bfloat16* p, float* f) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p) + g);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 t = __bfloat1622float2(h[e]);
            f[g * 8 + 2 * e] = t.x;
            f[g * 8 + 2 * e + 1] = t.y;
        }
    }
}
__device__ __forceinline__ void store16(float* p, const float* f) {
#pragma unroll
    for (int g = 0; g < 4; ++g) reinterpret_cast<float4*>(p)[g] = *reinterpret_cast<const float4*>(f + g * 4);
}
__device__ __forceinline__ void store16(__nv_bfloat16* p, const float* f) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[g * 8 + 2 * e], f[g * 8 + 2 * e + 1]);
        reinterpret_cast<uint4*>(p)[g] = raw;
    }
}

// ------------------------------------------------------------------ single step -----
// T == 1 (recurrent decoding): the whole cost is reading and writing the 64x64 state once, so the
// kernel is a straight HBM stream.  256 threads per (batch, head): thread (i = tid/4, q = tid%4) owns
// row i, columns 16q..16q+15.  jaxrwkv has no kernel here (it falls back to the unrolled Python loop,
// src/jaxrwkv/rwkv7.py:469-470).
template <typename T>
__global__ void __launch_bounds__(256)
wkv7_step_kernel(int H, const T* __restrict__ w, const T* __restrict__ r, const T* __restrict__ k,
                 const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                 const T* __restrict__ s0, const uint32_t* __restrict__ length,
                 const uint8_t* __restrict__ new_starts, T* __restrict__ y, T* __restrict__ s_out) {
    const int bh = blockIdx.x, bi = bh / H;
    const int tid = threadIdx.x, i = tid >> 2, q = tid & 3;
    __shared__ __align__(16) float vec[6][kN];   // decay, r, k, v, a, b
    const T* src[6] = {w, r, k, v, a, b};
    if (tid < 96) {   // 6 streams x 16 groups of 4 elements
        const int m = tid >> 4, lc = (tid & 15) * 4;
        float4 x = load4(src[m] + (size_t)bh * kN + lc);
        if (m == 0) x = make_float4(expf(-expf(x.x)), expf(-expf(x.y)), expf(-expf(x.z)), expf(-expf(x.w)));
        *reinterpret_cast<float4*>(&vec[m][lc]) = x;
    }
    const size_t st = ((size_t)bh * kN + i) * kN + q * 16;
    float S[16];
    load16(s0 + st, S);
    const bool keep_input = (length[bi] == 0);   // length == 0 returns the input state untouched
    if (keep_input) store16(s_out + st, S);
    if (new_starts[bi]) {
#pragma unroll
        for (int j = 0; j < 16; ++j) S[j] = 0.f;
    }
    __syncthreads();
    float sa = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) sa = fmaf(S[j], vec[4][q * 16 + j], sa);
    sa += __shfl_xor_sync(0xffffffffu, sa, 1);
    sa += __shfl_xor_sync(0xffffffffu, sa, 2);
    const float vi = vec[3][i];
    float yy = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int c = q * 16 + j;
        S[j] = fmaf(S[j], vec[0][c], fmaf(vi, vec[2][c], sa * vec[5][c]));
        yy = fmaf(S[j], vec[1][c], yy);
    }
    yy += __shfl_xor_sync(0xffffffffu, yy, 1);
    yy += __shfl_xor_sync(0xffffffffu, yy, 2);
    if (q == 0) y[(size_t)bh * kN + i] = from_f32<T>(yy);
    if (!keep_input) store16(s_out + st, S);
}

// ------------------------------------------------------------------ launchers -------
size_t wkv7_seq_residual_bytes(int B, int T, int H) {
    return (size_t)B * H * ((T + kCk - 1) / kCk) * kN * kN * sizeof(float);
}

template <typename T>
static int launch_fwd(cudaStream_t st, int B, int Tlen, int H, const void* w, const void* r, const void* k,
                      const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                      const uint8_t* ns, void* y, void* s_out, void* residual, const int* run_if, int run_ticket,
                      int* residual_mark) {
    auto kern = wkv7_seq_fwd_kernel<T>;
    static DeviceOnce smem_attr;   // one per template instance; the attribute is per device
    if (!smem_attr.ok([kern]() { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(FwdSmem)); }))
        return B200WKV_ELAUNCH;
    kern<<<B * H, 128, sizeof(FwdSmem), st>>>(Tlen, H, (const T*)w, (const T*)r, (const T*)k, (const T*)v,
                                              (const T*)a, (const T*)b, (const T*)s0, length, ns, (T*)y,
                                              (T*)s_out, (float*)residual, run_if, run_ticket, residual_mark);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

template <typename T>
static int launch_bwd(cudaStream_t st, int B, int Tlen, int H, const void* w, const void* r, const void* k,
                      const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                      const uint8_t* ns, const void* dy, const void* ds_out, const void* residual, void* dw,
                      void* dr, void* dk, void* dv, void* da, void* db, void* ds0, const int* run_if) {
    auto kern = wkv7_seq_bwd_kernel<T>;
    static DeviceOnce smem_attr;   // one per template instance; the attribute is per device
    if (!smem_attr.ok([kern]() { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(BwdSmem)); }))
        return B200WKV_ELAUNCH;
    kern<<<B * H, 256, sizeof(BwdSmem), st>>>(Tlen, H, (const T*)w, (const T*)r, (const T*)k, (const T*)v,
                                              (const T*)a, (const T*)b, (const T*)s0, length, ns, (const T*)dy,
                                              (const T*)ds_out, (const float*)residual, (T*)dw, (T*)dr, (T*)dk,
                                              (T*)dv, (T*)da, (T*)db, (T*)ds0, run_if);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

int wkv7_step_stream(cudaStream_t st, int dtype, int B, int H, const void* w, const void* r, const void* k, const void* v,
                     const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                     void* s_out, long long s_batch_stride);

int wkv7_step(cudaStream_t st, int dtype, int B, int H, const void* w, const void* r, const void* k, const void* v,
              const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
              void* s_out) {
    // operands on 16-byte and the result state on 32-byte boundaries (every framework allocation is) take the
    // pipelined stream kernel
    const uintptr_t in_bits = reinterpret_cast<uintptr_t>(s0) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(r) |
                              reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(a) |
                              reinterpret_cast<uintptr_t>(b);
    if ((in_bits & 15u) == 0 && (reinterpret_cast<uintptr_t>(s_out) & 31u) == 0)
        return wkv7_step_stream(st, dtype, B, H, w, r, k, v, a, b, s0, length, ns, y, s_out, (long long)H * kN * kN);
    if (dtype == B200WKV_F32)
        wkv7_step_kernel<float><<<B * H, 256, 0, st>>>(H, (const float*)w, (const float*)r, (const float*)k, (const float*)v,
                                                       (const float*)a, (const float*)b, (const float*)s0, length, ns,
                                                       (float*)y, (float*)s_out);
    else
        wkv7_step_kernel<__nv_bfloat16><<<B * H, 256, 0, st>>>(H, (const __nv_bfloat16*)w, (const __nv_bfloat16*)r,
                                                               (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                               (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                               (const __nv_bfloat16*)s0, length, ns, (__nv_bfloat16*)y,
                                                               (__nv_bfloat16*)s_out);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

// run_if / run_ticket / residual_mark: see the kernels; all NULL / 0 for an unconditional call
int wkv7_seq_fwd(cudaStream_t st, int dtype, int B, int T, int H, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* ns, void* y, void* s_out, void* residual, const int* run_if, int run_ticket,
                 int* residual_mark) {
    if (dtype == B200WKV_F32)
        return launch_fwd<float>(st, B, T, H, w, r, k, v, a, b, s0, length, ns, y, s_out, residual, run_if, run_ticket, residual_mark);
    return launch_fwd<__nv_bfloat16>(st, B, T, H, w, r, k, v, a, b, s0, length, ns, y, s_out, residual, run_if, run_ticket, residual_mark);
}

int wkv7_seq_bwd(cudaStream_t st, int dtype, int B, int T, int H, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* ns, const void* dy, const void* ds_out, const void* residual, void* dw, void* dr,
                 void* dk, void* dv, void* da, void* db, void* ds0, const int* run_if) {
    if (dtype == B200WKV_F32)
        return launch_bwd<float>(st, B, T, H, w, r, k, v, a, b, s0, length, ns, dy, ds_out, residual, dw, dr, dk, dv, da, db, ds0, run_if);
    return launch_bwd<__nv_bfloat16>(st, B, T, H, w, r, k, v, a, b, s0, length, ns, dy, ds_out, residual, dw, dr, dk, dv, da, db, ds0, run_if);
}

}  // namespace b200wkv

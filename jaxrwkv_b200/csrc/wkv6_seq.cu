// RWKV-5 / 5.2 / 6 WKV recurrence, token-sequential CUDA-core kernels (fp32 arithmetic).
//
// State S is indexed [key][value] (transposed with respect to RWKV-7):
//   y_t[v] = sum_k r_t[k] (u[k] k_t[k] v_t[v] + S[k][v])      (state before the update)
//   S[k][v] <- k_t[k] v_t[v] + d_t[k] S[k][v]
// The decay d comes either per token as exp(w_t) (RWKV-6) or as one constant vector per head
// (RWKV-5 / 5.2).  Semantics: BaseRWKV.inner_loop of jaxrwkv, src/jaxrwkv/rwkv6.py:174-191,
// rwkv5_2.py:164-180, rwkv5.py:161-177; the backward is the reverse-time recurrence of that loop.
#include "common.cuh"
#include "device_once.cuh"

namespace b200wkv {

namespace {
constexpr int kCk6 = 16;  // tokens per staged chunk == checkpoint spacing

struct DecaySrc {
    const void* w;        // v6: (B,T,H,N) log-decay ; v5/5.2: (H,N) decay
    int per_token;        // 1: index by (b,t,h) and apply exp ; 0: index by h only, use as is
};

// ------------------------------------------------------------------ forward ---------
// 192 threads: warps 0-3 compute, thread (v = tid % 64, half = tid / 64) owns keys 32 half .. 32 half + 31 of
// column v of S: the output is an in-thread dot product over its keys (the two halves are added when the
// chunk's outputs are flushed) and every token-vector read is a warp-uniform broadcast; warps 4-5 stream the
// next chunk.  Half a column per thread halves the dependent instruction stream per token and the registers,
// so that four CTAs fit on an SM.
struct Fwd6Smem {
    float in[2][4][kCk6][kN];  // decay, r, k, v
    float y[2][2][kCk6][kN];   // partial outputs of the two key halves
    uint8_t ns[2][kCk6];
};

template <typename T>
__global__ void __launch_bounds__(192, 4)
wkv6_seq_fwd_kernel(int Tlen, int H, const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                    const T* __restrict__ w, int w_per_token, const T* __restrict__ u, const T* __restrict__ s0,
                    const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts, T* __restrict__ y,
                    T* __restrict__ s_out, float* __restrict__ ckpt, const int* __restrict__ run_if, int run_ticket,
                    int* __restrict__ residual_mark) {
    // As the fallback behind the chunked kernel: run only when that kernel left its ticket in *run_if, and
    // mark the residual as being in this kernel's format.
    if (run_if != nullptr && *run_if != run_ticket) return;
    if (residual_mark != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *residual_mark = 1;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Fwd6Smem& sm = *reinterpret_cast<Fwd6Smem*>(smem_raw);
    const int bh = blockIdx.x, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x;
    const bool streamer = tid >= 128;
    const int i = tid & 63, half = (tid >> 6) & 1, k0 = half * 32;
    const size_t seq_base = (size_t)bi * Tlen * H * kN + (size_t)h * kN;
    const size_t tok_stride = (size_t)H * kN;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kCk6 - 1) / kCk6;
    const T* src[3] = {r, k, v};

    auto stage = [&](int c, int buf) {
        const int t0 = c * kCk6;
#pragma unroll
        for (int u4 = 0; u4 < 4; ++u4) {
            const int g = i + 64 * u4, lt = g >> 4, lc = (g & 15) * 4;
            const bool ok = t0 + lt < Tlen;
            float4 d4;
            if (w_per_token) {
                d4 = ok ? load4(w + seq_base + (size_t)(t0 + lt) * tok_stride + lc) : make_float4(0.f, 0.f, 0.f, 0.f);
                d4 = make_float4(expf(d4.x), expf(d4.y), expf(d4.z), expf(d4.w));
            } else {
                d4 = load4(w + (size_t)h * kN + lc);
            }
            *reinterpret_cast<float4*>(&sm.in[buf][0][lt][lc]) = d4;
#pragma unroll
            for (int m = 0; m < 3; ++m) {
                const float4 x = ok ? load4(src[m] + seq_base + (size_t)(t0 + lt) * tok_stride + lc) : make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(&sm.in[buf][m + 1][lt][lc]) = x;
            }
        }
        if (i < kCk6) sm.ns[buf][i] = (t0 + i < Tlen) ? new_starts[(size_t)bi * Tlen + t0 + i] : 0;
    };
    auto flush_y = [&](int c, int buf) {
        const int t0 = c * kCk6;
#pragma unroll
        for (int u4 = 0; u4 < 4; ++u4) {
            const int g = i + 64 * u4, lt = g >> 4, lc = (g & 15) * 4;
            if (t0 + lt < Tlen) {
                const float4 a = *reinterpret_cast<const float4*>(&sm.y[buf][0][lt][lc]);
                const float4 b = *reinterpret_cast<const float4*>(&sm.y[buf][1][lt][lc]);
                store4(y + seq_base + (size_t)(t0 + lt) * tok_stride + lc, make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w));
            }
        }
    };

    float S[32], uu[32];
    if (!streamer) {
#pragma unroll
        for (int kk = 0; kk < 32; ++kk) {
            S[kk] = to_f32(s0[((size_t)bh * kN + k0 + kk) * kN + i]);
            uu[kk] = to_f32(u[(size_t)h * kN + k0 + kk]);
        }
        if (L == 0) {
#pragma unroll
            for (int kk = 0; kk < 32; ++kk) s_out[((size_t)bh * kN + k0 + kk) * kN + i] = from_f32<T>(S[kk]);
        }
    } else {
        stage(0, 0);
    }
    __syncthreads();

    for (int c = 0; c < nC; ++c) {
        const int buf = c & 1, t0 = c * kCk6;
        if (streamer) {
            if (c > 0) flush_y(c - 1, buf ^ 1);
            if (c + 1 < nC) stage(c + 1, buf ^ 1);
        } else {
            if (ckpt != nullptr) {
                float* dst = ckpt + ((size_t)bh * nC + c) * kN * kN + (size_t)k0 * kN + i;
#pragma unroll
                for (int kk = 0; kk < 32; ++kk) dst[kk * kN] = S[kk];
            }
            const int nt = min(kCk6, Tlen - t0);
            for (int tt = 0; tt < nt; ++tt) {
                if (sm.ns[buf][tt]) {
#pragma unroll
                    for (int kk = 0; kk < 32; ++kk) S[kk] = 0.f;
                }
                const float vi = sm.in[buf][3][tt][i];
                float y0 = 0.f, y1 = 0.f, y2 = 0.f, y3 = 0.f;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const float4 dv = *reinterpret_cast<const float4*>(&sm.in[buf][0][tt][k0 + g * 4]);
                    const float4 rv = *reinterpret_cast<const float4*>(&sm.in[buf][1][tt][k0 + g * 4]);
                    const float4 kv = *reinterpret_cast<const float4*>(&sm.in[buf][2][tt][k0 + g * 4]);
                    float* s4 = &S[g * 4];
                    const float* u4 = &uu[g * 4];
                    const float a0 = kv.x * vi, a1 = kv.y * vi, a2 = kv.z * vi, a3 = kv.w * vi;
                    y0 = fmaf(rv.x, fmaf(u4[0], a0, s4[0]), y0); y1 = fmaf(rv.y, fmaf(u4[1], a1, s4[1]), y1);
                    y2 = fmaf(rv.z, fmaf(u4[2], a2, s4[2]), y2); y3 = fmaf(rv.w, fmaf(u4[3], a3, s4[3]), y3);
                    s4[0] = fmaf(dv.x, s4[0], a0); s4[1] = fmaf(dv.y, s4[1], a1);
                    s4[2] = fmaf(dv.z, s4[2], a2); s4[3] = fmaf(dv.w, s4[3], a3);
                }
                sm.y[buf][half][tt][i] = (y0 + y1) + (y2 + y3);
                if (t0 + tt == L - 1) {
#pragma unroll
                    for (int kk = 0; kk < 32; ++kk) s_out[((size_t)bh * kN + k0 + kk) * kN + i] = from_f32<T>(S[kk]);
                }
            }
        }
        __syncthreads();
    }
    if (streamer) flush_y(nC - 1, (nC - 1) & 1);
}

// ------------------------------------------------------------------ backward --------
// 256 threads: thread (ti, tj) owns the 4x4 tile keys 4ti.., values 4tj.. of S and dS, tj = lane%16,
// ti = 2*warp + lane/16.  Sums over values stay inside a half-warp; sums over keys take one shuffle plus an
// ordered 8-way add through shared memory.  Each 16-token chunk is replayed from its checkpoint in
// two halves of 8 tokens whose entering states are kept in registers for the reverse sweep.
struct Bwd6Smem {
    float in[5][kCk6][kN];     // decay, r, k, v, dy
    float dyv[kCk6];           // dy_t . v_t
    float ruk[kCk6];           // sum_k r u k
    float out[4][kCk6][kN];    // dr, dk, dv, dw (per token; dw only for per-token decay)
    float red[2][8][kN];       // per-warp partial key sums for dv
    float uu[kN];
    uint8_t ns[kCk6];
};

template <typename T>
__global__ void __launch_bounds__(256, 2)
wkv6_seq_bwd_kernel(int Tlen, int H, const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                    const T* __restrict__ w, int w_per_token, const T* __restrict__ u,
                    const uint32_t* __restrict__ length, const uint8_t* __restrict__ new_starts,
                    const T* __restrict__ dy, const T* __restrict__ ds_out, const float* __restrict__ ckpt,
                    T* __restrict__ dr, T* __restrict__ dk, T* __restrict__ dv, T* __restrict__ dw_tok,
                    float* __restrict__ dw_head, float* __restrict__ du_head, T* __restrict__ ds0,
                    const int* __restrict__ run_if) {
    if (run_if != nullptr && *run_if == 0) return;   // the residual is in the chunked kernels' format
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Bwd6Smem& sm = *reinterpret_cast<Bwd6Smem*>(smem_raw);
    const int bh = blockIdx.x, bi = bh / H, h = bh % H;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tj = lane & 15, ti = warp * 2 + (lane >> 4);
    const size_t seq_base = (size_t)bi * Tlen * H * kN + (size_t)h * kN;
    const size_t tok_stride = (size_t)H * kN;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kCk6 - 1) / kCk6;
    const int lt = tid >> 4, lc = (tid & 15) * 4;
    const T* src[4] = {r, k, v, dy};
    T* dst[4] = {dr, dk, dv, dw_tok};
    const size_t tile_base = ((size_t)bh * kN + 4 * ti) * kN + 4 * tj;

    if (tid < kN) sm.uu[tid] = to_f32(u[(size_t)h * kN + tid]);
    float dS[4][4];
    float du_acc[4] = {0.f, 0.f, 0.f, 0.f}, dd_acc[4] = {0.f, 0.f, 0.f, 0.f};   // per key row, summed over tokens
#pragma unroll
    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) dS[ii][jj] = 0.f;

    int step = 0;
    for (int c = nC - 1; c >= 0; --c) {
        const int t0 = c * kCk6;
        __syncthreads();
        {
            const int t = t0 + lt;
            const bool ok = t < Tlen;
            float4 d4;
            if (w_per_token) {
                d4 = ok ? load4(w + seq_base + (size_t)t * tok_stride + lc) : make_float4(0.f, 0.f, 0.f, 0.f);
                d4 = make_float4(expf(d4.x), expf(d4.y), expf(d4.z), expf(d4.w));
            } else {
                d4 = load4(w + (size_t)h * kN + lc);
            }
            *reinterpret_cast<float4*>(&sm.in[0][lt][lc]) = d4;
            float4 x[4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                x[m] = (ok && src[m] != nullptr) ? load4(src[m] + seq_base + (size_t)t * tok_stride + lc) : make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(&sm.in[m + 1][lt][lc]) = x[m];
            }
            // per-token scalars: dy.v and sum r u k, reduced over the 16 threads that staged the token
            const float4 u4 = *reinterpret_cast<const float4*>(&sm.uu[lc]);
            float a = x[3].x * x[2].x + x[3].y * x[2].y + x[3].z * x[2].z + x[3].w * x[2].w;
            float bq = x[0].x * u4.x * x[1].x + x[0].y * u4.y * x[1].y + x[0].z * u4.z * x[1].z + x[0].w * u4.w * x[1].w;
#pragma unroll
            for (int m = 1; m < 16; m <<= 1) {
                a += __shfl_xor_sync(0xffffffffu, a, m);
                bq += __shfl_xor_sync(0xffffffffu, bq, m);
            }
            if ((tid & 15) == 0) { sm.dyv[lt] = a; sm.ruk[lt] = bq; }
            if (tid < kCk6) sm.ns[tid] = (t0 + tid < Tlen) ? new_starts[(size_t)bi * Tlen + t0 + tid] : 0;
        }
        __syncthreads();

        for (int hb = 1; hb >= 0; --hb) {
            const int tb = hb * 8;
            if (t0 + tb >= Tlen) continue;
            float S[4][4];
            {
                const float* cp = ckpt + ((size_t)bh * nC + c) * kN * kN + (4 * ti) * kN + 4 * tj;
#pragma unroll
                for (int ii = 0; ii < 4; ++ii) {
                    float4 x = *reinterpret_cast<const float4*>(cp + ii * kN);
                    S[ii][0] = x.x; S[ii][1] = x.y; S[ii][2] = x.z; S[ii][3] = x.w;
                }
            }
            auto advance = [&](int t) {
                if (sm.ns[t]) {
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) S[ii][jj] = 0.f;
                }
            };
            auto update = [&](int t) {
                const float4 d4 = *reinterpret_cast<const float4*>(&sm.in[0][t][4 * ti]);
                const float4 k4 = *reinterpret_cast<const float4*>(&sm.in[2][t][4 * ti]);
                const float4 v4 = *reinterpret_cast<const float4*>(&sm.in[3][t][4 * tj]);
                const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
                const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
                for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) S[ii][jj] = fmaf(dd[ii], S[ii][jj], kk[ii] * vv[jj]);
            };
            float hist[8][4][4];
            for (int t = 0; t < tb; ++t) { advance(t); update(t); }
#pragma unroll
            for (int tt = 0; tt < 8; ++tt) {
                const int t = tb + tt;
                if (t0 + t < Tlen) {
                    advance(t);
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) hist[tt][ii][jj] = S[ii][jj];
                    update(t);
                }
            }
#pragma unroll
            for (int tt = 7; tt >= 0; --tt) {
                const int t = tb + tt;
                if (t0 + t < Tlen) {
                    const float4 d4 = *reinterpret_cast<const float4*>(&sm.in[0][t][4 * ti]);
                    const float4 r4 = *reinterpret_cast<const float4*>(&sm.in[1][t][4 * ti]);
                    const float4 k4 = *reinterpret_cast<const float4*>(&sm.in[2][t][4 * ti]);
                    const float4 u4 = *reinterpret_cast<const float4*>(&sm.uu[4 * ti]);
                    const float4 v4 = *reinterpret_cast<const float4*>(&sm.in[3][t][4 * tj]);
                    const float4 g4 = *reinterpret_cast<const float4*>(&sm.in[4][t][4 * tj]);
                    const float di[4] = {d4.x, d4.y, d4.z, d4.w}, ri[4] = {r4.x, r4.y, r4.z, r4.w};
                    const float ki[4] = {k4.x, k4.y, k4.z, k4.w}, ui[4] = {u4.x, u4.y, u4.z, u4.w};
                    const float vj[4] = {v4.x, v4.y, v4.z, v4.w}, gj[4] = {g4.x, g4.y, g4.z, g4.w};
                    const float dyv = sm.dyv[t], ruk = sm.ruk[t];
                    if (t0 + t == L - 1 && ds_out != nullptr) {
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii) {
                            float4 x = load4(ds_out + tile_base + ii * kN);
                            dS[ii][0] += x.x; dS[ii][1] += x.y; dS[ii][2] += x.z; dS[ii][3] += x.w;
                        }
                    }
                    float pdr[4], pdk[4], pdd[4], pdv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
                        pdr[ii] = 0.f; pdk[ii] = 0.f; pdd[ii] = 0.f;
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const float hs = hist[tt][ii][jj], d = dS[ii][jj];
                            pdr[ii] = fmaf(hs, gj[jj], pdr[ii]);
                            pdk[ii] = fmaf(d, vj[jj], pdk[ii]);
                            pdd[ii] = fmaf(d, hs, pdd[ii]);
                            pdv[jj] = fmaf(d, ki[ii], pdv[jj]);
                            dS[ii][jj] = fmaf(di[ii], d, ri[ii] * gj[jj]);
                        }
                    }
#pragma unroll
                    for (int ii = 0; ii < 4; ++ii) {
#pragma unroll
                        for (int m = 1; m < 16; m <<= 1) {
                            pdr[ii] += __shfl_xor_sync(0xffffffffu, pdr[ii], m);
                            pdk[ii] += __shfl_xor_sync(0xffffffffu, pdk[ii], m);
                            pdd[ii] += __shfl_xor_sync(0xffffffffu, pdd[ii], m);
                        }
                    }
                    if (sm.ns[t]) {
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii)
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) dS[ii][jj] = 0.f;
                    }
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) pdv[jj] += __shfl_xor_sync(0xffffffffu, pdv[jj], 16);
                    const int buf = step & 1;
                    if (lane < 16) *reinterpret_cast<float4*>(&sm.red[buf][warp][4 * tj]) = make_float4(pdv[0], pdv[1], pdv[2], pdv[3]);
                    if (tj == 0) {
                        float o_r[4], o_k[4], o_w[4];
#pragma unroll
                        for (int ii = 0; ii < 4; ++ii) {
                            o_r[ii] = fmaf(ui[ii] * ki[ii], dyv, pdr[ii]);
                            o_k[ii] = fmaf(ri[ii] * ui[ii], dyv, pdk[ii]);
                            o_w[ii] = pdd[ii] * di[ii];             // gradient of the log-decay (per-token decay)
                            du_acc[ii] = fmaf(ri[ii] * ki[ii], dyv, du_acc[ii]);
                            dd_acc[ii] += pdd[ii];                   // gradient of a constant decay
                        }
                        *reinterpret_cast<float4*>(&sm.out[0][t][4 * ti]) = make_float4(o_r[0], o_r[1], o_r[2], o_r[3]);
                        *reinterpret_cast<float4*>(&sm.out[1][t][4 * ti]) = make_float4(o_k[0], o_k[1], o_k[2], o_k[3]);
                        *reinterpret_cast<float4*>(&sm.out[3][t][4 * ti]) = make_float4(o_w[0], o_w[1], o_w[2], o_w[3]);
                    }
                    __syncthreads();
                    ++step;
                    if (tid < kN) {
                        float s = 0.f;
#pragma unroll
                        for (int wq = 0; wq < 8; ++wq) s += sm.red[buf][wq][tid];
                        sm.out[2][t][tid] = fmaf(ruk, sm.in[4][t][tid], s);
                    }
                }
            }
        }
        __syncthreads();
        if (t0 + lt < Tlen) {
#pragma unroll
            for (int m = 0; m < 4; ++m)
                if (dst[m] != nullptr)
                    store4(dst[m] + seq_base + (size_t)(t0 + lt) * tok_stride + lc, *reinterpret_cast<const float4*>(&sm.out[m][lt][lc]));
        }
    }
    if (L == 0 && ds_out != nullptr) {
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
            float4 x = load4(ds_out + tile_base + ii * kN);
            dS[ii][0] += x.x; dS[ii][1] += x.y; dS[ii][2] += x.z; dS[ii][3] += x.w;
        }
    }
#pragma unroll
    for (int ii = 0; ii < 4; ++ii) store4(ds0 + tile_base + ii * kN, make_float4(dS[ii][0], dS[ii][1], dS[ii][2], dS[ii][3]));
    if (tj == 0) {
        *reinterpret_cast<float4*>(du_head + (size_t)bh * kN + 4 * ti) = make_float4(du_acc[0], du_acc[1], du_acc[2], du_acc[3]);
        if (dw_head != nullptr)
            *reinterpret_cast<float4*>(dw_head + (size_t)bh * kN + 4 * ti) = make_float4(dd_acc[0], dd_acc[1], dd_acc[2], dd_acc[3]);
    }
}

template <typename T>
int launch_fwd6(cudaStream_t st, int B, int Tlen, int H, const void* r, const void* k, const void* v, const void* w,
                int per_token, const void* u, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                void* s_out, void* residual, const int* run_if, int run_ticket, int* residual_mark) {
    auto kern = wkv6_seq_fwd_kernel<T>;
    static DeviceOnce smem_attr;   // one per template instance; the attribute is per device
    if (!smem_attr.ok([kern]() { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Fwd6Smem)); }))
        return B200WKV_ELAUNCH;
    kern<<<B * H, 192, sizeof(Fwd6Smem), st>>>(Tlen, H, (const T*)r, (const T*)k, (const T*)v, (const T*)w, per_token,
                                               (const T*)u, (const T*)s0, length, ns, (T*)y, (T*)s_out, (float*)residual,
                                               run_if, run_ticket, residual_mark);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

template <typename T>
int launch_bwd6(cudaStream_t st, int B, int Tlen, int H, const void* r, const void* k, const void* v, const void* w,
                int per_token, const void* u, const uint32_t* length, const uint8_t* ns, const void* dy,
                const void* ds_out, const void* residual, void* dr, void* dk, void* dv, void* dw, void* du, void* ds0,
                const int* run_if) {
    auto kern = wkv6_seq_bwd_kernel<T>;
    static DeviceOnce smem_attr;   // one per template instance; the attribute is per device
    if (!smem_attr.ok([kern]() { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Bwd6Smem)); }))
        return B200WKV_ELAUNCH;
    kern<<<B * H, 256, sizeof(Bwd6Smem), st>>>(Tlen, H, (const T*)r, (const T*)k, (const T*)v, (const T*)w, per_token,
                                               (const T*)u, length, ns, (const T*)dy, (const T*)ds_out,
                                               (const float*)residual, (T*)dr, (T*)dk, (T*)dv,
                                               per_token ? (T*)dw : nullptr, per_token ? nullptr : (float*)dw,
                                               (float*)du, (T*)ds0, run_if);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}
}  // namespace

size_t wkv6_seq_residual_bytes(int B, int T, int H) {
    return (size_t)B * H * ((T + kCk6 - 1) / kCk6) * kN * kN * sizeof(float);
}

int wkv6_seq_fwd(cudaStream_t st, int dtype, int B, int T, int H, const void* r, const void* k, const void* v,
                 const void* w, int per_token, const void* u, const void* s0, const uint32_t* length,
                 const uint8_t* ns, void* y, void* s_out, void* residual, const int* run_if, int run_ticket,
                 int* residual_mark) {
    if (dtype == B200WKV_F32)
        return launch_fwd6<float>(st, B, T, H, r, k, v, w, per_token, u, s0, length, ns, y, s_out, residual, run_if, run_ticket, residual_mark);
    return launch_fwd6<__nv_bfloat16>(st, B, T, H, r, k, v, w, per_token, u, s0, length, ns, y, s_out, residual, run_if, run_ticket,
                                      residual_mark);
}

int wkv6_seq_bwd(cudaStream_t st, int dtype, int B, int T, int H, const void* r, const void* k, const void* v,
                 const void* w, int per_token, const void* u, const uint32_t* length, const uint8_t* ns,
                 const void* dy, const void* ds_out, const void* residual, void* dr, void* dk, void* dv, void* dw,
                 void* du, void* ds0, const int* run_if) {
    if (dtype == B200WKV_F32)
        return launch_bwd6<float>(st, B, T, H, r, k, v, w, per_token, u, length, ns, dy, ds_out, residual, dr, dk, dv, dw, du, ds0, run_if);
    return launch_bwd6<__nv_bfloat16>(st, B, T, H, r, k, v, w, per_token, u, length, ns, dy, ds_out, residual, dr, dk, dv, dw, du, ds0,
                                      run_if);
}

}  // namespace b200wkv

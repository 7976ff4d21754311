// The elementwise work on either side of the RWKV-7 recurrence inside jaxrwkv's time mixing
// (src/jaxrwkv/rwkv7.py:238-252 before the operator, :263-265 after it), each side as ONE pass over its
// streams, forward and backward:
//
//   before:  w  = -softplus(-(w0 + wl)) - 0.5                       (rwkv7.py:238, wl = the decay LoRA's output)
//            a  = sigmoid(a0 + al)                                  (:245)
//            v' = v + (v_first - v) * sigmoid(v0 + vl)              (:243, layers after the first)
//            kk = normalise_per_head(k * k_k)                       (:248-251, norm clamped at 1e-12)
//            k' = k * (1 + (a - 1) * k_a)                           (:252)
//            a_i = -kk,  b_i = kk * a                               (:257)
//   after:   x = (group_norm_per_head(y) * ln_w + ln_b + (sum_j r_j k'_j r_k_j) * v') * g    (:263-265)
//
// Rows are tokens (B*T of them), a row has H heads of 64 channels.  A thread owns eight consecutive channels
// (16 bytes of bf16) of a fixed position in the row and walks rows with the grid's stride, so the per-channel
// parameters stay in registers and the parameter gradients accumulate in registers, leaving one fp32 partial
// sum per thread that the caller adds up (deterministic: no atomics).  The eight lanes of a head reduce the
// per-head sums with three shuffles.  Everything is computed in fp32 whatever the element type.
#include "common.cuh"
#include "device_once.cuh"

namespace b200wkv {

namespace {

constexpr int kOct = 8;   // channels per thread
#ifndef MIX_THREADS_PER_SM
#define MIX_THREADS_PER_SM 512
#endif
#define MIX_MINB(MAXT) (MIX_THREADS_PER_SM / (MAXT) > 0 ? MIX_THREADS_PER_SM / (MAXT) : 1)

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* f);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        f[2 * e] = __uint_as_float(w[e] << 16);
        f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
    }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float* f);
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

// Eight elements as they lie in memory: the loads of an iteration are all issued before the first is unpacked,
// and what waits in registers is the packed form (4 registers per bf16 octet).
template <typename T> struct Raw;
template <> struct Raw<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) {
        a = *reinterpret_cast<const float4*>(p);
        b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ void get(float* f) const {
        f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    }
};
template <> struct Raw<__nv_bfloat16> {
    uint4 raw;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void get(float* f) const {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            f[2 * e] = __uint_as_float(w[e] << 16);
            f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
    }
};

__device__ __forceinline__ float head_sum(float x) {   // over the eight lanes that hold one head of one row
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    x += __shfl_xor_sync(0xffffffffu, x, 4);
    return x;
}
// The kernels are bound by HBM only if their arithmetic stays cheap: exp / log / reciprocal as single
// special-function instructions (relative error ~1e-7 on results of magnitude >= 1e-2 here).
__device__ __forceinline__ float sigmoidf(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// softplus(x) = log(1 + e^x), stable on both sides; the result is only ever used as -softplus - 0.5
__device__ __forceinline__ float softplusf(float x) { return fmaxf(x, 0.f) + __logf(1.f + __expf(-fabsf(x))); }

// A block holds `rows_per_block` rows side by side; thread t: row slot t / (C/8), channels 8 * (t % (C/8)).
struct Walk {
    int row, row_step, c;
    bool live;
};
__device__ __forceinline__ Walk make_walk(int C) {
    const int per_row = C / kOct;
    Walk w;
    const int slot = threadIdx.x / per_row, slots = blockDim.x / per_row;
    w.c = (threadIdx.x % per_row) * kOct;
    w.row = blockIdx.x * slots + slot;
    w.row_step = gridDim.x * slots;
    w.live = slot < slots;
    return w;
}

constexpr float kNormFloor = 1e-12f;

template <typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, MIX_MINB(MAXT))
mix_pre_fwd_kernel(int rows, int C, int use_vmix, const T* __restrict__ k, const T* __restrict__ wl, const T* __restrict__ al,
                   const T* __restrict__ v, const T* __restrict__ vf, const T* __restrict__ vl,
                   const T* __restrict__ w0, const T* __restrict__ a0, const T* __restrict__ v0,
                   const T* __restrict__ k_k, const T* __restrict__ k_a, T* __restrict__ w_out, T* __restrict__ kp_out,
                   T* __restrict__ vp_out, T* __restrict__ ai_out, T* __restrict__ bi_out) {
    const Walk wk = make_walk(C);
    if (!wk.live) return;
    float pw0[8], pa0[8], pv0[8], pkk[8], pka[8];
    load8(w0 + wk.c, pw0); load8(a0 + wk.c, pa0); load8(k_k + wk.c, pkk); load8(k_a + wk.c, pka);
    if (use_vmix) load8(v0 + wk.c, pv0);
    // rows beyond the end still take part in the shuffles (their lanes share a warp with live rows)
    const int n_it = (rows - (int)(blockIdx.x * (blockDim.x / (C / kOct))) + wk.row_step - 1) / wk.row_step;
    for (int it = 0, row = wk.row; it < n_it; ++it, row += wk.row_step) {
        const bool in = row < rows;
        const size_t off = (size_t)(in ? row : 0) * C + wk.c;
        Raw<T> qk, qw, qa, qv, qf, ql;
        qk.load(k + off); qa.load(al + off); qw.load(wl + off); qv.load(v + off);
        if (use_vmix) { qf.load(vf + off); ql.load(vl + off); }
        float xk[8], xa[8], u[8], n2 = 0.f;
        qk.get(xk); qa.get(xa);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            u[e] = xk[e] * pkk[e];
            n2 = fmaf(u[e], u[e], n2);
        }
        const float inv = 1.f / fmaxf(sqrtf(head_sum(n2)), kNormFloor);
        {
            float okp[8], oai[8], obi[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = sigmoidf(pa0[e] + xa[e]);
                const float kk = u[e] * inv;
                okp[e] = xk[e] * (1.f + (a - 1.f) * pka[e]);
                oai[e] = -kk;
                obi[e] = kk * a;
            }
            if (in) { store8(kp_out + off, okp); store8(ai_out + off, oai); store8(bi_out + off, obi); }
        }
        {
            float xw[8];
            qw.get(xw);
#pragma unroll
            for (int e = 0; e < 8; ++e) xw[e] = -softplusf(-(pw0[e] + xw[e])) - 0.5f;
            if (in) store8(w_out + off, xw);
        }
        {
            float xv[8];
            qv.get(xv);
            if (use_vmix) {
                float xf[8], xl[8];
                qf.get(xf); ql.get(xl);
#pragma unroll
                for (int e = 0; e < 8; ++e) xv[e] = xv[e] + (xf[e] - xv[e]) * sigmoidf(pv0[e] + xl[e]);
            }
            if (in) store8(vp_out + off, xv);
        }
    }
}

// partial: [gridDim.x * slots][5][C] fp32 in the order dw0, da0, dv0, dk_k, dk_a
template <typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, MIX_MINB(MAXT))
mix_pre_bwd_kernel(int rows, int C, int use_vmix, const T* __restrict__ k, const T* __restrict__ wl, const T* __restrict__ al,
                   const T* __restrict__ v, const T* __restrict__ vf, const T* __restrict__ vl,
                   const T* __restrict__ w0, const T* __restrict__ a0, const T* __restrict__ v0,
                   const T* __restrict__ k_k, const T* __restrict__ k_a, const T* __restrict__ gw, const T* __restrict__ gkp,
                   const T* __restrict__ gvp, const T* __restrict__ gai, const T* __restrict__ gbi, T* __restrict__ dk,
                   T* __restrict__ dwl, T* __restrict__ dal, T* __restrict__ dv, T* __restrict__ dvf, T* __restrict__ dvl,
                   float* __restrict__ partial) {
    const Walk wk = make_walk(C);
    if (!wk.live) return;
    float pw0[8], pa0[8], pv0[8], pkk[8], pka[8];
    load8(w0 + wk.c, pw0); load8(a0 + wk.c, pa0); load8(k_k + wk.c, pkk); load8(k_a + wk.c, pka);
    if (use_vmix) load8(v0 + wk.c, pv0);
    float s_w0[8] = {0}, s_a0[8] = {0}, s_v0[8] = {0}, s_kk[8] = {0}, s_ka[8] = {0};
    const int slots = blockDim.x / (C / kOct);
    const int n_it = (rows - (int)(blockIdx.x * slots) + wk.row_step - 1) / wk.row_step;
    for (int it = 0, row = wk.row; it < n_it; ++it, row += wk.row_step) {
        const bool in = row < rows;
        const size_t off = (size_t)(in ? row : 0) * C + wk.c;
        const float live = in ? 1.f : 0.f;   // rows beyond the end contribute nothing to the parameter sums
        Raw<T> qk, qa, qgk, qgai, qgbi, qw, qgw, qv, qf, ql, qgv;
        qk.load(k + off); qa.load(al + off); qgk.load(gkp + off); qgai.load(gai + off); qgbi.load(gbi + off);
        qw.load(wl + off); qgw.load(gw + off); qgv.load(gvp + off);
        if (use_vmix) { qv.load(v + off); qf.load(vf + off); ql.load(vl + off); }
        {   // the key / a group
            float xk[8], xa[8], g_kp[8], g_ai[8], g_bi[8];
            qk.get(xk); qa.get(xa); qgk.get(g_kp); qgai.get(g_ai); qgbi.get(g_bi);
            float u[8], n2 = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                u[e] = xk[e] * pkk[e];
                n2 = fmaf(u[e], u[e], n2);
            }
            const float nrm = sqrtf(head_sum(n2));
            const bool floored = nrm < kNormFloor;
            const float inv = 1.f / fmaxf(nrm, kNormFloor);
            float a[8], kk[8], dkk[8], dot = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a[e] = sigmoidf(pa0[e] + xa[e]);
                kk[e] = u[e] * inv;
                dkk[e] = -g_ai[e] + a[e] * g_bi[e];
                dot = fmaf(kk[e], dkk[e], dot);
            }
            dot = head_sum(dot);
            if (floored) dot = 0.f;                  // below the floor kk = u / 1e-12 is linear in u
            float o_dk[8], o_dal[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float du = (dkk[e] - kk[e] * dot) * inv;
                const float da = g_bi[e] * kk[e] + g_kp[e] * xk[e] * pka[e];
                o_dk[e] = g_kp[e] * (1.f + (a[e] - 1.f) * pka[e]) + du * pkk[e];
                o_dal[e] = da * a[e] * (1.f - a[e]);
                s_kk[e] = fmaf(live * du, xk[e], s_kk[e]);
                s_ka[e] = fmaf(live * g_kp[e] * xk[e], a[e] - 1.f, s_ka[e]);
                s_a0[e] = fmaf(live, o_dal[e], s_a0[e]);
            }
            if (in) { store8(dk + off, o_dk); store8(dal + off, o_dal); }
        }
        {   // the decay
            float xw[8], g_w[8];
            qw.get(xw); qgw.get(g_w);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                xw[e] = g_w[e] * sigmoidf(-(pw0[e] + xw[e]));
                s_w0[e] = fmaf(live, xw[e], s_w0[e]);
            }
            if (in) store8(dwl + off, xw);
        }
        {   // the value
            float g_vp[8];
            qgv.get(g_vp);
            if (use_vmix) {
                float xv[8], xf[8], xl[8], o_dv[8], o_dvf[8], o_dvl[8];
                qv.get(xv); qf.get(xf); ql.get(xl);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float sg = sigmoidf(pv0[e] + xl[e]);
                    o_dv[e] = g_vp[e] * (1.f - sg);
                    o_dvf[e] = g_vp[e] * sg;
                    o_dvl[e] = g_vp[e] * (xf[e] - xv[e]) * sg * (1.f - sg);
                    s_v0[e] = fmaf(live, o_dvl[e], s_v0[e]);
                }
                if (in) { store8(dv + off, o_dv); store8(dvf + off, o_dvf); store8(dvl + off, o_dvl); }
            } else if (in) {
                store8(dv + off, g_vp);
            }
        }
    }
    float* dst = partial + ((size_t)(blockIdx.x * slots + threadIdx.x / (C / kOct)) * 5) * C + wk.c;
    store8(dst, s_w0); store8(dst + C, s_a0); store8(dst + 2 * (size_t)C, s_v0);
    store8(dst + 3 * (size_t)C, s_kk); store8(dst + 4 * (size_t)C, s_ka);
}

template <typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, MIX_MINB(MAXT))
mix_post_fwd_kernel(int rows, int C, float eps, const T* __restrict__ y, const T* __restrict__ r, const T* __restrict__ kp,
                    const T* __restrict__ vp, const T* __restrict__ g, const T* __restrict__ ln_w, const T* __restrict__ ln_b,
                    const T* __restrict__ r_k, T* __restrict__ x_out) {
    const Walk wk = make_walk(C);
    if (!wk.live) return;
    float plw[8], plb[8], prk[8];
    load8(ln_w + wk.c, plw); load8(ln_b + wk.c, plb); load8(r_k + wk.c, prk);
    const int slots = blockDim.x / (C / kOct);
    const int n_it = (rows - (int)(blockIdx.x * slots) + wk.row_step - 1) / wk.row_step;
    for (int it = 0, row = wk.row; it < n_it; ++it, row += wk.row_step) {
        const bool in = row < rows;
        const size_t off = (size_t)(in ? row : 0) * C + wk.c;
        float xy[8], xr[8], xk[8], xv[8], xg[8];
        load8(y + off, xy); load8(r + off, xr); load8(kp + off, xk); load8(vp + off, xv); load8(g + off, xg);
        float s1 = 0.f, cc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            s1 += xy[e];
            cc = fmaf(xr[e] * xk[e], prk[e], cc);
        }
        const float mean = head_sum(s1) * (1.f / kN);
        float s2 = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s2 = fmaf(xy[e] - mean, xy[e] - mean, s2);
        const float rstd = rsqrtf(head_sum(s2) * (1.f / kN) + eps);
        cc = head_sum(cc);
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = ((xy[e] - mean) * rstd * plw[e] + plb[e] + cc * xv[e]) * xg[e];
        if (in) store8(x_out + off, o);
    }
}

// partial: [gridDim.x * slots][3][C] fp32 in the order d ln_w, d ln_b, d r_k
template <typename T, int MAXT>
__global__ void __launch_bounds__(MAXT, MIX_MINB(MAXT))
mix_post_bwd_kernel(int rows, int C, float eps, const T* __restrict__ y, const T* __restrict__ r, const T* __restrict__ kp,
                    const T* __restrict__ vp, const T* __restrict__ g, const T* __restrict__ ln_w, const T* __restrict__ ln_b,
                    const T* __restrict__ r_k, const T* __restrict__ gx, T* __restrict__ dy, T* __restrict__ dr,
                    T* __restrict__ dkp, T* __restrict__ dvp, T* __restrict__ dg, float* __restrict__ partial) {
    const Walk wk = make_walk(C);
    if (!wk.live) return;
    float plw[8], plb[8], prk[8];
    load8(ln_w + wk.c, plw); load8(ln_b + wk.c, plb); load8(r_k + wk.c, prk);
    float s_lw[8] = {0}, s_lb[8] = {0}, s_rk[8] = {0};
    const int slots = blockDim.x / (C / kOct);
    const int n_it = (rows - (int)(blockIdx.x * slots) + wk.row_step - 1) / wk.row_step;
    for (int it = 0, row = wk.row; it < n_it; ++it, row += wk.row_step) {
        const bool in = row < rows;
        const size_t off = (size_t)(in ? row : 0) * C + wk.c;
        const float live = in ? 1.f : 0.f;
        float xy[8], xr[8], xk[8], xv[8], xg[8], gxo[8];
        load8(y + off, xy); load8(r + off, xr); load8(kp + off, xk); load8(vp + off, xv); load8(g + off, xg);
        load8(gx + off, gxo);
        float s1 = 0.f, cc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            s1 += xy[e];
            cc = fmaf(xr[e] * xk[e], prk[e], cc);
        }
        const float mean = head_sum(s1) * (1.f / kN);
        float s2 = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) s2 = fmaf(xy[e] - mean, xy[e] - mean, s2);
        const float rstd = rsqrtf(head_sum(s2) * (1.f / kN) + eps);
        cc = head_sum(cc);
        float xh[8], dt[8], dxh[8], o_dg[8], m1 = 0.f, m2 = 0.f, dc = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            xh[e] = (xy[e] - mean) * rstd;
            o_dg[e] = gxo[e] * (xh[e] * plw[e] + plb[e] + cc * xv[e]);
            dt[e] = gxo[e] * xg[e];
            dxh[e] = dt[e] * plw[e];
            m1 += dxh[e];
            m2 = fmaf(dxh[e], xh[e], m2);
            dc = fmaf(dt[e], xv[e], dc);
            s_lw[e] = fmaf(live * dt[e], xh[e], s_lw[e]);
            s_lb[e] = fmaf(live, dt[e], s_lb[e]);
        }
        m1 = head_sum(m1) * (1.f / kN);
        m2 = head_sum(m2) * (1.f / kN);
        dc = head_sum(dc);
        float o_dy[8], o_dr[8], o_dk[8], o_dv[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            o_dy[e] = (dxh[e] - m1 - xh[e] * m2) * rstd;
            o_dv[e] = dt[e] * cc;
            o_dr[e] = dc * xk[e] * prk[e];
            o_dk[e] = dc * xr[e] * prk[e];
            s_rk[e] = fmaf(live * dc * xr[e], xk[e], s_rk[e]);
        }
        if (in) {
            store8(dy + off, o_dy); store8(dr + off, o_dr); store8(dkp + off, o_dk); store8(dvp + off, o_dv);
            store8(dg + off, o_dg);
        }
    }
    float* dst = partial + ((size_t)(blockIdx.x * slots + threadIdx.x / (C / kOct)) * 3) * C + wk.c;
    store8(dst, s_lw); store8(dst + C, s_lb); store8(dst + 2 * (size_t)C, s_rk);
}

// the block size (threads per row x rows side by side) picks the instantiation, so that the register budget
// of the common shapes (<= 256 threads) is not the one a 1024-thread block forces
#define B200WKV_MIX_LAUNCH(KERNEL, ...)                                                   \
    do {                                                                                  \
        if (g.block <= 256) KERNEL<T, 256><<<g.grid, g.block, 0, st>>>(__VA_ARGS__);      \
        else if (g.block <= 512) KERNEL<T, 512><<<g.grid, g.block, 0, st>>>(__VA_ARGS__); \
        else KERNEL<T, 1024><<<g.grid, g.block, 0, st>>>(__VA_ARGS__);                    \
    } while (0)

struct Geometry {
    int block, slots, grid;
};
// Threads per row = C / 8; a block holds as many rows side by side as fit ~256 threads; the grid is what is
// resident at once (the walk is grid-strided), capped by the number of row groups.
Geometry geometry(int rows, int C) {
    Geometry g;
    const int per_row = C / kOct;
    g.slots = per_row >= 256 ? 1 : 256 / per_row;
    g.block = per_row * g.slots;
    const long long groups = ((long long)rows + g.slots - 1) / g.slots;
    const long long resident = (long long)sm_count_of_current_device() * (2048 / g.block > 0 ? 2048 / g.block : 1);
    g.grid = (int)(groups < resident ? groups : resident);
    return g;
}

}  // namespace

int wkv7_mix_partial_rows(int rows, int C) {
    const Geometry g = geometry(rows, C);
    return g.grid * g.slots;
}

template <typename T>
int mix_pre_fwd_t(cudaStream_t st, int rows, int C, int use_vmix, const void* k, const void* wl, const void* al, const void* v,
                  const void* vf, const void* vl, const void* w0, const void* a0, const void* v0, const void* k_k,
                  const void* k_a, void* w, void* kp, void* vp, void* ai, void* bi) {
    const Geometry g = geometry(rows, C);
    B200WKV_MIX_LAUNCH(mix_pre_fwd_kernel, rows, C, use_vmix, (const T*)k, (const T*)wl, (const T*)al, (const T*)v,
                                                      (const T*)vf, (const T*)vl, (const T*)w0, (const T*)a0, (const T*)v0,
                                                      (const T*)k_k, (const T*)k_a, (T*)w, (T*)kp, (T*)vp, (T*)ai, (T*)bi);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}
template <typename T>
int mix_pre_bwd_t(cudaStream_t st, int rows, int C, int use_vmix, const void* k, const void* wl, const void* al, const void* v,
                  const void* vf, const void* vl, const void* w0, const void* a0, const void* v0, const void* k_k,
                  const void* k_a, const void* gw, const void* gkp, const void* gvp, const void* gai, const void* gbi,
                  void* dk, void* dwl, void* dal, void* dv, void* dvf, void* dvl, float* partial) {
    const Geometry g = geometry(rows, C);
    B200WKV_MIX_LAUNCH(mix_pre_bwd_kernel, rows, C, use_vmix, (const T*)k, (const T*)wl, (const T*)al, (const T*)v, (const T*)vf, (const T*)vl, (const T*)w0,
        (const T*)a0, (const T*)v0, (const T*)k_k, (const T*)k_a, (const T*)gw, (const T*)gkp, (const T*)gvp, (const T*)gai,
        (const T*)gbi, (T*)dk, (T*)dwl, (T*)dal, (T*)dv, (T*)dvf, (T*)dvl, partial);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}
template <typename T>
int mix_post_fwd_t(cudaStream_t st, int rows, int C, float eps, const void* y, const void* r, const void* kp, const void* vp,
                   const void* g_, const void* ln_w, const void* ln_b, const void* r_k, void* x) {
    const Geometry g = geometry(rows, C);
    B200WKV_MIX_LAUNCH(mix_post_fwd_kernel, rows, C, eps, (const T*)y, (const T*)r, (const T*)kp, (const T*)vp,
                                                       (const T*)g_, (const T*)ln_w, (const T*)ln_b, (const T*)r_k, (T*)x);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}
template <typename T>
int mix_post_bwd_t(cudaStream_t st, int rows, int C, float eps, const void* y, const void* r, const void* kp, const void* vp,
                   const void* g_, const void* ln_w, const void* ln_b, const void* r_k, const void* gx, void* dy, void* dr,
                   void* dkp, void* dvp, void* dg, float* partial) {
    const Geometry g = geometry(rows, C);
    B200WKV_MIX_LAUNCH(mix_post_bwd_kernel, rows, C, eps, (const T*)y, (const T*)r, (const T*)kp, (const T*)vp,
                                                       (const T*)g_, (const T*)ln_w, (const T*)ln_b, (const T*)r_k,
                                                       (const T*)gx, (T*)dy, (T*)dr, (T*)dkp, (T*)dvp, (T*)dg, partial);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

int wkv7_mix_pre_fwd(cudaStream_t st, int dtype, int rows, int C, int use_vmix, const void* k, const void* wl, const void* al,
                     const void* v, const void* vf, const void* vl, const void* w0, const void* a0, const void* v0,
                     const void* k_k, const void* k_a, void* w, void* kp, void* vp, void* ai, void* bi) {
    return dtype == B200WKV_F32 ? mix_pre_fwd_t<float>(st, rows, C, use_vmix, k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, w, kp, vp, ai, bi)
                                : mix_pre_fwd_t<__nv_bfloat16>(st, rows, C, use_vmix, k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, w, kp, vp, ai, bi);
}
int wkv7_mix_pre_bwd(cudaStream_t st, int dtype, int rows, int C, int use_vmix, const void* k, const void* wl, const void* al,
                     const void* v, const void* vf, const void* vl, const void* w0, const void* a0, const void* v0,
                     const void* k_k, const void* k_a, const void* gw, const void* gkp, const void* gvp, const void* gai,
                     const void* gbi, void* dk, void* dwl, void* dal, void* dv, void* dvf, void* dvl, float* partial) {
    return dtype == B200WKV_F32
               ? mix_pre_bwd_t<float>(st, rows, C, use_vmix, k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, gw, gkp, gvp, gai, gbi, dk, dwl, dal, dv, dvf, dvl, partial)
               : mix_pre_bwd_t<__nv_bfloat16>(st, rows, C, use_vmix, k, wl, al, v, vf, vl, w0, a0, v0, k_k, k_a, gw, gkp, gvp, gai, gbi, dk, dwl, dal, dv, dvf, dvl, partial);
}
int wkv7_mix_post_fwd(cudaStream_t st, int dtype, int rows, int C, float eps, const void* y, const void* r, const void* kp,
                      const void* vp, const void* g, const void* ln_w, const void* ln_b, const void* r_k, void* x) {
    return dtype == B200WKV_F32 ? mix_post_fwd_t<float>(st, rows, C, eps, y, r, kp, vp, g, ln_w, ln_b, r_k, x)
                                : mix_post_fwd_t<__nv_bfloat16>(st, rows, C, eps, y, r, kp, vp, g, ln_w, ln_b, r_k, x);
}
int wkv7_mix_post_bwd(cudaStream_t st, int dtype, int rows, int C, float eps, const void* y, const void* r, const void* kp,
                      const void* vp, const void* g, const void* ln_w, const void* ln_b, const void* r_k, const void* gx, void* dy,
                      void* dr, void* dkp, void* dvp, void* dg, float* partial) {
    return dtype == B200WKV_F32
               ? mix_post_bwd_t<float>(st, rows, C, eps, y, r, kp, vp, g, ln_w, ln_b, r_k, gx, dy, dr, dkp, dvp, dg, partial)
               : mix_post_bwd_t<__nv_bfloat16>(st, rows, C, eps, y, r, kp, vp, g, ln_w, ln_b, r_k, gx, dy, dr, dkp, dvp, dg, partial);
}

}  // namespace b200wkv

// RWKV-4 WKV recurrence: one thread per (batch, channel), token-sequential, fp32 arithmetic.
//
// Per channel the state is (aa, bb, pp): numerator, denominator and the exponent both are scaled
// by.  With w' = -exp(w) (applied by the caller, as jaxrwkv does at src/jaxrwkv/rwkv4.py:312) and
// u = time_first:
//   q  = max(pp, u + k_t)      y_t = (e^{pp-q} aa + e^{u+k_t-q} v_t) / (e^{pp-q} bb + e^{u+k_t-q})
//   q' = max(pp + w', k_t)     aa <- e^{pp+w'-q'} aa + e^{k_t-q'} v_t,  bb likewise with 1,  pp <- q'
// A start flag resets the state to (0, 0, -1e30).  The kernel returns y without the receptance
// factor; the caller multiplies by r (rwkv4.py:406).  Semantics: BaseRWKV.inner_loop, rwkv4.py:143-172.
// The backward differentiates exactly these stabilised operations in reverse, replaying each block
// of 32 tokens from a saved state.
#include "common.cuh"

namespace b200wkv {

namespace {
constexpr int kCk4 = 32;

template <typename T>
__global__ void __launch_bounds__(128)
wkv4_fwd_kernel(int B, int Tlen, int C, const T* __restrict__ w, const T* __restrict__ u, const T* __restrict__ k,
                const T* __restrict__ v, const T* __restrict__ s0, const uint32_t* __restrict__ length,
                const uint8_t* __restrict__ new_starts, T* __restrict__ s_out, T* __restrict__ y,
                float* __restrict__ ckpt) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * C) return;
    const int bi = idx / C, c = idx % C;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kCk4 - 1) / kCk4;
    const float ww = to_f32(w[c]), uu = to_f32(u[c]);
    const size_t sb = (size_t)bi * 3 * C + c;
    float aa = to_f32(s0[sb]), bb = to_f32(s0[sb + C]), pp = to_f32(s0[sb + 2 * C]);
    if (L == 0) { s_out[sb] = from_f32<T>(aa); s_out[sb + C] = from_f32<T>(bb); s_out[sb + 2 * C] = from_f32<T>(pp); }
    const size_t base = (size_t)bi * Tlen * C + c;
    for (int t = 0; t < Tlen; ++t) {
        if (ckpt != nullptr && (t % kCk4) == 0) {
            float* cp = ckpt + (((size_t)bi * nC + t / kCk4) * 3) * C + c;
            cp[0] = aa; cp[C] = bb; cp[2 * C] = pp;
        }
        if (new_starts[(size_t)bi * Tlen + t]) { aa = 0.f; bb = 0.f; pp = -1e30f; }
        const float kt = to_f32(k[base + (size_t)t * C]), vt = to_f32(v[base + (size_t)t * C]);
        float x = uu + kt;
        float q = fmaxf(pp, x);
        float e1 = expf(pp - q), e2 = expf(x - q);
        y[base + (size_t)t * C] = from_f32<T>((e1 * aa + e2 * vt) / (e1 * bb + e2));
        x = pp + ww;
        q = fmaxf(x, kt);
        e1 = expf(x - q); e2 = expf(kt - q);
        aa = e1 * aa + e2 * vt; bb = e1 * bb + e2; pp = q;
        if (t == L - 1) { s_out[sb] = from_f32<T>(aa); s_out[sb + C] = from_f32<T>(bb); s_out[sb + 2 * C] = from_f32<T>(pp); }
    }
}

template <typename T>
__global__ void __launch_bounds__(128)
wkv4_bwd_kernel(int B, int Tlen, int C, const T* __restrict__ w, const T* __restrict__ u, const T* __restrict__ k,
                const T* __restrict__ v, const T* __restrict__ gy, const uint32_t* __restrict__ length,
                const uint8_t* __restrict__ new_starts, const T* __restrict__ gs_new, const float* __restrict__ ckpt,
                float* __restrict__ gw, float* __restrict__ gu, T* __restrict__ gk, T* __restrict__ gv,
                T* __restrict__ gs) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * C) return;
    const int bi = idx / C, c = idx % C;
    const int L = min((int)length[bi], Tlen);
    const int nC = (Tlen + kCk4 - 1) / kCk4;
    const float ww = to_f32(w[c]), uu = to_f32(u[c]);
    const size_t sb = (size_t)bi * 3 * C + c;
    const size_t base = (size_t)bi * Tlen * C + c;
    float gaa = 0.f, gbb = 0.f, gpp = 0.f;   // cotangent of the state after the token being processed
    float gw_acc = 0.f, gu_acc = 0.f;
    for (int blk = nC - 1; blk >= 0; --blk) {
        const int t0 = blk * kCk4;
        const float* cp = ckpt + (((size_t)bi * nC + blk) * 3) * C + c;
        float aa = cp[0], bb = cp[C], pp = cp[2 * C];
        float ha[kCk4], hb[kCk4], hp[kCk4], hk[kCk4], hv[kCk4];   // state entering each token (after a reset), k, v
#pragma unroll
        for (int tt = 0; tt < kCk4; ++tt) {
            const int t = t0 + tt;
            if (t < Tlen) {
                if (new_starts[(size_t)bi * Tlen + t]) { aa = 0.f; bb = 0.f; pp = -1e30f; }
                const float kt = to_f32(k[base + (size_t)t * C]), vt = to_f32(v[base + (size_t)t * C]);
                ha[tt] = aa; hb[tt] = bb; hp[tt] = pp; hk[tt] = kt; hv[tt] = vt;
                const float x = pp + ww, q = fmaxf(x, kt);
                const float e1 = expf(x - q), e2 = expf(kt - q);
                aa = e1 * aa + e2 * vt; bb = e1 * bb + e2; pp = q;
            }
        }
#pragma unroll
        for (int tt = kCk4 - 1; tt >= 0; --tt) {
            const int t = t0 + tt;
            if (t < Tlen) {
                if (t == L - 1 && gs_new != nullptr) {
                    gaa += to_f32(gs_new[sb]); gbb += to_f32(gs_new[sb + C]); gpp += to_f32(gs_new[sb + 2 * C]);
                }
                const float a0 = ha[tt], b0 = hb[tt], p0 = hp[tt], kt = hk[tt], vt = hv[tt];
                // ---- state update, reversed
                float x = p0 + ww, q = fmaxf(x, kt);
                float e1 = expf(x - q), e2 = expf(kt - q);
                float ge1 = a0 * gaa + b0 * gbb, ge2 = vt * gaa + gbb;
                float gq = gpp - e1 * ge1 - e2 * ge2;
                const bool first = x >= kt;
                float gx = e1 * ge1 + (first ? gq : 0.f);
                float gkt = e2 * ge2 + (first ? 0.f : gq);
                float gvt = e2 * gaa;
                float na = e1 * gaa, nb = e1 * gbb, np = gx;
                gw_acc += gx;
                // ---- output, reversed (the max shift cancels in y, so no term flows through q)
                const float g = (gy != nullptr) ? to_f32(gy[base + (size_t)t * C]) : 0.f;
                x = uu + kt; q = fmaxf(p0, x);
                e1 = expf(p0 - q); e2 = expf(x - q);
                const float num = e1 * a0 + e2 * vt, den = e1 * b0 + e2;
                const float gnum = g / den, gden = -g * num / (den * den);
                ge1 = a0 * gnum + b0 * gden; ge2 = vt * gnum + gden;
                na += e1 * gnum; nb += e1 * gden; gvt += e2 * gnum;
                np += e1 * ge1;
                const float gxx = e2 * ge2;
                gu_acc += gxx; gkt += gxx;
                gk[base + (size_t)t * C] = from_f32<T>(gkt);
                gv[base + (size_t)t * C] = from_f32<T>(gvt);
                gaa = na; gbb = nb; gpp = np;
                if (new_starts[(size_t)bi * Tlen + t]) { gaa = 0.f; gbb = 0.f; gpp = 0.f; }
            }
        }
    }
    if (L == 0 && gs_new != nullptr) {
        gaa += to_f32(gs_new[sb]); gbb += to_f32(gs_new[sb + C]); gpp += to_f32(gs_new[sb + 2 * C]);
    }
    gs[sb] = from_f32<T>(gaa); gs[sb + C] = from_f32<T>(gbb); gs[sb + 2 * C] = from_f32<T>(gpp);
    gw[(size_t)bi * C + c] = gw_acc;
    gu[(size_t)bi * C + c] = gu_acc;
}
}  // namespace

size_t wkv4_residual_bytes(int B, int T, int C) { return (size_t)B * ((T + kCk4 - 1) / kCk4) * 3 * C * sizeof(float); }

int wkv4_fwd(cudaStream_t st, int dtype, int B, int T, int C, const void* w, const void* u, const void* k, const void* v,
             const void* s0, const uint32_t* length, const uint8_t* ns, void* s_out, void* y, void* residual) {
    const int grid = (B * C + 127) / 128;
    if (dtype == B200WKV_F32)
        wkv4_fwd_kernel<float><<<grid, 128, 0, st>>>(B, T, C, (const float*)w, (const float*)u, (const float*)k, (const float*)v,
                                                     (const float*)s0, length, ns, (float*)s_out, (float*)y, (float*)residual);
    else
        wkv4_fwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(B, T, C, (const __nv_bfloat16*)w, (const __nv_bfloat16*)u,
                                                             (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                             (const __nv_bfloat16*)s0, length, ns, (__nv_bfloat16*)s_out,
                                                             (__nv_bfloat16*)y, (float*)residual);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

int wkv4_bwd(cudaStream_t st, int dtype, int B, int T, int C, const void* w, const void* u, const void* k, const void* v,
             const void* gy, const uint32_t* length, const uint8_t* ns, const void* gs_new, const void* residual,
             void* gw, void* gu, void* gk, void* gv, void* gs) {
    const int grid = (B * C + 127) / 128;
    if (dtype == B200WKV_F32)
        wkv4_bwd_kernel<float><<<grid, 128, 0, st>>>(B, T, C, (const float*)w, (const float*)u, (const float*)k, (const float*)v,
                                                     (const float*)gy, length, ns, (const float*)gs_new, (const float*)residual,
                                                     (float*)gw, (float*)gu, (float*)gk, (float*)gv, (float*)gs);
    else
        wkv4_bwd_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(B, T, C, (const __nv_bfloat16*)w, (const __nv_bfloat16*)u,
                                                             (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                             (const __nv_bfloat16*)gy, length, ns, (const __nv_bfloat16*)gs_new,
                                                             (const float*)residual, (float*)gw, (float*)gu,
                                                             (__nv_bfloat16*)gk, (__nv_bfloat16*)gv, (__nv_bfloat16*)gs);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace b200wkv

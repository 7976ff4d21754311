// Token shift with start flags and the carried last row: the per-token state that the callers of the
// WKV operator maintain next to it (jaxrwkv src/jaxrwkv/rwkv7.py:226-235 and :254 for time mixing,
// :192-197 for channel mixing).  For every mix m:
//   shifted[t] = new_starts[t] ? 0 : (t == 0 ? prev : x[t-1])
//   out_m[t]   = x[t] + (shifted[t] - x[t]) * mix_m
//   state_out  = x[(length - 1) mod T]            (the reference indexes x[length-1]; length 0 wraps)
// One pass over x, M outputs: purely HBM-bound, so every thread moves V channels per access with
// V = 16 bytes / element size when the channel count allows it (else V = 4).
#include "common.cuh"

namespace b200wkv {
namespace {

template <int V> struct Vec { float f[V]; };

template <int V, typename T> __device__ __forceinline__ Vec<V> loadv(const T* p);
template <> __device__ __forceinline__ Vec<4> loadv<4, float>(const float* p) {
    const float4 q = load4(p);
    return Vec<4>{{q.x, q.y, q.z, q.w}};
}
template <> __device__ __forceinline__ Vec<4> loadv<4, __nv_bfloat16>(const __nv_bfloat16* p) {
    const float4 q = load4(p);
    return Vec<4>{{q.x, q.y, q.z, q.w}};
}
template <> __device__ __forceinline__ Vec<8> loadv<8, __nv_bfloat16>(const __nv_bfloat16* p) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
    Vec<8> r;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        r.f[2 * i] = t.x;
        r.f[2 * i + 1] = t.y;
    }
    return r;
}
__device__ __forceinline__ void storev(float* p, const Vec<4>& v) { store4(p, make_float4(v.f[0], v.f[1], v.f[2], v.f[3])); }
__device__ __forceinline__ void storev(__nv_bfloat16* p, const Vec<4>& v) {
    store4(p, make_float4(v.f[0], v.f[1], v.f[2], v.f[3]));
}
__device__ __forceinline__ void storev(__nv_bfloat16* p, const Vec<8>& v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v.f[2 * i], v.f[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}
// V channels as they lie in memory (16 or 8 bytes): what a thread keeps of a load until it uses it
template <int V, typename T> struct RawVec;
template <> struct RawVec<4, float> {
    float4 q;
    __device__ __forceinline__ void load(const float* p) { q = *reinterpret_cast<const float4*>(p); }
    __device__ __forceinline__ Vec<4> get() const { return Vec<4>{{q.x, q.y, q.z, q.w}}; }
};
template <> struct RawVec<4, __nv_bfloat16> {
    uint2 q;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { q = *reinterpret_cast<const uint2*>(p); }
    __device__ __forceinline__ Vec<4> get() const {
        return Vec<4>{{__uint_as_float(q.x << 16), __uint_as_float(q.x & 0xffff0000u), __uint_as_float(q.y << 16),
                       __uint_as_float(q.y & 0xffff0000u)}};
    }
};
template <> struct RawVec<8, __nv_bfloat16> {
    uint4 q;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { q = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ Vec<8> get() const {
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        Vec<8> r;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            r.f[2 * i] = __uint_as_float(w[i] << 16);
            r.f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
        return r;
    }
};

template <int V> __device__ __forceinline__ Vec<V> zerov() {
    Vec<V> r;
#pragma unroll
    for (int i = 0; i < V; ++i) r.f[i] = 0.f;
    return r;
}

__device__ __forceinline__ int last_row(uint32_t length, int Tlen) {
    const int L = (int)min(length, (uint32_t)0x7fffffff);
    return ((L - 1) % Tlen + Tlen) % Tlen;
}

// grid (B*T, ceil(D / V / 128)); one token row per blockIdx.x
template <typename T, int V>
__global__ void token_shift_fwd_kernel(int B, int Tlen, int D, int M, const T* __restrict__ x, const T* __restrict__ prev,
                                       const T* __restrict__ mix, const uint32_t* __restrict__ length,
                                       const uint8_t* __restrict__ new_starts, T* __restrict__ out,
                                       T* __restrict__ state_out) {
    const int d = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int bt = blockIdx.x;
    if (d >= D) return;
    const int bi = bt / Tlen, t = bt % Tlen;
    const size_t row = (size_t)bt * D + d;
    const Vec<V> xc = loadv<V>(x + row);
    Vec<V> df = zerov<V>();
    if (!new_starts[bt]) df = (t == 0) ? loadv<V>(prev + (size_t)bi * D + d) : loadv<V>(x + row - D);
#pragma unroll
    for (int i = 0; i < V; ++i) df.f[i] -= xc.f[i];
    for (int m = 0; m < M; ++m) {
        const Vec<V> c = loadv<V>(mix + (size_t)m * D + d);
        Vec<V> o;
#pragma unroll
        for (int i = 0; i < V; ++i) o.f[i] = fmaf(df.f[i], c.f[i], xc.f[i]);
        storev(out + ((size_t)m * B * Tlen + bt) * D + d, o);
    }
    if (t == last_row(length[bi], Tlen)) storev(state_out + (size_t)bi * D + d, xc);
}

// Backward.  Each thread owns V channels of one tile of B200WKV_SHIFT_TILE tokens of one batch row and
// walks it from the last token to the first (the loads do not depend on the walk, so they pipeline).
// The mix gradients leave as one fp32 partial sum per (batch row, tile): deterministic, no atomics.
//   gx[t] = sum_m g_m[t] (1 - c_m) + [t+1 < T and not start[t+1]] sum_m g_m[t+1] c_m + [t == last] gstate
// grid (ceil(D / V / 64), tiles, B)
template <typename T, int V, int MM>
__global__ void __launch_bounds__(64)
token_shift_bwd_kernel(int B, int Tlen, int D, const T* __restrict__ x, const T* __restrict__ prev,
                       const T* __restrict__ mix, const uint32_t* __restrict__ length,
                       const uint8_t* __restrict__ new_starts, const T* __restrict__ gout,
                       const T* __restrict__ gstate, T* __restrict__ gx, T* __restrict__ gprev,
                       float* __restrict__ gmix) {
    const int d = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    const int tile = blockIdx.y, ntile = gridDim.y;
    const int bi = blockIdx.z;
    if (d >= D) return;
    const int t0 = tile * B200WKV_SHIFT_TILE;
    const int t1 = min(Tlen, t0 + B200WKV_SHIFT_TILE);
    const int last = last_row(length[bi], Tlen);
    RawVec<V, T> craw[MM];   // the mix coefficients stay packed; unpacking them at each use is cheaper than the registers
    Vec<V> acc[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) {
        craw[m].load(mix + (size_t)m * D + d);
        acc[m] = zerov<V>();
    }
    const size_t base = (size_t)bi * Tlen * D + d;
    const size_t mstride = (size_t)B * Tlen * D;
    const uint8_t* ns = new_starts + (size_t)bi * Tlen;
    Vec<V> carry = zerov<V>();   // what token t+1 hands back to token t
    if (t1 < Tlen && !ns[t1]) {
#pragma unroll
        for (int m = 0; m < MM; ++m) {
            const Vec<V> g = loadv<V>(gout + m * mstride + base + (size_t)t1 * D);
            const Vec<V> cm = craw[m].get();
#pragma unroll
            for (int i = 0; i < V; ++i) carry.f[i] = fmaf(g.f[i], cm.f[i], carry.f[i]);
        }
    }
    Vec<V> xc = loadv<V>(x + base + (size_t)(t1 - 1) * D);
    // Tokens are taken four at a time: the 4 x (MM + 1) loads of a group are all issued, in packed form, before
    // the first token of the group is worked on, so a thread has ~450 bytes in flight at 255 registers.
    constexpr int G = 4;
    for (int tg = t1 - 1; tg >= t0; tg -= G) {
        RawVec<V, T> rg[G][MM], rx[G];
#pragma unroll
        for (int j = 0; j < G; ++j) {
            const int t = tg - j;
            if (t >= t0) {
#pragma unroll
                for (int m = 0; m < MM; ++m) rg[j][m].load(gout + m * mstride + base + (size_t)t * D);
                // the row before: needed as this token's shift and as the next token's x
                rx[j].load(t > 0 ? x + base + (size_t)(t - 1) * D : prev + (size_t)bi * D + d);
            }
        }
#pragma unroll
        for (int j = 0; j < G; ++j) {
            const int t = tg - j;
            if (t < t0) break;
            const bool st = ns[t] != 0;
            const Vec<V> xp = rx[j].get();
            Vec<V> keep = zerov<V>(), pass = zerov<V>(), df;
#pragma unroll
            for (int i = 0; i < V; ++i) df.f[i] = (st ? 0.f : xp.f[i]) - xc.f[i];
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                const Vec<V> g = rg[j][m].get();
                const Vec<V> cm = craw[m].get();
#pragma unroll
                for (int i = 0; i < V; ++i) {
                    keep.f[i] = fmaf(g.f[i], 1.f - cm.f[i], keep.f[i]);
                    pass.f[i] = fmaf(g.f[i], cm.f[i], pass.f[i]);
                    acc[m].f[i] = fmaf(g.f[i], df.f[i], acc[m].f[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < V; ++i) keep.f[i] += carry.f[i];
            if (t == last && gstate != nullptr) {
                const Vec<V> gs = loadv<V>(gstate + (size_t)bi * D + d);
#pragma unroll
                for (int i = 0; i < V; ++i) keep.f[i] += gs.f[i];
            }
            storev(gx + base + (size_t)t * D, keep);
#pragma unroll
            for (int i = 0; i < V; ++i) carry.f[i] = st ? 0.f : pass.f[i];
            xc = xp;
        }
    }
    if (tile == 0) storev(gprev + (size_t)bi * D + d, carry);
#pragma unroll
    for (int m = 0; m < MM; ++m) {
        float* dst = gmix + (((size_t)bi * ntile + tile) * MM + m) * D + d;
#pragma unroll
        for (int i = 0; i < V; i += 4) store4(dst + i, make_float4(acc[m].f[i], acc[m].f[i + 1], acc[m].f[i + 2], acc[m].f[i + 3]));
    }
}

template <typename T, int V>
void launch_fwd(cudaStream_t st, int B, int Tlen, int D, int M, const void* x, const void* prev, const void* mix,
                const uint32_t* length, const uint8_t* ns, void* out, void* state_out) {
    dim3 grid(B * Tlen, (D / V + 127) / 128);
    token_shift_fwd_kernel<T, V><<<grid, 128, 0, st>>>(B, Tlen, D, M, (const T*)x, (const T*)prev, (const T*)mix, length, ns,
                                                       (T*)out, (T*)state_out);
}

template <typename T, int V, int MM>
void launch_bwd_m(cudaStream_t st, int B, int Tlen, int D, const void* x, const void* prev, const void* mix,
                  const uint32_t* length, const uint8_t* ns, const void* gout, const void* gstate, void* gx, void* gprev,
                  void* gmix) {
    dim3 grid((D / V + 63) / 64, (Tlen + B200WKV_SHIFT_TILE - 1) / B200WKV_SHIFT_TILE, B);
    token_shift_bwd_kernel<T, V, MM><<<grid, 64, 0, st>>>(B, Tlen, D, (const T*)x, (const T*)prev, (const T*)mix, length, ns,
                                                          (const T*)gout, (const T*)gstate, (T*)gx, (T*)gprev, (float*)gmix);
}

template <typename T, int V>
void launch_bwd(cudaStream_t st, int B, int Tlen, int D, int M, const void* x, const void* prev, const void* mix,
                const uint32_t* length, const uint8_t* ns, const void* gout, const void* gstate, void* gx, void* gprev,
                void* gmix) {
#define B200WKV_SHIFT_CASE(MM) \
    case MM: launch_bwd_m<T, V, MM>(st, B, Tlen, D, x, prev, mix, length, ns, gout, gstate, gx, gprev, gmix); break;
    switch (M) {
        B200WKV_SHIFT_CASE(1) B200WKV_SHIFT_CASE(2) B200WKV_SHIFT_CASE(3) B200WKV_SHIFT_CASE(4)
        B200WKV_SHIFT_CASE(5) B200WKV_SHIFT_CASE(6) B200WKV_SHIFT_CASE(7) B200WKV_SHIFT_CASE(8)
    }
#undef B200WKV_SHIFT_CASE
}
}  // namespace

int token_shift_fwd(cudaStream_t st, int dtype, int B, int T, int D, int M, const void* x, const void* prev,
                    const void* mix, const uint32_t* length, const uint8_t* ns, void* out, void* state_out) {
    if (dtype == B200WKV_F32) launch_fwd<float, 4>(st, B, T, D, M, x, prev, mix, length, ns, out, state_out);
    else if (D % 8 == 0) launch_fwd<__nv_bfloat16, 8>(st, B, T, D, M, x, prev, mix, length, ns, out, state_out);
    else launch_fwd<__nv_bfloat16, 4>(st, B, T, D, M, x, prev, mix, length, ns, out, state_out);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

int token_shift_bwd(cudaStream_t st, int dtype, int B, int T, int D, int M, const void* x, const void* prev,
                    const void* mix, const uint32_t* length, const uint8_t* ns, const void* gout, const void* gstate,
                    void* gx, void* gprev, void* gmix) {
    if (dtype == B200WKV_F32) launch_bwd<float, 4>(st, B, T, D, M, x, prev, mix, length, ns, gout, gstate, gx, gprev, gmix);
    else if (D % 8 == 0) launch_bwd<__nv_bfloat16, 8>(st, B, T, D, M, x, prev, mix, length, ns, gout, gstate, gx, gprev, gmix);
    else launch_bwd<__nv_bfloat16, 4>(st, B, T, D, M, x, prev, mix, length, ns, gout, gstate, gx, gprev, gmix);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace b200wkv

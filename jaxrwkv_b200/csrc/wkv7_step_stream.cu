// RWKV-7 single-token step (recurrent decoding, T == 1) as a pipelined HBM stream.
//
// The whole cost of a decoding step is reading and writing every 64x64 state once.  Each CTA walks a
// strided list of (batch, head) pairs; the 8 KB (bf16) or 16 KB (fp32) state of the pairs ahead is
// brought into a ring of shared-memory stages by bulk asynchronous copies (one elected thread, an
// mbarrier per stage counts the bytes), so several states per CTA are in flight while the current
// one is updated in registers (eight columns of two rows per thread, see Own<T>).
// Same arithmetic as the plain step kernel; jaxrwkv has no kernel here (it falls back to the
// unrolled Python loop, src/jaxrwkv/rwkv7.py:469-470), the recurrence is rwkv7.py:199-220.
#include "common.cuh"
#include "device_once.cuh"
#include "tc05.cuh"

namespace b200wkv {

int* wkv7_chunk_status_word();

namespace {

constexpr int kStages = 4;
constexpr int kStateElems = kN * kN;
constexpr int kVecPitch = kN + 4;   // channel c of a vector sits at c + 4 * (c / 32): see vidx()

// A thread owns eight columns of two rows.  Lane = 8 * rsel + p: piece p of rows 8 * warp + rsel and
// + 4.  bf16: columns 8p..8p+7 (one 16-byte piece per row); fp32: columns 4p..4p+3 and 32+4p..32+4p+3
// (two 16-byte pieces).  Either way the eight lanes of a shared-memory access phase cover 128
// contiguous bytes of one row, and with the padded vector layout their float4 vector reads fall on
// distinct banks.
__device__ __forceinline__ int vidx(int c) { return c + ((c >> 5) << 2); }

template <typename T> struct Own;
template <> struct Own<__nv_bfloat16> {
    static __device__ __forceinline__ int col0(int p) { return 8 * p; }       // first four columns
    static __device__ __forceinline__ int col1(int p) { return 8 * p + 4; }   // last four columns
    static __device__ __forceinline__ void load(const __nv_bfloat16* row, int p, float* f) {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + 8 * p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 t = __bfloat1622float2(h[e]);
            f[2 * e] = t.x;
            f[2 * e + 1] = t.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* row, int p, const float* f) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        *reinterpret_cast<uint4*>(row + 8 * p) = raw;
    }
};
template <> struct Own<float> {
    static __device__ __forceinline__ int col0(int p) { return 4 * p; }
    static __device__ __forceinline__ int col1(int p) { return 32 + 4 * p; }
    static __device__ __forceinline__ void load(const float* row, int p, float* f) {
        *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(row + 4 * p);
        *reinterpret_cast<float4*>(f + 4) = *reinterpret_cast<const float4*>(row + 32 + 4 * p);
    }
    static __device__ __forceinline__ void store(float* row, int p, const float* f) {
        *reinterpret_cast<float4*>(row + 4 * p) = *reinterpret_cast<const float4*>(f);
        *reinterpret_cast<float4*>(row + 32 + 4 * p) = *reinterpret_cast<const float4*>(f + 4);
    }
};

template <typename T>
struct StepSmem {
    alignas(128) T stage[kStages][kStateElems];
    alignas(16) float vec[2][6][kVecPitch];   // decay, r, k, v, a, b of the current and the next pair
    uint64_t full[kStages];
};

__device__ __forceinline__ void vec8(const float* vec, int c0, int c1, float* f) {
    *reinterpret_cast<float4*>(f) = *reinterpret_cast<const float4*>(vec + vidx(c0));
    *reinterpret_cast<float4*>(f + 4) = *reinterpret_cast<const float4*>(vec + vidx(c1));
}
__device__ __forceinline__ float sum8(float x) {   // over the eight lanes that share a row
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    x += __shfl_xor_sync(0xffffffffu, x, 4);
    return x;
}

template <typename T>
__global__ void __launch_bounds__(256)
wkv7_step_stream_kernel(int BH, int H, const T* __restrict__ w, const T* __restrict__ r, const T* __restrict__ k,
                        const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                        const T* __restrict__ s0, const uint32_t* __restrict__ length,
                        const uint8_t* __restrict__ new_starts, T* __restrict__ y, T* __restrict__ s_out,
                        int* __restrict__ status, long long s_batch_stride) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    StepSmem<T>& sm = *reinterpret_cast<StepSmem<T>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = lane & 7, ra = warp * 8 + (lane >> 3), rb = ra + 4;
    const int c0 = Own<T>::col0(p), c1 = Own<T>::col1(p);
    const int first = blockIdx.x, stride = gridDim.x;
    const int n_my = (BH - first + stride - 1) / stride;   // pairs first, first + stride, ...
    constexpr uint32_t kTileBytes = kStateElems * sizeof(T);
    // element offset of the state of pair q: batch rows may be s_batch_stride elements apart (a state
    // that lives inside a larger per-sequence container), heads of one row are contiguous
    auto state_off = [&](int q) { return (size_t)(q / H) * (size_t)s_batch_stride + (size_t)(q % H) * kStateElems; };
    // threads 0..95 fetch the six vectors: stream vm, channels vc..vc+3
    const int vm = tid >> 4, vc = (tid & 15) * 4;
    const T* vsrc = vm == 0 ? w : vm == 1 ? r : vm == 2 ? k : vm == 3 ? v : vm == 4 ? a : b;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) tc::mbar_init(&sm.full[s], 1);
        tc::mbar_init_fence();
    }
    __syncthreads();
    if (tid == 0) {
        for (int s = 0; s < kStages && s < n_my; ++s) {
            tc::mbar_expect_tx(&sm.full[s], kTileBytes);
            tc::bulk_load(sm.stage[s], s0 + state_off(first + s * stride), kTileBytes, &sm.full[s]);
        }
    }
    if (tid < 96) {
        float4 x = load4(vsrc + (size_t)first * kN + vc);
        if (vm == 0) x = make_float4(expf(-expf(x.x)), expf(-expf(x.y)), expf(-expf(x.z)), expf(-expf(x.w)));
        *reinterpret_cast<float4*>(&sm.vec[0][vm][vidx(vc)]) = x;
    }
    bool failed = false;
    for (int it = 0; it < n_my; ++it) {
        const int bh = first + it * stride, bi = bh / H;
        const int s = it % kStages;
        const uint32_t parity = (uint32_t)(it / kStages) & 1u;
        // vectors of the next pair travel while this one is computed
        float4 nx = make_float4(0.f, 0.f, 0.f, 0.f);
        const bool more = it + 1 < n_my;
        if (more && tid < 96) nx = load4(vsrc + (size_t)(bh + stride) * kN + vc);
        const bool keep_input = (length[bi] == 0);   // length == 0 returns the input state untouched
        const bool reset = new_starts[bi] != 0;
        if (!tc::mbar_wait(&sm.full[s], parity)) failed = true;
        float Sa[8], Sb[8];
        Own<T>::load(&sm.stage[s][ra * kN], p, Sa);
        Own<T>::load(&sm.stage[s][rb * kN], p, Sb);
        __syncthreads();   // every thread holds its part of stage s; vec[it & 1] is complete
        if (tid == 0 && it + kStages < n_my) {
            tc::mbar_expect_tx(&sm.full[s], kTileBytes);
            tc::bulk_load(sm.stage[s], s0 + state_off(bh + kStages * stride), kTileBytes, &sm.full[s]);
        }
        if (more && tid < 96) {
            if (vm == 0) nx = make_float4(expf(-expf(nx.x)), expf(-expf(nx.y)), expf(-expf(nx.z)), expf(-expf(nx.w)));
            *reinterpret_cast<float4*>(&sm.vec[(it + 1) & 1][vm][vidx(vc)]) = nx;
        }
        const float (*vec)[kVecPitch] = sm.vec[it & 1];
        T* out_a = s_out + state_off(bh) + (size_t)ra * kN;
        T* out_b = s_out + state_off(bh) + (size_t)rb * kN;
        if (keep_input) {
            Own<T>::store(out_a, p, Sa);
            Own<T>::store(out_b, p, Sb);
        }
        if (reset) {
#pragma unroll
            for (int e = 0; e < 8; ++e) Sa[e] = Sb[e] = 0.f;
        }
        float x[8];
        vec8(vec[4], c0, c1, x);   // a
        float sa_a = 0.f, sa_b = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            sa_a = fmaf(Sa[e], x[e], sa_a);
            sa_b = fmaf(Sb[e], x[e], sa_b);
        }
        sa_a = sum8(sa_a);
        sa_b = sum8(sa_b);
        const float va = vec[3][vidx(ra)], vb = vec[3][vidx(rb)];
        float dec[8], kk[8];
        vec8(vec[0], c0, c1, dec);
        vec8(vec[2], c0, c1, kk);
        vec8(vec[5], c0, c1, x);   // b
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            Sa[e] = fmaf(Sa[e], dec[e], fmaf(va, kk[e], sa_a * x[e]));
            Sb[e] = fmaf(Sb[e], dec[e], fmaf(vb, kk[e], sa_b * x[e]));
        }
        vec8(vec[1], c0, c1, x);   // r
        float ya = 0.f, yb = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            ya = fmaf(Sa[e], x[e], ya);
            yb = fmaf(Sb[e], x[e], yb);
        }
        ya = sum8(ya);
        yb = sum8(yb);
        if (p == 0) {
            y[(size_t)bh * kN + ra] = from_f32<T>(ya);
            y[(size_t)bh * kN + rb] = from_f32<T>(yb);
        }
        if (!keep_input) {
            Own<T>::store(out_a, p, Sa);
            Own<T>::store(out_b, p, Sb);
        }
    }
    if (failed && status != nullptr) atomicExch(status, 3);
}

template <typename T>
int launch(cudaStream_t st, int B, int H, const void* w, const void* r, const void* k, const void* v, const void* a,
           const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y, void* s_out,
           long long s_batch_stride) {
    // facts that depend only on (kernel instance, device) are looked up once per device: the shared-memory
    // opt-in, how many CTAs of this kernel fit an SM, and the address of the device status word
    auto kern = wkv7_step_stream_kernel<T>;
    const int smem = (int)sizeof(StepSmem<T>);
    static DeviceOnce setup;
    static int per_sm_of[kMaxDevices];
    static int* status_of[kMaxDevices];
    const int dev = current_device();
    if (dev < 0) return B200WKV_ELAUNCH;
    if (!setup.ok([&]() {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess) return e;
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, 256, smem) != cudaSuccess || n < 1) n = 1;
            per_sm_of[dev] = n;
            status_of[dev] = wkv7_chunk_status_word();
            return cudaSuccess;
        }))
        return B200WKV_ELAUNCH;
    const int sm_count = sm_count_of_current_device(), per_sm = per_sm_of[dev];
    const int BH = B * H;
    const int grid = BH < sm_count * per_sm ? BH : sm_count * per_sm;   // one wave: every CTA resident
    kern<<<grid, 256, smem, st>>>(BH, H, (const T*)w, (const T*)r, (const T*)k, (const T*)v, (const T*)a, (const T*)b,
                                  (const T*)s0, length, ns, (T*)y, (T*)s_out, status_of[dev], s_batch_stride);
    return cudaGetLastError() == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace

// Requires s0 and s_out 16-byte aligned (the bulk copies and the vector stores) and a batch stride
// that keeps every row aligned; the caller checks.  s_out may be s0 (update in place): a pair's state
// is read into the ring before its own write-back and no other pair touches it.
int wkv7_step_stream(cudaStream_t st, int dtype, int B, int H, const void* w, const void* r, const void* k, const void* v,
                     const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                     void* s_out, long long s_batch_stride) {
    if (dtype == B200WKV_F32) return launch<float>(st, B, H, w, r, k, v, a, b, s0, length, ns, y, s_out, s_batch_stride);
    return launch<__nv_bfloat16>(st, B, H, w, r, k, v, a, b, s0, length, ns, y, s_out, s_batch_stride);
}

}  // namespace b200wkv

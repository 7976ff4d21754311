// RWKV-7 single-token step (recurrent decoding, T == 1) as a pipelined HBM stream.
//
// The whole cost of a decoding step is reading and writing every 64x64 state once.  Each CTA (64
// computing threads and one copy thread) walks a strided list of (batch, head) pairs; the 8 KB (bf16) or
// 16 KB (fp32) state of the pairs ahead is brought into a ring of shared-memory stages by bulk
// asynchronous copies (an mbarrier per stage counts the bytes).  The current state is updated in
// registers, four rows of sixteen columns per thread (64 elements: the fixed cost of an iteration and
// the reads of the six vectors are spread over them).  A stage is handed back to the copy thread as soon
// as its state is in registers, so the whole ring is loads in flight; results leave the registers as
// 32-byte stores (one full sector per lane).  The six vectors of a pair travel into its stage with the
// state and the start / length flags are fetched 64 pairs at a time: no iteration waits for a global
// load of its own, which under a saturated memory system would cost microseconds each.
// jaxrwkv has no kernel here (it falls back to the unrolled Python loop, src/jaxrwkv/rwkv7.py:469-470);
// the recurrence is rwkv7.py:199-220.
#include "common.cuh"
#include "device_once.cuh"
#include "tc05.cuh"

namespace b200wkv {

int* wkv7_chunk_status_word();

namespace {

constexpr int kStateElems = kN * kN;
constexpr int kComputeThreads = 64;
constexpr int kThreads = 96;   // two computing warps and the warp of the copy thread

// Thread layout.  Lane = 4 * rsel + p: piece p (columns 16p..16p+15) of rows 32 * warp + 8 * g + rsel,
// g = 0..3.  A piece is 2 (bf16) or 4 (fp32) 16-byte chunks; rows are 128 or 256 bytes apart, so the two
// rows of a shared-memory access phase (eight lanes: rsel, rsel + 1) would meet in the same banks.  Lanes
// of odd rsel therefore walk their chunks in the order q ^ 1: register slot q of such a lane holds
// chunk q ^ 1, and it reads the vectors with the matching permutation (vgroup()).
template <typename T> struct Tile;
template <> struct Tile<__nv_bfloat16> {
    static constexpr int kStages = 5, kChunks = 2, kChunkElems = 8, kVecFlip = 2;
    static __device__ __forceinline__ void unpack(const uint4& raw, float* f) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            f[2 * e] = __uint_as_float(w[e] << 16);
            f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) h[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        return raw;
    }
};
template <> struct Tile<float> {
    static constexpr int kStages = 3, kChunks = 4, kChunkElems = 4, kVecFlip = 1;
    static __device__ __forceinline__ void unpack(const uint4& raw, float* f) {
        f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y);
        f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};

constexpr int kFlagBatch = 64;   // the computing threads fetch the flags of this many pairs at a time

template <typename T>
struct StepStage {
    alignas(128) T state[kStateElems];
    T raw[6][kN];                      // w, r, k, v, a, b of the pair as they lie in global memory
};

template <typename T>
struct StepSmem {
    StepStage<T> stage[Tile<T>::kStages];
    alignas(16) float vec[2][6][kN];   // decay, r, k, v, a, b of the current and the next pair
    unsigned char flags[2][kFlagBatch];
    uint64_t full[Tile<T>::kStages];   // the stage's bytes have arrived
    uint64_t done[Tile<T>::kStages];   // both computing warps have taken the stage into registers
};

__device__ __forceinline__ void compute_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tc::smem_u32(bar)) : "memory");
}
// 32 bytes to global memory in one instruction: a whole sector per lane
__device__ __forceinline__ void store32(void* dst, const uint4& lo, const uint4& hi) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(__cvta_generic_to_global(dst)), "r"(lo.x),
                 "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                 : "memory");
}

__device__ __forceinline__ float sum4(float x) {   // over the four lanes that share a row
    x += __shfl_xor_sync(0xffffffffu, x, 1);
    x += __shfl_xor_sync(0xffffffffu, x, 2);
    return x;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
wkv7_step_stream_kernel(int BH, int H, const T* __restrict__ w, const T* __restrict__ r, const T* __restrict__ k,
                        const T* __restrict__ v, const T* __restrict__ a, const T* __restrict__ b,
                        const T* __restrict__ s0, const uint32_t* __restrict__ length,
                        const uint8_t* __restrict__ new_starts, T* __restrict__ y, T* __restrict__ s_out,
                        int* __restrict__ status, long long s_batch_stride) {
    typedef Tile<T> TL;
    constexpr int kStages = TL::kStages, kChunks = TL::kChunks, kCE = TL::kChunkElems;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    StepSmem<T>& sm = *reinterpret_cast<StepSmem<T>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = lane & 3, rsel = lane >> 2, sw = rsel & 1;
    const int row0 = warp * 32 + rsel;                       // rows row0 + 8 g
    const int first = blockIdx.x, stride = gridDim.x;
    const int n_my = (BH - first + stride - 1) / stride;     // pairs first, first + stride, ...
    constexpr uint32_t kTileBytes = kStateElems * sizeof(T), kVecBytes = kN * sizeof(T);
    // element offset of the state of pair q: batch rows may be s_batch_stride elements apart (a state
    // that lives inside a larger per-sequence container), heads of one row are contiguous
    auto state_off = [&](int q) { return (size_t)(q / H) * (size_t)s_batch_stride + (size_t)(q % H) * kStateElems; };
    // byte offset inside a stage of register slot q of row group g, and float offset inside a vector of
    // the four columns that register elements 4 cc .. 4 cc + 3 hold
    auto chunk_off = [&](int g, int q) { return (uint32_t)(((row0 + 8 * g) * kN + 16 * p) * (int)sizeof(T) + ((q ^ sw) << 4)); };
    auto vgroup = [&](int cc) { return 16 * p + 4 * (cc ^ (sw * TL::kVecFlip)); };

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(&sm.full[s], 1);
            tc::mbar_init(&sm.done[s], 2);
        }
        tc::mbar_init_fence();
    }
    // Launched with programmatic stream serialization: the CTAs of this grid may become resident while the
    // kernel before it in the stream is still draining, and the grid after it likewise (it is released at
    // once: a dependent grid waits for the completion of this one where it needs it).  Nothing above reads or
    // writes global memory; everything below comes after the wait, i.e. after the preceding grid has
    // completed and its writes are visible.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __syncthreads();
    if (tid >= kComputeThreads) {
        // ---- copy warp: fill the ring, then refill every stage the computing warps hand back.  A
        // stage receives the state and the six vectors of its pair, so that everything an iteration
        // reads was requested a whole ring ahead of it.
        // Lane 0 announces the bytes and copies the state, lanes 1..6 copy one vector each: the seven
        // copies of a stage are issued side by side instead of one after another.
        const T* const src = lane == 1 ? w : lane == 2 ? r : lane == 3 ? k : lane == 4 ? v : lane == 5 ? a : b;
        auto fill = [&](int it, int s) {
            const int q = first + it * stride;
            if (lane == 0) {
                tc::mbar_expect_tx(&sm.full[s], kTileBytes + 6 * kVecBytes);
                tc::bulk_load(sm.stage[s].state, s0 + state_off(q), kTileBytes, &sm.full[s]);
            } else if (lane <= 6) {
                tc::bulk_load(sm.stage[s].raw[lane - 1], src + (size_t)q * kN, kVecBytes, &sm.full[s]);
            }
        };
        bool bad = false;
        for (int s = 0; s < kStages && s < n_my; ++s) fill(s, s);
        for (int it = 0; it + kStages < n_my; ++it) {
            const int s = it % kStages;
            if (!tc::mbar_wait(&sm.done[s], (uint32_t)(it / kStages) & 1u)) bad = true;
            fill(it + kStages, s);
        }
        if (bad && lane == 0 && status != nullptr) atomicExch(status, 3);
        return;
    }
    // ---- computing warps
    bool failed = false;
    // flags of the pairs of a batch of iterations: bit 0 = length is zero, bit 1 = start flag
    auto fetch_flags = [&](int it0) {
        const int it = it0 + tid;
        if (it < n_my) {
            const int bi = (first + it * stride) / H;
            sm.flags[(it0 / kFlagBatch) & 1][tid] = (unsigned char)((length[bi] == 0 ? 1 : 0) | (new_starts[bi] != 0 ? 2 : 0));
        }
    };
    // thread c turns channel c of the six vectors of a stage into fp32 (the decay into exp(-exp(w)))
    auto stage_vectors = [&](int it) {
        const int s = it % kStages;
        if (!tc::mbar_wait(&sm.full[s], (uint32_t)(it / kStages) & 1u)) failed = true;
#pragma unroll
        for (int m = 0; m < 6; ++m) {
            float x = to_f32<T>(sm.stage[s].raw[m][tid]);
            if (m == 0) x = expf(-expf(x));
            sm.vec[it & 1][m][tid] = x;
        }
    };
    fetch_flags(0);
    stage_vectors(0);
    compute_barrier();
    for (int it = 0; it < n_my; ++it) {
        const int bh = first + it * stride;
        const int s = it % kStages;
        const unsigned fl = sm.flags[(it / kFlagBatch) & 1][it % kFlagBatch];
        const bool keep_input = (fl & 1u) != 0;   // length == 0 returns the input state untouched
        const bool reset = (fl & 2u) != 0;
        const unsigned char* stage = reinterpret_cast<const unsigned char*>(sm.stage[s].state);
        float S[4][16];
#pragma unroll
        for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int q = 0; q < kChunks; ++q) TL::unpack(*reinterpret_cast<const uint4*>(stage + chunk_off(g, q)), &S[g][q * kCE]);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.done[s]);   // this warp has its half of the stage in registers
        T* const out = s_out + state_off(bh) + (size_t)row0 * kN + 16 * p;
        // register slot q of a lane of odd rsel holds chunk q ^ 1: such a lane stores its slots swapped
        auto write_state = [&]() {
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int q = 0; q < kChunks; q += 2) {
                    const uint4 c0 = TL::pack(&S[g][q * kCE]), c1 = TL::pack(&S[g][(q + 1) * kCE]);
                    if (sw) store32(out + (size_t)8 * g * kN + q * kCE, c1, c0);
                    else store32(out + (size_t)8 * g * kN + q * kCE, c0, c1);
                }
        };
        if (keep_input && s_out != s0) write_state();   // the input state goes out unchanged
        if (reset) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int e = 0; e < 16; ++e) S[g][e] = 0.f;
        }
        const float (*vec)[kN] = sm.vec[it & 1];
        float sa[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const float4 x = *reinterpret_cast<const float4*>(&vec[4][vgroup(cc)]);   // a
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                sa[g] = fmaf(S[g][4 * cc], x.x, sa[g]);
                sa[g] = fmaf(S[g][4 * cc + 1], x.y, sa[g]);
                sa[g] = fmaf(S[g][4 * cc + 2], x.z, sa[g]);
                sa[g] = fmaf(S[g][4 * cc + 3], x.w, sa[g]);
            }
        }
        float vv[4], yy[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            sa[g] = sum4(sa[g]);
            vv[g] = vec[3][row0 + 8 * g];
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const int c = vgroup(cc);
            const float4 d4 = *reinterpret_cast<const float4*>(&vec[0][c]);
            const float4 k4 = *reinterpret_cast<const float4*>(&vec[2][c]);
            const float4 b4 = *reinterpret_cast<const float4*>(&vec[5][c]);
            const float4 r4 = *reinterpret_cast<const float4*>(&vec[1][c]);
            const float dd[4] = {d4.x, d4.y, d4.z, d4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w};
            const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, rr[4] = {r4.x, r4.y, r4.z, r4.w};
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float& x = S[g][4 * cc + e];
                    x = fmaf(x, dd[e], fmaf(vv[g], kk[e], sa[g] * bb[e]));
                    yy[g] = fmaf(x, rr[e], yy[g]);
                }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            yy[g] = sum4(yy[g]);
            if (p == 0) y[(size_t)bh * kN + row0 + 8 * g] = from_f32<T>(yy[g]);
        }
        if (!keep_input) write_state();
        if (it + 1 < n_my) {
            if ((it + 1) % kFlagBatch == 0) fetch_flags(it + 1);
            stage_vectors(it + 1);
        }
        compute_barrier();   // the next pair's vectors (and flags) are complete
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
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem) != cudaSuccess || n < 1) n = 1;
            per_sm_of[dev] = n;
            status_of[dev] = wkv7_chunk_status_word();
            return cudaSuccess;
        }))
        return B200WKV_ELAUNCH;
    const int sm_count = sm_count_of_current_device(), per_sm = per_sm_of[dev];
    const int BH = B * H;
    const int grid = BH < sm_count * per_sm ? BH : sm_count * per_sm;   // one wave: every CTA resident
    // one step moves little data (177 MB at 256 sequences x 40 heads), so the microseconds between two launches
    // count: with this attribute the grid's CTAs are scheduled and set up while the previous kernel of the
    // stream finishes, and wait (griddepcontrol.wait) before they touch memory
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, BH, H, (const T*)w, (const T*)r, (const T*)k, (const T*)v, (const T*)a,
                                             (const T*)b, (const T*)s0, length, ns, (T*)y, (T*)s_out, status_of[dev],
                                             s_batch_stride);
    return e == cudaSuccess ? B200WKV_OK : B200WKV_ELAUNCH;
}

}  // namespace

// Requires s0 and the six streams 16-byte aligned (bulk copies), s_out 32-byte aligned (32-byte stores)
// and a batch stride that keeps every state so aligned; the caller checks.  s_out may be s0 (update in place): a pair's state
// is read into the ring before its own write-back and no other pair touches it.
int wkv7_step_stream(cudaStream_t st, int dtype, int B, int H, const void* w, const void* r, const void* k, const void* v,
                     const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                     void* s_out, long long s_batch_stride) {
    if (dtype == B200WKV_F32) return launch<float>(st, B, H, w, r, k, v, a, b, s0, length, ns, y, s_out, s_batch_stride);
    return launch<__nv_bfloat16>(st, B, H, w, r, k, v, a, b, s0, length, ns, y, s_out, s_batch_stride);
}

}  // namespace b200wkv

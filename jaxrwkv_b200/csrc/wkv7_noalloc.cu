// b200wkv7_fwd_bwd_static: forward + backward of the RWKV-7 recurrence in one call, with the
// state checkpoints that the backward re-enters from kept in a fixed device array that is part
// of the library image instead of a caller-provided residual buffer.
//
// Who needs this: a host that may not allocate device memory at the point where it wants the
// gradients.  The typical case is a custom-call handler running inside a compiled XLA program
// whose layer body is rematerialised (jaxrwkv wraps every layer in jax.checkpoint,
// src/jaxrwkv/rwkv7.py:276-277, so the WKV forward is executed again during the backward pass):
// the framework owns all device memory through its own pool, a handler is not allowed to call the
// CUDA allocator (it would synchronise the device and bypass the pool's accounting), and the
// recomputed forward has nowhere to put a residual unless the compiler adds one more result
// buffer.  With this entry point the handler passes only the operands and results it already has.
#include <mutex>

#include "common.cuh"

namespace b200wkv {
size_t wkv7_seq_residual_bytes(int B, int T, int H);
size_t wkv7_chunk_residual_bytes(int B, int T, int H);
}

extern "C" {
size_t b200wkv7_residual_bytes(int dtype, int B, int T, int H, int N);
int b200wkv7_fwd(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, void* y, void* s_out, void* residual, size_t residual_bytes,
                 unsigned flags);
int b200wkv7_bwd(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, const void* dy, const void* ds_out, void* residual,
                 size_t residual_bytes, void* dw, void* dr, void* dk, void* dv, void* da, void* db, void* ds0,
                 unsigned flags);
}

namespace {

constexpr size_t kStaticScratchBytes = (size_t)64 << 20;   // 64 MiB per device that loads the library

// File-scope device array: part of this translation unit's device module, not obtained from the
// allocator by any call.  With CUDA's default lazy module loading the module (and with it the
// backing of the array) is materialised on a device when the address is first asked for, i.e.
// inside the first call of the entry point on that device: that first call may therefore take
// device memory and synchronise, and it fails with B200WKV_ESYMBOL if a framework's pool has
// already taken all of it.  Make the first call (or set CUDA_MODULE_LOADING=EAGER) before the
// pool grows.  In host code the name is only a handle for cudaGetSymbolAddress; it is not a
// device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {};   // device address of g_static_scratch, per device ordinal

// One-time set-up for the current device: resolve the device address of the static array.
int static_scratch_for_current_device(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return B200WKV_ELAUNCH;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return B200WKV_ESYMBOL;
        }
        g_scratch_ptr[dev] = p;
    }
    *out = g_scratch_ptr[dev];
    return B200WKV_OK;
}

}  // namespace

extern "C" {

size_t b200wkv7_static_scratch_bytes(void) { return kStaticScratchBytes; }

int b200wkv7_fwd_bwd_static(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r,
                            const void* k, const void* v, const void* a, const void* b, const void* s0,
                            const uint32_t* length, const uint8_t* new_starts, const void* dy, const void* ds_out,
                            void* y, void* s_out, void* dw, void* dr, void* dk, void* dv, void* da, void* db,
                            void* ds0, unsigned flags) {
    const size_t need = b200wkv7_residual_bytes(dtype, B, T, H, N);
    if (need == 0) {
        // let the regular entry point produce the precise dtype / shape status
        return b200wkv7_fwd(stream, dtype, B, T, H, N, w, r, k, v, a, b, s0, length, new_starts, y, s_out, nullptr, 0, flags);
    }
    if (need > kStaticScratchBytes) return B200WKV_ESCRATCH;
    // everything either kernel pair could refuse is checked here, so that a bad argument of the
    // backward is reported before the forward has been enqueued
    if (!w || !r || !k || !v || !a || !b || !s0 || !length || !new_starts || !y || !s_out || !dw || !dr || !dk || !dv ||
        !da || !db || !ds0)
        return B200WKV_ENULL;
    void* scratch = nullptr;
    int st = static_scratch_for_current_device(&scratch);
    if (st != B200WKV_OK) return st;
    st = b200wkv7_fwd(stream, dtype, B, T, H, N, w, r, k, v, a, b, s0, length, new_starts, y, s_out, scratch, need, flags);
    if (st != B200WKV_OK) return st;
    return b200wkv7_bwd(stream, dtype, B, T, H, N, w, r, k, v, a, b, s0, length, new_starts, dy, ds_out, scratch, need,
                        dw, dr, dk, dv, da, db, ds0, flags);
}

}  // extern "C"

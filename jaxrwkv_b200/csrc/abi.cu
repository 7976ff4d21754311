// extern "C" entry points declared in include/b200wkv.h: argument validation and dispatch.
#include "common.cuh"

namespace b200wkv {
size_t wkv7_seq_residual_bytes(int B, int T, int H);
int wkv7_seq_fwd(cudaStream_t st, int dtype, int B, int T, int H, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* ns, void* y, void* s_out, void* residual);
int wkv7_seq_bwd(cudaStream_t st, int dtype, int B, int T, int H, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* ns, const void* dy, const void* ds_out, const void* residual, void* dw, void* dr,
                 void* dk, void* dv, void* da, void* db, void* ds0);

size_t wkv7_chunk_residual_bytes(int B, int T, int H);
int wkv7_chunk_fwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                   const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                   void* s_out, void* residual, void* dbg);
int wkv7_chunk_bwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                   const void* a, const void* b, const uint32_t* length, const uint8_t* ns, const void* dy,
                   const void* ds_out, const void* residual, void* dw, void* dr, void* dk, void* dv, void* da,
                   void* db, void* ds0);
int wkv7_chunk_status();

static int check_dims(int dtype, int B, int T, int H, int N) {
    if (dtype != B200WKV_F32 && dtype != B200WKV_BF16) return B200WKV_EDTYPE;
    if (B < 1 || T < 1 || H < 1 || N != kN) return B200WKV_ESHAPE;
    // element counts are indexed with size_t; the grid is B*H blocks
    if ((long long)B * H > 2147483647LL) return B200WKV_ESHAPE;
    return B200WKV_OK;
}
}  // namespace b200wkv

using namespace b200wkv;

extern "C" {

const char* b200wkv_strerror(int status) {
    switch (status) {
        case B200WKV_OK: return "ok";
        case B200WKV_EDTYPE: return "unsupported element type (expected B200WKV_F32 or B200WKV_BF16)";
        case B200WKV_ESHAPE: return "bad shape (every dimension must be >= 1 and the head size must be 64)";
        case B200WKV_ENULL: return "a required pointer is NULL";
        case B200WKV_ERESIDUAL: return "residual buffer is smaller than the size reported by *_residual_bytes";
        case B200WKV_ELAUNCH: return "CUDA kernel launch failed";
        case B200WKV_EUNSUPPORTED: return "combination not available in this build";
        case B200WKV_ESCRATCH: return "problem exceeds the fixed built-in scratch area";
        default: return "unknown status";
    }
}

int b200wkv_abi_version(void) { return 1; }

size_t b200wkv7_residual_bytes(int dtype, int B, int T, int H, int N) {
    if (check_dims(dtype, B, T, H, N) != B200WKV_OK) return 0;
    // fp32 uses the sequential kernels (a state every 16 tokens); bf16 uses the chunked tensor-core
    // kernels (a state every 64 tokens) unless B200WKV_FLAG_SEQUENTIAL asks otherwise, so size for both
    const size_t seq = wkv7_seq_residual_bytes(B, T, H);
    if (dtype == B200WKV_F32) return seq;
    const size_t chk = wkv7_chunk_residual_bytes(B, T, H);
    return seq > chk ? seq : chk;
}

int b200wkv7_fwd(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, void* y, void* s_out, void* residual, size_t residual_bytes,
                 unsigned flags) {
    int st = check_dims(dtype, B, T, H, N);
    if (st != B200WKV_OK) return st;
    if (!w || !r || !k || !v || !a || !b || !s0 || !length || !new_starts || !y || !s_out) return B200WKV_ENULL;
    if (residual != nullptr && residual_bytes < b200wkv7_residual_bytes(dtype, B, T, H, N)) return B200WKV_ERESIDUAL;
    if (dtype == B200WKV_BF16 && !(flags & B200WKV_FLAG_SEQUENTIAL))
        return wkv7_chunk_fwd((cudaStream_t)stream, B, T, H, w, r, k, v, a, b, s0, length, new_starts, y, s_out,
                              residual, nullptr);
    return wkv7_seq_fwd((cudaStream_t)stream, dtype, B, T, H, w, r, k, v, a, b, s0, length, new_starts, y, s_out,
                        residual);
}

int b200wkv7_bwd(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, const void* dy, const void* ds_out, const void* residual,
                 size_t residual_bytes, void* dw, void* dr, void* dk, void* dv, void* da, void* db, void* ds0,
                 unsigned flags) {
    int st = check_dims(dtype, B, T, H, N);
    if (st != B200WKV_OK) return st;
    if (!w || !r || !k || !v || !a || !b || !s0 || !length || !new_starts || !residual || !dw || !dr || !dk || !dv ||
        !da || !db || !ds0)
        return B200WKV_ENULL;
    if (residual_bytes < b200wkv7_residual_bytes(dtype, B, T, H, N)) return B200WKV_ERESIDUAL;
    // must match the kernel family that filled the residual in b200wkv7_fwd (same dtype and flags)
    if (dtype == B200WKV_BF16 && !(flags & B200WKV_FLAG_SEQUENTIAL))
        return wkv7_chunk_bwd((cudaStream_t)stream, B, T, H, w, r, k, v, a, b, length, new_starts, dy, ds_out,
                              residual, dw, dr, dk, dv, da, db, ds0);
    return wkv7_seq_bwd((cudaStream_t)stream, dtype, B, T, H, w, r, k, v, a, b, s0, length, new_starts, dy, ds_out,
                        residual, dw, dr, dk, dv, da, db, ds0);
}

}  // extern "C"

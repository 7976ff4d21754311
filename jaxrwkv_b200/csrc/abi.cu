// extern "C" entry points declared in include/b200wkv.h: argument validation and dispatch.
#include <initializer_list>
#include "common.cuh"
#include "chunk_common.cuh"
#include "../../include/b200wkv_debug.h"

namespace b200wkv {
size_t wkv7_seq_residual_bytes(int B, int T, int H);
int wkv7_seq_fwd(cudaStream_t st, int dtype, int B, int T, int H, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* ns, void* y, void* s_out, void* residual, const int* run_if, int run_ticket,
                 int* residual_mark);
int wkv7_seq_bwd(cudaStream_t st, int dtype, int B, int T, int H, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* ns, const void* dy, const void* ds_out, const void* residual, void* dw, void* dr,
                 void* dk, void* dv, void* da, void* db, void* ds0, const int* run_if);

int wkv7_step(cudaStream_t st, int dtype, int B, int H, const void* w, const void* r, const void* k, const void* v,
              const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
              void* s_out);
int wkv7_step_stream(cudaStream_t st, int dtype, int B, int H, const void* w, const void* r, const void* k, const void* v,
                     const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                     void* s_out, long long s_batch_stride);
size_t wkv7_chunk_residual_bytes(int B, int T, int H);
int wkv7_chunk_fwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                   const void* a, const void* b, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                   void* s_out, void* residual, int* residual_mark, int** range_flag, int* range_ticket);
int wkv7_chunk_bwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                   const void* a, const void* b, const uint32_t* length, const uint8_t* ns, const void* dy,
                   const void* ds_out, void* residual, const int* residual_mark, const int* fast, void* dw, void* dr,
                   void* dk, void* dv, void* da, void* db, void* ds0);
int wkv7_carry_bwd(cudaStream_t st, int B, int T, int H, const uint32_t* length, const uint8_t* ns, const void* dy,
                   const void* ds_out, void* residual, const int* residual_mark, void* ds0);
int wkv7_grad_bwd(cudaStream_t st, int B, int T, int H, const void* w, const void* r, const void* k, const void* v,
                  const void* a, const void* b, const uint32_t* length, const uint8_t* ns, const void* dy, void* residual,
                  const int* residual_mark, void* dw, void* dr, void* dk, void* dv, void* da, void* db);
int wkv7_chunk_status();

size_t wkv6_seq_residual_bytes(int B, int T, int H);
int wkv6_seq_fwd(cudaStream_t st, int dtype, int B, int T, int H, const void* r, const void* k, const void* v,
                 const void* w, int per_token, const void* u, const void* s0, const uint32_t* length,
                 const uint8_t* ns, void* y, void* s_out, void* residual, const int* run_if, int run_ticket,
                 int* residual_mark);
int wkv6_seq_bwd(cudaStream_t st, int dtype, int B, int T, int H, const void* r, const void* k, const void* v,
                 const void* w, int per_token, const void* u, const uint32_t* length, const uint8_t* ns,
                 const void* dy, const void* ds_out, const void* residual, void* dr, void* dk, void* dv, void* dw,
                 void* du, void* ds0, const int* run_if);
size_t wkv6_chunk_residual_bytes(int B, int T, int H);
int wkv6_chunk_fwd(cudaStream_t st, int B, int T, int H, const void* r, const void* k, const void* v, const void* w,
                   int per_token, const void* u, const void* s0, const uint32_t* length, const uint8_t* ns, void* y,
                   void* s_out, void* residual, int* residual_mark, int** flag, int* ticket);
int wkv6_chunk_bwd(cudaStream_t st, int B, int T, int H, const void* r, const void* k, const void* v, const void* w,
                   int per_token, const void* u, const uint32_t* length, const uint8_t* ns, const void* dy, const void* ds_out,
                   void* residual, const int* residual_mark, void* dr, void* dk, void* dv, void* dw, void* du, void* ds0);
size_t wkv4_residual_bytes(int B, int T, int C);
int wkv4_fwd(cudaStream_t st, int dtype, int B, int T, int C, const void* w, const void* u, const void* k, const void* v,
             const void* s0, const uint32_t* length, const uint8_t* ns, void* s_out, void* y, void* residual);
int wkv4_bwd(cudaStream_t st, int dtype, int B, int T, int C, const void* w, const void* u, const void* k, const void* v,
             const void* gy, const uint32_t* length, const uint8_t* ns, const void* gs_new, const void* residual,
             void* gw, void* gu, void* gk, void* gv, void* gs);

int wkv7_mix_partial_rows(int rows, int C);
int wkv7_mix_pre_fwd(cudaStream_t st, int dtype, int rows, int C, int use_vmix, const void* k, const void* wl, const void* al,
                     const void* v, const void* vf, const void* vl, const void* w0, const void* a0, const void* v0,
                     const void* k_k, const void* k_a, void* w, void* kp, void* vp, void* ai, void* bi);
int wkv7_mix_pre_bwd(cudaStream_t st, int dtype, int rows, int C, int use_vmix, const void* k, const void* wl, const void* al,
                     const void* v, const void* vf, const void* vl, const void* w0, const void* a0, const void* v0,
                     const void* k_k, const void* k_a, const void* gw, const void* gkp, const void* gvp, const void* gai,
                     const void* gbi, void* dk, void* dwl, void* dal, void* dv, void* dvf, void* dvl, float* partial);
int wkv7_mix_post_fwd(cudaStream_t st, int dtype, int rows, int C, float eps, const void* y, const void* r, const void* kp,
                      const void* vp, const void* g, const void* ln_w, const void* ln_b, const void* r_k, void* x);
int wkv7_mix_post_bwd(cudaStream_t st, int dtype, int rows, int C, float eps, const void* y, const void* r, const void* kp,
                      const void* vp, const void* g, const void* ln_w, const void* ln_b, const void* r_k, const void* gx, void* dy,
                      void* dr, void* dkp, void* dvp, void* dg, float* partial);
int token_shift_fwd(cudaStream_t st, int dtype, int B, int T, int D, int M, const void* x, const void* prev,
                    const void* mix, const uint32_t* length, const uint8_t* ns, void* out, void* state_out);
int token_shift_bwd(cudaStream_t st, int dtype, int B, int T, int D, int M, const void* x, const void* prev,
                    const void* mix, const uint32_t* length, const uint8_t* ns, const void* gout, const void* gstate,
                    void* gx, void* gprev, void* gmix);

// The bf16 forward normally runs the chunked tensor-core kernel; a decay outside that kernel's range makes
// the token-sequential kernel behind it redo the call.  The last bytes of the residual tell the backward
// which of the two wrote it.
constexpr size_t kResidualMarkBytes = 16;
static int* residual_mark_of(void* residual, size_t bytes) {
    return residual ? reinterpret_cast<int*>(static_cast<char*>(residual) + bytes - kResidualMarkBytes) : nullptr;
}

static int check_dims(int dtype, int B, int T, int H, int N) {
    if (dtype != B200WKV_F32 && dtype != B200WKV_BF16) return B200WKV_EDTYPE;
    if (B < 1 || T < 1 || H < 1 || N != kN) return B200WKV_ESHAPE;
    // element counts are indexed with size_t; the grid is B*H blocks
    if ((long long)B * H > 2147483647LL || (long long)B * T > 2147483647LL) return B200WKV_ESHAPE;   // token rows index tensor maps
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
        case B200WKV_ESYMBOL: return "the built-in scratch area could not be materialised on this device (module load failed: out of device memory?)";
        default: return "unknown status";
    }
}

int b200wkv_abi_version(void) { return 2; }

int b200wkv_device_status(void) { return wkv7_chunk_status(); }

size_t b200wkv7_residual_bytes(int dtype, int B, int T, int H, int N) {
    if (check_dims(dtype, B, T, H, N) != B200WKV_OK) return 0;
    // fp32 uses the sequential kernels (a state every 16 tokens); bf16 uses the chunked tensor-core
    // kernels (a state every 64 tokens) unless B200WKV_FLAG_SEQUENTIAL asks otherwise, so size for both
    const size_t seq = wkv7_seq_residual_bytes(B, T, H);
    if (dtype == B200WKV_F32) return seq;
    const size_t chk = wkv7_chunk_residual_bytes(B, T, H);
    // + one word at the end that says which of the two formats the forward left (see residual_mark_of)
    return (seq > chk ? seq : chk) + kResidualMarkBytes;
}

int b200wkv7_fwd(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, void* y, void* s_out, void* residual, size_t residual_bytes,
                 unsigned flags) {
    int st = check_dims(dtype, B, T, H, N);
    if (st != B200WKV_OK) return st;
    if (!w || !r || !k || !v || !a || !b || !s0 || !length || !new_starts || !y || !s_out) return B200WKV_ENULL;
    if (residual != nullptr && residual_bytes < b200wkv7_residual_bytes(dtype, B, T, H, N)) return B200WKV_ERESIDUAL;
    // one token and no residual wanted (recurrent decoding): a single pass over the state
    if (T == 1 && residual == nullptr)
        return wkv7_step((cudaStream_t)stream, dtype, B, H, w, r, k, v, a, b, s0, length, new_starts, y, s_out);
    if (dtype == B200WKV_BF16 && !(flags & B200WKV_FLAG_SEQUENTIAL)) {
        int* mark = residual_mark_of(residual, b200wkv7_residual_bytes(dtype, B, T, H, N));
        int *range_flag = nullptr, ticket = 0;
        st = wkv7_chunk_fwd((cudaStream_t)stream, B, T, H, w, r, k, v, a, b, s0, length, new_starts, y, s_out, residual, mark,
                            &range_flag, &ticket);
        if (st != B200WKV_OK) return st;
        // does nothing unless the kernel above met a decay outside its range and left its ticket
        return wkv7_seq_fwd((cudaStream_t)stream, dtype, B, T, H, w, r, k, v, a, b, s0, length, new_starts, y, s_out, residual,
                            range_flag, ticket, mark);
    }
    return wkv7_seq_fwd((cudaStream_t)stream, dtype, B, T, H, w, r, k, v, a, b, s0, length, new_starts, y, s_out,
                        residual, nullptr, 0, nullptr);
}

int b200wkv7_bwd(void* stream, int dtype, int B, int T, int H, int N, const void* w, const void* r, const void* k,
                 const void* v, const void* a, const void* b, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, const void* dy, const void* ds_out, void* residual,
                 size_t residual_bytes, void* dw, void* dr, void* dk, void* dv, void* da, void* db, void* ds0,
                 unsigned flags) {
    int st = check_dims(dtype, B, T, H, N);
    if (st != B200WKV_OK) return st;
    if (!w || !r || !k || !v || !a || !b || !s0 || !length || !new_starts || !residual || !dw || !dr || !dk || !dv ||
        !da || !db || !ds0)
        return B200WKV_ENULL;
    if (residual_bytes < b200wkv7_residual_bytes(dtype, B, T, H, N)) return B200WKV_ERESIDUAL;
    // must match the kernel family that filled the residual in b200wkv7_fwd (same dtype and flags)
    if (dtype == B200WKV_BF16 && !(flags & B200WKV_FLAG_SEQUENTIAL)) {
        const int* mark = residual_mark_of(residual, b200wkv7_residual_bytes(dtype, B, T, H, N));
        const int* fast = reinterpret_cast<const int*>(static_cast<const char*>(residual) + carry_layout(B, T, H).fast);
        if (T % kC == 0) {
            // sequences the forward walked in full saved blocks: the sequential state-gradient carry, then the
            // gradients of all blocks in parallel
            st = wkv7_carry_bwd((cudaStream_t)stream, B, T, H, length, new_starts, dy, ds_out, residual, mark, ds0);
            if (st != B200WKV_OK) return st;
            st = wkv7_grad_bwd((cudaStream_t)stream, B, T, H, w, r, k, v, a, b, length, new_starts, dy, residual, mark, dw, dr, dk,
                               dv, da, db);
            if (st != B200WKV_OK) return st;
        }
        // every other sequence (start flags or `length` inside a block, ragged T): the one-kernel backward
        st = wkv7_chunk_bwd((cudaStream_t)stream, B, T, H, w, r, k, v, a, b, length, new_starts, dy, ds_out, residual, mark,
                            fast, dw, dr, dk, dv, da, db, ds0);
        if (st != B200WKV_OK) return st;
        return wkv7_seq_bwd((cudaStream_t)stream, dtype, B, T, H, w, r, k, v, a, b, s0, length, new_starts, dy, ds_out,
                            residual, dw, dr, dk, dv, da, db, ds0, mark);
    }
    return wkv7_seq_bwd((cudaStream_t)stream, dtype, B, T, H, w, r, k, v, a, b, s0, length, new_starts, dy, ds_out,
                        residual, dw, dr, dk, dv, da, db, ds0, nullptr);
}

size_t b200wkv6_residual_bytes(int dtype, int B, int T, int H, int N) {
    if (check_dims(dtype, B, T, H, N) != B200WKV_OK) return 0;
    // fp32 uses the sequential kernels (an fp32 state every 16 tokens); bf16 uses the chunked tensor-core kernels (a
    // bf16 state every 16 tokens) with the sequential ones as their fallback, so size for both, plus one word at
    // the end that says which of the two formats the forward left
    const size_t seq = wkv6_seq_residual_bytes(B, T, H);
    if (dtype == B200WKV_F32) return seq;
    const size_t chk = wkv6_chunk_residual_bytes(B, T, H);
    return (seq > chk ? seq : chk) + kResidualMarkBytes;
}

int b200wkv6_fwd(void* stream, int dtype, int version, int B, int T, int H, int N, const void* r, const void* k,
                 const void* v, const void* w, const void* u, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, void* y, void* s_out, void* residual, size_t residual_bytes,
                 unsigned flags) {
    int st = check_dims(dtype, B, T, H, N);
    if (st != B200WKV_OK) return st;
    if (version != 5 && version != 6) return B200WKV_EUNSUPPORTED;
    if (!r || !k || !v || !w || !u || !s0 || !length || !new_starts || !y || !s_out) return B200WKV_ENULL;
    if (residual != nullptr && residual_bytes < b200wkv6_residual_bytes(dtype, B, T, H, N)) return B200WKV_ERESIDUAL;
    if (dtype == B200WKV_BF16) {
        int* mark = residual_mark_of(residual, b200wkv6_residual_bytes(dtype, B, T, H, N));
        // With a constant decay (versions 5, 5.2) the decay's gradient is a sum over ALL tokens of per-token terms that
        // largely cancel; taken from bf16 tensor-core products it is only good to a few percent (10 % on short
        // sequences), so training calls of those versions keep the fp32-arithmetic sequential kernels.  Their
        // inference calls, and everything of version 6, take the chunked kernels.
        if ((flags & B200WKV_FLAG_SEQUENTIAL) || (version != 6 && residual != nullptr))
            return wkv6_seq_fwd((cudaStream_t)stream, dtype, B, T, H, r, k, v, w, version == 6, u, s0, length, new_starts, y,
                                s_out, residual, nullptr, 0, mark);
        // the chunked tensor-core kernel, and behind it the sequential kernel, which runs only if the chunked one met
        // something outside its domain (it then redoes the whole call and marks the residual as its own)
        int* flag = nullptr;
        int ticket = 0;
        st = wkv6_chunk_fwd((cudaStream_t)stream, B, T, H, r, k, v, w, version == 6, u, s0, length, new_starts, y, s_out,
                            residual, mark, &flag, &ticket);
        if (st != B200WKV_OK) return st;
        return wkv6_seq_fwd((cudaStream_t)stream, dtype, B, T, H, r, k, v, w, version == 6, u, s0, length, new_starts, y,
                            s_out, residual, flag, ticket, mark);
    }
    return wkv6_seq_fwd((cudaStream_t)stream, dtype, B, T, H, r, k, v, w, version == 6, u, s0, length, new_starts, y,
                        s_out, residual, nullptr, 0, nullptr);
}

int b200wkv6_bwd(void* stream, int dtype, int version, int B, int T, int H, int N, const void* r, const void* k,
                 const void* v, const void* w, const void* u, const void* s0, const uint32_t* length,
                 const uint8_t* new_starts, const void* dy, const void* ds_out, void* residual,
                 size_t residual_bytes, void* dr, void* dk, void* dv, void* dw, void* du, void* ds0, unsigned flags) {
    int st = check_dims(dtype, B, T, H, N);
    if (st != B200WKV_OK) return st;
    if (version != 5 && version != 6) return B200WKV_EUNSUPPORTED;
    if (!r || !k || !v || !w || !u || !s0 || !length || !new_starts || !residual || !dr || !dk || !dv || !dw || !du || !ds0)
        return B200WKV_ENULL;
    if (residual_bytes < b200wkv6_residual_bytes(dtype, B, T, H, N)) return B200WKV_ERESIDUAL;
    (void)flags;
    if (dtype == B200WKV_BF16) {
        // the forward's mark decides on the device which of the two runs; the other returns at once
        const int* mark = residual_mark_of(residual, b200wkv6_residual_bytes(dtype, B, T, H, N));
        st = wkv6_chunk_bwd((cudaStream_t)stream, B, T, H, r, k, v, w, version == 6, u, length, new_starts, dy, ds_out,
                            residual, mark, dr, dk, dv, dw, du, ds0);
        if (st != B200WKV_OK) return st;
        return wkv6_seq_bwd((cudaStream_t)stream, dtype, B, T, H, r, k, v, w, version == 6, u, length, new_starts, dy, ds_out,
                            residual, dr, dk, dv, dw, du, ds0, mark);
    }
    return wkv6_seq_bwd((cudaStream_t)stream, dtype, B, T, H, r, k, v, w, version == 6, u, length, new_starts, dy,
                        ds_out, residual, dr, dk, dv, dw, du, ds0, nullptr);
}

size_t b200wkv4_residual_bytes(int dtype, int B, int T, int C) {
    if ((dtype != B200WKV_F32 && dtype != B200WKV_BF16) || B < 1 || T < 1 || C < 1) return 0;
    return wkv4_residual_bytes(B, T, C);
}

int b200wkv4_fwd(void* stream, int dtype, int B, int T, int C, const void* w, const void* u, const void* k,
                 const void* v, const void* s0, const uint32_t* length, const uint8_t* new_starts, void* s_out, void* y,
                 void* residual, size_t residual_bytes, unsigned flags) {
    if (dtype != B200WKV_F32 && dtype != B200WKV_BF16) return B200WKV_EDTYPE;
    if (B < 1 || T < 1 || C < 1 || (long long)B * C > 2147483647LL) return B200WKV_ESHAPE;
    if (!w || !u || !k || !v || !s0 || !length || !new_starts || !s_out || !y) return B200WKV_ENULL;
    if (residual != nullptr && residual_bytes < wkv4_residual_bytes(B, T, C)) return B200WKV_ERESIDUAL;
    (void)flags;
    return wkv4_fwd((cudaStream_t)stream, dtype, B, T, C, w, u, k, v, s0, length, new_starts, s_out, y, residual);
}

int b200wkv4_bwd(void* stream, int dtype, int B, int T, int C, const void* w, const void* u, const void* k,
                 const void* v, const void* gy, const void* s0, const uint32_t* length, const uint8_t* new_starts,
                 const void* gs_new, const void* residual, size_t residual_bytes, void* gw, void* gu, void* gk,
                 void* gv, void* gs, unsigned flags) {
    if (dtype != B200WKV_F32 && dtype != B200WKV_BF16) return B200WKV_EDTYPE;
    if (B < 1 || T < 1 || C < 1 || (long long)B * C > 2147483647LL) return B200WKV_ESHAPE;
    if (!w || !u || !k || !v || !s0 || !length || !new_starts || !residual || !gw || !gu || !gk || !gv || !gs)
        return B200WKV_ENULL;
    if (residual_bytes < wkv4_residual_bytes(B, T, C)) return B200WKV_ERESIDUAL;
    (void)flags;
    return wkv4_bwd((cudaStream_t)stream, dtype, B, T, C, w, u, k, v, gy, length, new_starts, gs_new, residual, gw, gu,
                    gk, gv, gs);
}

int b200wkv7_step_inplace(void* stream, int dtype, int B, int H, int N, const void* w, const void* r, const void* k,
                          const void* v, const void* a, const void* b, void* state, long long state_batch_stride,
                          const uint32_t* length, const uint8_t* new_starts, void* y) {
    int st = check_dims(dtype, B, 1, H, N);
    if (st != B200WKV_OK) return st;
    if (!w || !r || !k || !v || !a || !b || !state || !length || !new_starts || !y) return B200WKV_ENULL;
    const long long esz = dtype == B200WKV_F32 ? 4 : 2;
    if (state_batch_stride < (long long)H * N * N) return B200WKV_ESHAPE;
    const uintptr_t vec_bits = reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(r) | reinterpret_cast<uintptr_t>(k) |
                               reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b);
    if ((reinterpret_cast<uintptr_t>(state) & 31u) != 0 || (state_batch_stride * esz) % 32 != 0 || (vec_bits & 15u) != 0)
        return B200WKV_EUNSUPPORTED;
    return wkv7_step_stream((cudaStream_t)stream, dtype, B, H, w, r, k, v, a, b, state, length, new_starts, y, state,
                            state_batch_stride);
}

namespace {
int check_mix(int dtype, long long rows, int H, int N) {
    if (dtype != B200WKV_F32 && dtype != B200WKV_BF16) return B200WKV_EDTYPE;
    if (N != kN || H < 1 || H > 128 || rows < 1 || rows > 2147483647LL) return B200WKV_ESHAPE;
    return B200WKV_OK;
}
bool aligned16(std::initializer_list<const void*> ps) {
    for (const void* p : ps)
        if ((reinterpret_cast<uintptr_t>(p) & 15u) != 0) return false;
    return true;
}
}  // namespace

int b200wkv7_mix_partial_rows(long long rows, int H, int N) {
    if (check_mix(B200WKV_F32, rows, H, N) != B200WKV_OK) return 0;
    return wkv7_mix_partial_rows((int)rows, H * N);
}

int b200wkv7_mix_pre_fwd(void* stream, int dtype, long long rows, int H, int N, int use_vmix, const void* k, const void* wl,
                         const void* al, const void* v, const void* v_first, const void* vl, const void* w0, const void* a0,
                         const void* v0, const void* k_k, const void* k_a, void* w, void* k_out, void* v_out, void* a_i,
                         void* b_i) {
    int st = check_mix(dtype, rows, H, N);
    if (st != B200WKV_OK) return st;
    if (!k || !wl || !al || !v || !w0 || !a0 || !k_k || !k_a || !w || !k_out || !v_out || !a_i || !b_i) return B200WKV_ENULL;
    if (use_vmix && (!v_first || !vl || !v0)) return B200WKV_ENULL;
    if (!aligned16({k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, w, k_out, v_out, a_i, b_i})) return B200WKV_EUNSUPPORTED;
    return wkv7_mix_pre_fwd((cudaStream_t)stream, dtype, (int)rows, H * N, use_vmix ? 1 : 0, k, wl, al, v, v_first, vl, w0, a0,
                            v0, k_k, k_a, w, k_out, v_out, a_i, b_i);
}

int b200wkv7_mix_pre_bwd(void* stream, int dtype, long long rows, int H, int N, int use_vmix, const void* k, const void* wl,
                         const void* al, const void* v, const void* v_first, const void* vl, const void* w0, const void* a0,
                         const void* v0, const void* k_k, const void* k_a, const void* gw, const void* gk_out,
                         const void* gv_out, const void* ga_i, const void* gb_i, void* dk, void* dwl, void* dal, void* dv,
                         void* dv_first, void* dvl, float* partial) {
    int st = check_mix(dtype, rows, H, N);
    if (st != B200WKV_OK) return st;
    if (!k || !wl || !al || !v || !w0 || !a0 || !k_k || !k_a || !gw || !gk_out || !gv_out || !ga_i || !gb_i || !dk || !dwl ||
        !dal || !dv || !partial)
        return B200WKV_ENULL;
    if (use_vmix && (!v_first || !vl || !v0 || !dv_first || !dvl)) return B200WKV_ENULL;
    if (!aligned16({k, wl, al, v, v_first, vl, w0, a0, v0, k_k, k_a, gw, gk_out, gv_out, ga_i, gb_i, dk, dwl, dal, dv, dv_first,
                    dvl, partial}))
        return B200WKV_EUNSUPPORTED;
    return wkv7_mix_pre_bwd((cudaStream_t)stream, dtype, (int)rows, H * N, use_vmix ? 1 : 0, k, wl, al, v, v_first, vl, w0, a0,
                            v0, k_k, k_a, gw, gk_out, gv_out, ga_i, gb_i, dk, dwl, dal, dv, dv_first, dvl, partial);
}

int b200wkv7_mix_post_fwd(void* stream, int dtype, long long rows, int H, int N, float eps, const void* y, const void* r,
                          const void* k, const void* v, const void* g, const void* ln_w, const void* ln_b, const void* r_k,
                          void* x) {
    int st = check_mix(dtype, rows, H, N);
    if (st != B200WKV_OK) return st;
    if (!y || !r || !k || !v || !g || !ln_w || !ln_b || !r_k || !x) return B200WKV_ENULL;
    if (!aligned16({y, r, k, v, g, ln_w, ln_b, r_k, x})) return B200WKV_EUNSUPPORTED;
    return wkv7_mix_post_fwd((cudaStream_t)stream, dtype, (int)rows, H * N, eps, y, r, k, v, g, ln_w, ln_b, r_k, x);
}

int b200wkv7_mix_post_bwd(void* stream, int dtype, long long rows, int H, int N, float eps, const void* y, const void* r,
                          const void* k, const void* v, const void* g, const void* ln_w, const void* ln_b, const void* r_k,
                          const void* gx, void* dy, void* dr, void* dk, void* dv, void* dg, float* partial) {
    int st = check_mix(dtype, rows, H, N);
    if (st != B200WKV_OK) return st;
    if (!y || !r || !k || !v || !g || !ln_w || !ln_b || !r_k || !gx || !dy || !dr || !dk || !dv || !dg || !partial)
        return B200WKV_ENULL;
    if (!aligned16({y, r, k, v, g, ln_w, ln_b, r_k, gx, dy, dr, dk, dv, dg, partial})) return B200WKV_EUNSUPPORTED;
    return wkv7_mix_post_bwd((cudaStream_t)stream, dtype, (int)rows, H * N, eps, y, r, k, v, g, ln_w, ln_b, r_k, gx, dy, dr, dk,
                             dv, dg, partial);
}

int b200wkv_debug_split_plan(int chains, int n_blk, int per_sm, int* grid, int* seg) {
    if (chains < 1 || n_blk < 1 || per_sm < 1 || !grid || !seg) return B200WKV_ESHAPE;
    const SplitPlan p = plan_split(chains, n_blk, per_sm, sm_count_of_current_device());
    *grid = p.grid;
    *seg = p.seg;
    return B200WKV_OK;
}

int b200wkv_debug_runs(int chains, int seg, int grid, int cta, int* runs, int capacity) {
    if (chains < 1 || seg < 1 || grid < 1 || cta < 0 || cta >= grid || !runs) return B200WKV_ESHAPE;
    const long long lo = (long long)chains * seg * cta / grid, hi = (long long)chains * seg * (cta + 1) / grid;
    if (hi <= lo) return 0;
    const int n = run_count(lo, hi, seg);
    for (int order = 0; order < n && order < capacity; ++order) {
        const RunPlan r = run_at(lo, hi, seg, order);
        runs[3 * order] = r.chain;
        runs[3 * order + 1] = r.seg_from;
        runs[3 * order + 2] = r.seg_to;
    }
    return n;
}

static int check_shift(int dtype, int B, int T, int D, int M) {
    if (dtype != B200WKV_F32 && dtype != B200WKV_BF16) return B200WKV_EDTYPE;
    if (B < 1 || T < 1 || D < 4 || (D % 4) != 0 || M < 1 || M > 8 || (long long)B * T > 2147483647LL || B > 65535) return B200WKV_ESHAPE;
    return B200WKV_OK;
}

int b200wkv_token_shift_fwd(void* stream, int dtype, int B, int T, int D, int M, const void* x, const void* prev,
                            const void* mix, const uint32_t* length, const uint8_t* new_starts, void* out,
                            void* state_out) {
    int st = check_shift(dtype, B, T, D, M);
    if (st != B200WKV_OK) return st;
    if (!x || !prev || !mix || !length || !new_starts || !out || !state_out) return B200WKV_ENULL;
    return token_shift_fwd((cudaStream_t)stream, dtype, B, T, D, M, x, prev, mix, length, new_starts, out, state_out);
}

int b200wkv_token_shift_bwd(void* stream, int dtype, int B, int T, int D, int M, const void* x, const void* prev,
                            const void* mix, const uint32_t* length, const uint8_t* new_starts, const void* gout,
                            const void* gstate, void* gx, void* gprev, void* gmix) {
    int st = check_shift(dtype, B, T, D, M);
    if (st != B200WKV_OK) return st;
    if (!x || !prev || !mix || !length || !new_starts || !gout || !gx || !gprev || !gmix) return B200WKV_ENULL;
    return token_shift_bwd((cudaStream_t)stream, dtype, B, T, D, M, x, prev, mix, length, new_starts, gout, gstate, gx,
                           gprev, gmix);
}

}  // extern "C"

/*
 * b200wkv — C ABI of the B200 (sm_100a) WKV state-recurrence kernels.
 *
 * This is the boundary a host framework binds: plain pointers and sizes, no
 * C++ or framework types.  Every pointer named "device" must be valid on the
 * CUDA device that is current when the call is made; `stream` is a
 * cudaStream_t passed as void* (NULL = the legacy default stream).  Calls only
 * enqueue work on `stream`: they never allocate, free, synchronise or retain
 * caller memory, and they return 0 on success or a negative B200WKV_E* code
 * (text via b200wkv_strerror) without having launched anything.
 *
 * Tensor layouts are the ones jaxrwkv's batched custom calls use (C order):
 *   r, w, k, v, a, b, y, d*   (B, T, H, N)   element type = `dtype`
 *   states                    (B, H, N, N)   element type = `dtype`
 *   length                    (B,)           uint32
 *   new_starts                (B, T)         one byte per flag (0 / non-zero)
 * N (the head size) must be 64.
 */
#ifndef B200WKV_H_
#define B200WKV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define B200WKV_F32  0
#define B200WKV_BF16 1

/* status codes */
#define B200WKV_OK            0
#define B200WKV_EDTYPE       -1   /* dtype is not B200WKV_F32 / B200WKV_BF16            */
#define B200WKV_ESHAPE       -2   /* a dimension is < 1, N != 64, or a size overflows   */
#define B200WKV_ENULL        -3   /* a required pointer is NULL                          */
#define B200WKV_ERESIDUAL    -4   /* residual buffer smaller than *_residual_bytes()     */
#define B200WKV_ELAUNCH      -5   /* the CUDA runtime refused the launch                 */
#define B200WKV_EUNSUPPORTED -6   /* combination not available in this build             */
#define B200WKV_ESCRATCH     -7   /* problem larger than a fixed built-in scratch area   */
#define B200WKV_ESYMBOL      -8   /* the built-in scratch area could not be materialised  */

/* flags (bit set) */
#define B200WKV_FLAG_SEQUENTIAL 1u   /* force the token-sequential CUDA-core kernels     */

const char* b200wkv_strerror(int status);
/* ABI version of the loaded library (incremented on incompatible change). */
int b200wkv_abi_version(void);
/* Diagnostics: reads and clears the device-side error word of the current device (0 = none).
 * The tensor-core kernels bound every wait on an asynchronous product; a wait that runs out is
 * recorded there (1 = forward, 2 = backward) and the kernel still terminates.  This call
 * synchronises the device, so it is not for the hot path.  Returns -1 if the CUDA runtime fails. */
int b200wkv_device_status(void);

/* ---------------------------------------------------------------- RWKV-7 ----
 * Replaces the XLA custom calls "wkv7-fwd-{fp32,bf16}" / "wkv7-bwd-{fp32,bf16}"
 * that jaxrwkv binds at src/jaxrwkv/rwkv7.py:372-375 and :406-408 (handlers
 * WKV7FwdF32/WKV7FwdBF16/WKV7BwdF32/WKV7BwdBF16 registered at :461-465).
 * Operand order follows those calls: (w, r, k, v, a, b, s, length, new_starts).
 * `w` is the raw log-log decay: the kernel applies exp(-exp(w)) itself, as
 * BaseRWKV.inner_loop does at rwkv7.py:201.
 *
 * Semantics are those of BaseRWKV.inner_loop (rwkv7.py:199-220): a start flag
 * zeroes the state before its token, s_out is the state after token length-1
 * (the input state when length == 0; length > T is treated as T), and the
 * state is carried in fp32 inside the kernel.
 *
 * `residual` is an opaque device buffer the forward fills for the backward
 * (the counterpart of the reference's s_restore/sa_restore results,
 * rwkv7.py:363-364).  Pass NULL/0 for inference: nothing is saved then.  The
 * backward must be called with the same dtype and flags as the forward that
 * filled the buffer, and it uses the tail of the buffer as scratch (carries
 * passed between thread blocks), so the buffer must be writable and one
 * buffer must not serve two backward calls that overlap on the GPU.
 */
size_t b200wkv7_residual_bytes(int dtype, int B, int T, int H, int N);

int b200wkv7_fwd(void* stream, int dtype, int B, int T, int H, int N,
                 const void* w, const void* r, const void* k, const void* v,
                 const void* a, const void* b, const void* s0,
                 const uint32_t* length, const uint8_t* new_starts,
                 void* y, void* s_out,
                 void* residual, size_t residual_bytes, unsigned flags);

/* One decoding step (T == 1) that updates the state IN PLACE where the caller keeps it.  jaxrwkv
 * carries the state of a model as (layers, 2 + N, D) per sequence (default_state,
 * src/jaxrwkv/rwkv7.py:175-180): rows 2.. of a layer are the (H, N, N) block of this operator
 * (rwkv7.py:255, :260), so under a batch the blocks of one layer are `state_batch_stride` elements
 * apart.  `state` points at the block of batch row 0; streams are (B, 1, H, N), y likewise.  No copy
 * of the state is made on either side of the step.  `state` must be 32-byte aligned, the stride a
 * multiple of 32 bytes and the six streams 16-byte aligned (B200WKV_EUNSUPPORTED otherwise).  length == 0 leaves a row's state as it
 * is; a start flag zeroes it before the token (as b200wkv7_fwd). */
int b200wkv7_step_inplace(void* stream, int dtype, int B, int H, int N,
                          const void* w, const void* r, const void* k, const void* v,
                          const void* a, const void* b,
                          void* state, long long state_batch_stride,
                          const uint32_t* length, const uint8_t* new_starts, void* y);

/* Backward: cotangents dy (B,T,H,N) and ds_out (B,H,N,N) in, gradients of all six
 * streams and of the initial state out (the reference's result order is
 * gw, gr, gk, gv, ga, gb, gs — rwkv7.py:406).  dy or ds_out may be NULL (= zeros).
 * Unlike the reference kernels (README "CudaRWKV" caveats), gradients flow from
 * s_out and into s0, and start flags cut the dependency exactly. */
int b200wkv7_bwd(void* stream, int dtype, int B, int T, int H, int N,
                 const void* w, const void* r, const void* k, const void* v,
                 const void* a, const void* b, const void* s0,
                 const uint32_t* length, const uint8_t* new_starts,
                 const void* dy, const void* ds_out,
                 void* residual, size_t residual_bytes,
                 void* dw, void* dr, void* dk, void* dv, void* da, void* db, void* ds0,
                 unsigned flags);

/* ------------------------------------------------------- RWKV-5 / 5.2 / 6 ----
 * jaxrwkv has no CudaRWKV class for these versions; the entry points serve the
 * same operator seam, inner_loop(r, k, v, w, time_first, s, length, new_starts)
 * of src/jaxrwkv/rwkv6.py:174-191, rwkv5_2.py:164-180 and rwkv5.py:161-177.
 * The state is indexed [key][value].  `version` selects the decay operand:
 *   6 : w is (B, T, H, N) log-decay, the kernel applies exp(w)   (rwkv6.py:176)
 *   5 : w is (H, N) and already the decay, constant over time    (rwkv5_2.py:198; a
 *       per-head scalar decay of RWKV-5.0 is passed broadcast to (H, N))
 * u (time_first) is (H, N).  Backward results: dr, dk, dv, ds0 as the primals;
 * dw is (B, T, H, N) in `dtype` for version 6 (gradient of the log-decay) and
 * (B, H, N) fp32 per-batch partial sums for version 5; du is (B, H, N) fp32
 * per-batch partial sums (the caller adds over B, as jaxrwkv does for RWKV-4 at
 * rwkv4.py:351). */
size_t b200wkv6_residual_bytes(int dtype, int B, int T, int H, int N);

int b200wkv6_fwd(void* stream, int dtype, int version, int B, int T, int H, int N,
                 const void* r, const void* k, const void* v, const void* w, const void* u,
                 const void* s0, const uint32_t* length, const uint8_t* new_starts,
                 void* y, void* s_out, void* residual, size_t residual_bytes, unsigned flags);

int b200wkv6_bwd(void* stream, int dtype, int version, int B, int T, int H, int N,
                 const void* r, const void* k, const void* v, const void* w, const void* u,
                 const void* s0, const uint32_t* length, const uint8_t* new_starts,
                 const void* dy, const void* ds_out, void* residual, size_t residual_bytes,
                 void* dr, void* dk, void* dv, void* dw, void* du, void* ds0, unsigned flags);

/* ---------------------------------------------------------------- RWKV-4 ----
 * Replaces the XLA custom calls "wkv4-fwd-*" / "wkv4-bwd-*" bound at
 * src/jaxrwkv/rwkv4.py:320-321 and :347-349 (handlers WKV4FwdF32/BF16 and WKV4BwdF32/BF16, :396-400).
 * Operand order follows those calls.  k, v, y are (B, T, C); w (already -exp(.),
 * rwkv4.py:312) and u are (C,); states are (B, 3, C) = (aa, bb, pp); a start flag
 * resets to (0, 0, -1e30).  y comes without the receptance factor (rwkv4.py:406).
 * gw, gu are (B, C) fp32 per-batch partial sums (summed by the caller, rwkv4.py:351). */
size_t b200wkv4_residual_bytes(int dtype, int B, int T, int C);

int b200wkv4_fwd(void* stream, int dtype, int B, int T, int C,
                 const void* w, const void* u, const void* k, const void* v, const void* s0,
                 const uint32_t* length, const uint8_t* new_starts,
                 void* s_out, void* y, void* residual, size_t residual_bytes, unsigned flags);

int b200wkv4_bwd(void* stream, int dtype, int B, int T, int C,
                 const void* w, const void* u, const void* k, const void* v, const void* gy,
                 const void* s0, const uint32_t* length, const uint8_t* new_starts, const void* gs_new,
                 const void* residual, size_t residual_bytes,
                 void* gw, void* gu, void* gk, void* gv, void* gs, unsigned flags);

/* ------------------------------------------------------------ token shift ----
 * The per-token state the callers of the operator keep next to it: the shift by one token with
 * the carried last row and start flags (src/jaxrwkv/rwkv7.py:226-235, :254 for time mixing and
 * :192-197 for channel mixing), fused with the M interpolations x + (shifted - x) * mix_m.
 * x (B, T, D), prev (B, D), mix (M, D) with M <= 8, D a multiple of 4; out (M, B, T, D);
 * state_out (B, D) = x[(length - 1) mod T] (the reference indexes x[length-1], so length 0 wraps
 * to the last row).  Backward: gout (M, B, T, D) and gstate (B, D, may be NULL) in; gx, gprev as
 * the primals; gmix (B, ceil(T / B200WKV_SHIFT_TILE), M, D) fp32 partial sums, one per batch row
 * and tile of tokens (the caller adds over the first two axes: deterministic, no atomics). */
#define B200WKV_SHIFT_TILE 64
int b200wkv_token_shift_fwd(void* stream, int dtype, int B, int T, int D, int M,
                            const void* x, const void* prev, const void* mix,
                            const uint32_t* length, const uint8_t* new_starts,
                            void* out, void* state_out);

int b200wkv_token_shift_bwd(void* stream, int dtype, int B, int T, int D, int M,
                            const void* x, const void* prev, const void* mix,
                            const uint32_t* length, const uint8_t* new_starts,
                            const void* gout, const void* gstate,
                            void* gx, void* gprev, void* gmix);

/* ------------------------------------------- around the operator: time mixing ----
 * The elementwise work jaxrwkv's time mixing does on either side of the recurrence
 * (src/jaxrwkv/rwkv7.py:238-252 and :263-265), each side in one pass.  Streams are (rows, H*N) with
 * rows = B*T and N == 64 (H <= 128); per-channel parameters are (H*N,); all of one element type; every
 * pointer 16-byte aligned (B200WKV_EUNSUPPORTED otherwise).
 *
 * before the operator:   w   = -softplus(-(w0 + wl)) - 0.5          wl = output of the decay LoRA (:238)
 *                        a   = sigmoid(a0 + al)                     al = output of the a LoRA (:245)
 *                        v'  = v + (v_first - v) * sigmoid(v0 + vl) when use_vmix (layers > 0, :243), else v
 *                        kk  = (k * k_k) / max(||k * k_k||_head, 1e-12)   (:248-251)
 *                        k'  = k * (1 + (a - 1) * k_a)              (:252)
 *                        a_i = -kk,  b_i = kk * a                   (:257)
 *   outputs w, k_out = k', v_out = v', a_i, b_i are the operator's operands (with r unchanged).
 * after the operator:    x = (group_norm(y; H groups, eps) * ln_w + ln_b + (sum_n r k' r_k) * v') * g   (:263-265)
 *
 * The backward calls take the forward's inputs again (nothing is saved) and the cotangents of the
 * outputs; parameter gradients come back as fp32 partial sums, `partial` =
 * (b200wkv7_mix_partial_rows(rows, H, N), P, H*N) with P = 5 (dw0, da0, dv0, dk_k, dk_a) before and
 * P = 3 (d ln_w, d ln_b, d r_k) after the operator; the caller adds over the first axis (deterministic,
 * no atomics).  With use_vmix == 0, v_first / vl / v0 and their gradients may be NULL. */
int b200wkv7_mix_partial_rows(long long rows, int H, int N);
int b200wkv7_mix_pre_fwd(void* stream, int dtype, long long rows, int H, int N, int use_vmix,
                         const void* k, const void* wl, const void* al, const void* v,
                         const void* v_first, const void* vl,
                         const void* w0, const void* a0, const void* v0, const void* k_k, const void* k_a,
                         void* w, void* k_out, void* v_out, void* a_i, void* b_i);
int b200wkv7_mix_pre_bwd(void* stream, int dtype, long long rows, int H, int N, int use_vmix,
                         const void* k, const void* wl, const void* al, const void* v,
                         const void* v_first, const void* vl,
                         const void* w0, const void* a0, const void* v0, const void* k_k, const void* k_a,
                         const void* gw, const void* gk_out, const void* gv_out, const void* ga_i, const void* gb_i,
                         void* dk, void* dwl, void* dal, void* dv, void* dv_first, void* dvl, float* partial);
int b200wkv7_mix_post_fwd(void* stream, int dtype, long long rows, int H, int N, float eps,
                          const void* y, const void* r, const void* k, const void* v, const void* g,
                          const void* ln_w, const void* ln_b, const void* r_k, void* x);
int b200wkv7_mix_post_bwd(void* stream, int dtype, long long rows, int H, int N, float eps,
                          const void* y, const void* r, const void* k, const void* v, const void* g,
                          const void* ln_w, const void* ln_b, const void* r_k, const void* gx,
                          void* dy, void* dr, void* dk, void* dv, void* dg, float* partial);

/* Forward + backward in one call with NO residual buffer from the caller (no counterpart in
 * jaxrwkv: its kernels always take the residuals as operands).
 *
 * For hosts that cannot allocate device memory where they need the gradients - e.g. a
 * custom-call handler inside a compiled program whose layer body is rematerialised, so the
 * forward is re-run during the backward pass and the framework's memory pool, not the handler,
 * owns every device byte.  The state checkpoints live in a fixed array inside the library image
 * (b200wkv7_static_scratch_bytes() bytes, 64 MiB, held by every GPU that loads the library until
 * the process exits).  Problems whose b200wkv7_residual_bytes() exceeds that size are refused
 * with B200WKV_ESCRATCH and nothing is launched.  The call itself never calls cudaMalloc/cudaFree
 * or any allocating routine; the first call on each device resolves the array's device address
 * (make that first call before starting a stream capture on that device).  Because CUDA loads
 * modules lazily by default, that first call is also where the driver materialises the array on the
 * device: it can take device memory and synchronise, and it returns B200WKV_ESYMBOL if none is left -
 * so make it (or set CUDA_MODULE_LOADING=EAGER) before a framework's memory pool claims the device.
 * Every argument is checked before anything is enqueued.  All calls on a device
 * share the one array and it keeps the previous call's contents (nothing in it needs clearing: the
 * forward rewrites every slot the backward reads), so two calls must not overlap on the GPU -
 * issue them on one stream or order them with events.
 * Results equal b200wkv7_fwd followed by b200wkv7_bwd with the same dtype and flags. */
size_t b200wkv7_static_scratch_bytes(void);

int b200wkv7_fwd_bwd_static(void* stream, int dtype, int B, int T, int H, int N,
                            const void* w, const void* r, const void* k, const void* v,
                            const void* a, const void* b, const void* s0,
                            const uint32_t* length, const uint8_t* new_starts,
                            const void* dy, const void* ds_out,
                            void* y, void* s_out,
                            void* dw, void* dr, void* dk, void* dv, void* da, void* db, void* ds0,
                            unsigned flags);

#ifdef __cplusplus
}
#endif
#endif  /* B200WKV_H_ */

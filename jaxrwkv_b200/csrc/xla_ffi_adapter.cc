// XLA FFI handlers over the C ABI of include/b200wkv.h: what jax.ffi.register_ffi_target binds.
//
// jaxrwkv registers the handler symbols WKV7FwdF32 / WKV7FwdBF16 / WKV7BwdF32 / WKV7BwdBF16
// (src/jaxrwkv/rwkv7.py:461-465) and WKV4FwdF32 / WKV4FwdBF16 / WKV4BwdF32 / WKV4BwdBF16
// (src/jaxrwkv/rwkv4.py:396-400) from a ctypes-loaded library.  This translation unit exports the
// same symbols (operand order of rwkv7.py:372-375, :406-408 and rwkv4.py:320-321, :347-349), plus
// handlers for what the reference has no kernel for: the forward without a residual (inference),
// RWKV-5/5.2/6, the in-place decoding step and the token shift.
//
// A handler only validates, translates buffers into pointers and enqueues on the stream XLA hands it:
// no allocation, no synchronisation, nothing retained; a failure is returned as an ffi::Error.
//
// Built into lib/libb200wkv_xla.so by jaxrwkv_b200/build.py when the XLA FFI headers can be found
// (python -c "import jax.ffi; print(jax.ffi.include_dir())"); it links against libb200wkv.so.
#include <cstdint>
#include <string>
#include <utility>

#include <cuda_runtime_api.h>

#include "xla/ffi/api/ffi.h"

#include "../../include/b200wkv.h"

namespace ffi = xla::ffi;

namespace {

using Buf = ffi::AnyBuffer;
using Res = ffi::Result<ffi::AnyBuffer>;

ffi::Error status_to_error(int st, const char* where) {
    if (st == B200WKV_OK) return ffi::Error::Success();
    return ffi::Error::InvalidArgument(std::string(where) + ": " + b200wkv_strerror(st));
}

// every tensor operand of a call must have the element type its target name promises
template <int CODE>
bool has_dtype(const Buf& b) {
    return b.element_type() == (CODE == B200WKV_F32 ? ffi::DataType::F32 : ffi::DataType::BF16);
}
template <int CODE, typename... Bs>
bool all_dtype(const Bs&... bs) { return (has_dtype<CODE>(bs) && ...); }

const uint32_t* as_u32(const Buf& b) { return static_cast<const uint32_t*>(b.untyped_data()); }
const uint8_t* as_u8(const Buf& b) { return static_cast<const uint8_t*>(b.untyped_data()); }
int head_size(const Buf& k) { return k.dimensions().size() ? (int)k.dimensions().back() : 0; }

// --------------------------------------------------------------------------------------- RWKV-7
// "wkv7-fwd-*": (w, r, k, v, a, b, s, length, new_starts) -> (out, residual, new_s); attrs B, T, H.
// `residual` (uint8[b200wkv7_residual_bytes]) stands where the reference returns s_restore and
// sa_restore (rwkv7.py:362-365).
template <int CODE>
ffi::Error Wkv7Fwd(cudaStream_t stream, Buf w, Buf r, Buf k, Buf v, Buf a, Buf b, Buf s, Buf length, Buf new_starts,
                   Res out, Res residual, Res new_s, uint64_t B, uint64_t T, uint64_t H) {
    if (!all_dtype<CODE>(w, r, k, v, a, b, s)) return ffi::Error::InvalidArgument("wkv7-fwd: operand element type does not match the target");
    return status_to_error(
        b200wkv7_fwd(stream, CODE, (int)B, (int)T, (int)H, head_size(k), w.untyped_data(), r.untyped_data(), k.untyped_data(),
                     v.untyped_data(), a.untyped_data(), b.untyped_data(), s.untyped_data(), as_u32(length), as_u8(new_starts),
                     out->untyped_data(), new_s->untyped_data(), residual->untyped_data(), residual->size_bytes(), 0u),
        "wkv7-fwd");
}

// "wkv7-infer-*": the same call when no gradient will be asked for: (..) -> (out, new_s), nothing saved.
template <int CODE>
ffi::Error Wkv7Infer(cudaStream_t stream, Buf w, Buf r, Buf k, Buf v, Buf a, Buf b, Buf s, Buf length, Buf new_starts,
                     Res out, Res new_s, uint64_t B, uint64_t T, uint64_t H) {
    if (!all_dtype<CODE>(w, r, k, v, a, b, s)) return ffi::Error::InvalidArgument("wkv7-infer: operand element type does not match the target");
    return status_to_error(
        b200wkv7_fwd(stream, CODE, (int)B, (int)T, (int)H, head_size(k), w.untyped_data(), r.untyped_data(), k.untyped_data(),
                     v.untyped_data(), a.untyped_data(), b.untyped_data(), s.untyped_data(), as_u32(length), as_u8(new_starts),
                     out->untyped_data(), new_s->untyped_data(), nullptr, 0, 0u),
        "wkv7-infer");
}

// "wkv7-bwd-*": (w, r, k, v, a, b, s, length, new_starts, gy, residual, gs_out) -> (gw, gr, gk, gv, ga, gb, gs,
// residual'); attrs B, T, H.  The backward uses part of the residual as scratch, so the caller aliases operand 10
// to result 7 (input_output_aliases={10: 7}): XLA then passes a buffer the handler may write, and both names
// refer to the same memory.
template <int CODE>
ffi::Error Wkv7Bwd(cudaStream_t stream, Buf w, Buf r, Buf k, Buf v, Buf a, Buf b, Buf s, Buf length, Buf new_starts,
                   Buf gy, Buf residual, Buf gs_out, Res gw, Res gr, Res gk, Res gv, Res ga, Res gb, Res gs,
                   Res residual_out, uint64_t B, uint64_t T, uint64_t H) {
    if (!all_dtype<CODE>(w, r, k, v, a, b, s, gy, gs_out)) return ffi::Error::InvalidArgument("wkv7-bwd: operand element type does not match the target");
    if (residual_out->untyped_data() != residual.untyped_data())
        return ffi::Error::InvalidArgument("wkv7-bwd: the residual operand must be aliased to the last result (input_output_aliases={10: 7})");
    return status_to_error(
        b200wkv7_bwd(stream, CODE, (int)B, (int)T, (int)H, head_size(k), w.untyped_data(), r.untyped_data(), k.untyped_data(),
                     v.untyped_data(), a.untyped_data(), b.untyped_data(), s.untyped_data(), as_u32(length), as_u8(new_starts),
                     gy.untyped_data(), gs_out.untyped_data(), residual_out->untyped_data(), residual_out->size_bytes(),
                     gw->untyped_data(), gr->untyped_data(), gk->untyped_data(), gv->untyped_data(), ga->untyped_data(),
                     gb->untyped_data(), gs->untyped_data(), 0u),
        "wkv7-bwd");
}

// "wkv7-step-*": one decoding token on the packed state container (B, L, 2+N, D) of default_state
// (rwkv7.py:175-180), updated where it lies: (w, r, k, v, a, b, state, length, new_starts) -> (out, state');
// attrs B, H, L, layer; the caller aliases operand 6 to result 1.
template <int CODE>
ffi::Error Wkv7Step(cudaStream_t stream, Buf w, Buf r, Buf k, Buf v, Buf a, Buf b, Buf state, Buf length, Buf new_starts,
                    Res out, Res state_out, uint64_t B, uint64_t H, uint64_t L, uint64_t layer) {
    if (!all_dtype<CODE>(w, r, k, v, a, b, state)) return ffi::Error::InvalidArgument("wkv7-step: operand element type does not match the target");
    if (state_out->untyped_data() != state.untyped_data())
        return ffi::Error::InvalidArgument("wkv7-step: the state operand must be aliased to the second result (input_output_aliases={6: 1})");
    if (layer >= L) return ffi::Error::InvalidArgument("wkv7-step: layer out of range");
    const int N = head_size(k);
    const long long D = (long long)H * N, rows = 2 + N, esz = CODE == B200WKV_F32 ? 4 : 2;
    char* block = static_cast<char*>(state_out->untyped_data()) + ((long long)layer * rows * D + 2 * D) * esz;
    return status_to_error(
        b200wkv7_step_inplace(stream, CODE, (int)B, (int)H, N, w.untyped_data(), r.untyped_data(), k.untyped_data(), v.untyped_data(),
                              a.untyped_data(), b.untyped_data(), block, (long long)L * rows * D, as_u32(length), as_u8(new_starts),
                              out->untyped_data()),
        "wkv7-step");
}

// --------------------------------------------------------------------------------------- RWKV-4
// "wkv4-fwd-*": (w, u, k, v, s, length, new_starts) -> (new_s, out, residual); attrs B, T, C  (rwkv4.py:320-321)
template <int CODE>
ffi::Error Wkv4Fwd(cudaStream_t stream, Buf w, Buf u, Buf k, Buf v, Buf s, Buf length, Buf new_starts, Res new_s, Res out,
                   Res residual, uint64_t B, uint64_t T, uint64_t C) {
    if (!all_dtype<CODE>(w, u, k, v, s)) return ffi::Error::InvalidArgument("wkv4-fwd: operand element type does not match the target");
    return status_to_error(
        b200wkv4_fwd(stream, CODE, (int)B, (int)T, (int)C, w.untyped_data(), u.untyped_data(), k.untyped_data(), v.untyped_data(),
                     s.untyped_data(), as_u32(length), as_u8(new_starts), new_s->untyped_data(), out->untyped_data(),
                     residual->untyped_data(), residual->size_bytes(), 0u),
        "wkv4-fwd");
}
// "wkv4-bwd-*": (w, u, k, v, gy, s, length, new_starts, gs_new, residual) -> (gw, gu, gk, gv, gs); attrs B, T, C
// (rwkv4.py:347-349).  gw and gu are (B, C) fp32 partial sums, added over B by the caller (rwkv4.py:351).
template <int CODE>
ffi::Error Wkv4Bwd(cudaStream_t stream, Buf w, Buf u, Buf k, Buf v, Buf gy, Buf s, Buf length, Buf new_starts, Buf gs_new,
                   Buf residual, Res gw, Res gu, Res gk, Res gv, Res gs, uint64_t B, uint64_t T, uint64_t C) {
    if (!all_dtype<CODE>(w, u, k, v, gy, s, gs_new)) return ffi::Error::InvalidArgument("wkv4-bwd: operand element type does not match the target");
    return status_to_error(
        b200wkv4_bwd(stream, CODE, (int)B, (int)T, (int)C, w.untyped_data(), u.untyped_data(), k.untyped_data(), v.untyped_data(),
                     gy.untyped_data(), s.untyped_data(), as_u32(length), as_u8(new_starts), gs_new.untyped_data(),
                     residual.untyped_data(), residual.size_bytes(), gw->untyped_data(), gu->untyped_data(), gk->untyped_data(),
                     gv->untyped_data(), gs->untyped_data(), 0u),
        "wkv4-bwd");
}

// ------------------------------------------------------------------------------- RWKV-5 / 5.2 / 6
// "wkv6-fwd-*": (r, k, v, w, u, s, length, new_starts) -> (out, residual, new_s); attrs B, T, H, version (5 or 6)
template <int CODE>
ffi::Error Wkv6Fwd(cudaStream_t stream, Buf r, Buf k, Buf v, Buf w, Buf u, Buf s, Buf length, Buf new_starts, Res out,
                   Res residual, Res new_s, uint64_t B, uint64_t T, uint64_t H, uint64_t version) {
    if (!all_dtype<CODE>(r, k, v, w, u, s)) return ffi::Error::InvalidArgument("wkv6-fwd: operand element type does not match the target");
    return status_to_error(
        b200wkv6_fwd(stream, CODE, (int)version, (int)B, (int)T, (int)H, head_size(k), r.untyped_data(), k.untyped_data(),
                     v.untyped_data(), w.untyped_data(), u.untyped_data(), s.untyped_data(), as_u32(length), as_u8(new_starts),
                     out->untyped_data(), new_s->untyped_data(), residual->untyped_data(), residual->size_bytes(), 0u),
        "wkv6-fwd");
}
// "wkv6-bwd-*": (r, k, v, w, u, s, length, new_starts, gy, residual, gs_out) -> (gr, gk, gv, gw, gu, gs, residual)
// The backward writes into the residual (state gradients at the ends of the runs it walks in parallel), so operand 9
// is donated to a seventh result: input_output_aliases={9: 6}.
template <int CODE>
ffi::Error Wkv6Bwd(cudaStream_t stream, Buf r, Buf k, Buf v, Buf w, Buf u, Buf s, Buf length, Buf new_starts, Buf gy,
                   Buf residual, Buf gs_out, Res gr, Res gk, Res gv, Res gw, Res gu, Res gs, Res residual_out, uint64_t B,
                   uint64_t T, uint64_t H, uint64_t version) {
    if (!all_dtype<CODE>(r, k, v, w, u, s, gy, gs_out)) return ffi::Error::InvalidArgument("wkv6-bwd: operand element type does not match the target");
    if (residual_out->untyped_data() != residual.untyped_data())
        return ffi::Error::InvalidArgument("wkv6-bwd: the residual operand must be aliased to the last result (input_output_aliases={9: 6})");
    return status_to_error(
        b200wkv6_bwd(stream, CODE, (int)version, (int)B, (int)T, (int)H, head_size(k), r.untyped_data(), k.untyped_data(),
                     v.untyped_data(), w.untyped_data(), u.untyped_data(), s.untyped_data(), as_u32(length), as_u8(new_starts),
                     gy.untyped_data(), gs_out.untyped_data(), residual_out->untyped_data(), residual_out->size_bytes(),
                     gr->untyped_data(), gk->untyped_data(), gv->untyped_data(), gw->untyped_data(), gu->untyped_data(),
                     gs->untyped_data(), 0u),
        "wkv6-bwd");
}

// ----------------------------------------------------------------------------------- token shift
// "token-shift-fwd-*": (x, prev, mix, length, new_starts) -> (mixed (M,B,T,D), new_prev (B,D)); attrs B, T, D, M
template <int CODE>
ffi::Error ShiftFwd(cudaStream_t stream, Buf x, Buf prev, Buf mix, Buf length, Buf new_starts, Res out, Res state_out,
                    uint64_t B, uint64_t T, uint64_t D, uint64_t M) {
    if (!all_dtype<CODE>(x, prev, mix)) return ffi::Error::InvalidArgument("token-shift-fwd: operand element type does not match the target");
    return status_to_error(
        b200wkv_token_shift_fwd(stream, CODE, (int)B, (int)T, (int)D, (int)M, x.untyped_data(), prev.untyped_data(), mix.untyped_data(),
                                as_u32(length), as_u8(new_starts), out->untyped_data(), state_out->untyped_data()),
        "token-shift-fwd");
}
// "token-shift-bwd-*": (x, prev, mix, length, new_starts, gout, gstate) -> (gx, gprev, gmix partial sums)
template <int CODE>
ffi::Error ShiftBwd(cudaStream_t stream, Buf x, Buf prev, Buf mix, Buf length, Buf new_starts, Buf gout, Buf gstate, Res gx,
                    Res gprev, Res gmix, uint64_t B, uint64_t T, uint64_t D, uint64_t M) {
    if (!all_dtype<CODE>(x, prev, mix, gout, gstate)) return ffi::Error::InvalidArgument("token-shift-bwd: operand element type does not match the target");
    return status_to_error(
        b200wkv_token_shift_bwd(stream, CODE, (int)B, (int)T, (int)D, (int)M, x.untyped_data(), prev.untyped_data(), mix.untyped_data(),
                                as_u32(length), as_u8(new_starts), gout.untyped_data(), gstate.untyped_data(), gx->untyped_data(),
                                gprev->untyped_data(), gmix->untyped_data()),
        "token-shift-bwd");
}

// NARGS operands and NRETS results of any element type (the named uint64 attributes follow at the use).
// The builder methods of an XLA FFI binding consume the binding they are called on, hence the moves.
template <int N, typename Binding>
auto add_args(Binding b) {
    if constexpr (N == 0) return b;
    else return add_args<N - 1>(std::move(b).template Arg<Buf>());
}
template <int N, typename Binding>
auto add_rets(Binding b) {
    if constexpr (N == 0) return b;
    else return add_rets<N - 1>(std::move(b).template Ret<Buf>());
}
template <int NARGS, int NRETS>
auto bind_buffers() {
    return add_rets<NRETS>(add_args<NARGS>(ffi::Ffi::Bind().Ctx<ffi::PlatformStream<cudaStream_t>>()));
}

}  // namespace

#define B200WKV_BTH .Attr<uint64_t>("B").Attr<uint64_t>("T").Attr<uint64_t>("H")
#define B200WKV_BTC .Attr<uint64_t>("B").Attr<uint64_t>("T").Attr<uint64_t>("C")
#define B200WKV_BTHV B200WKV_BTH.Attr<uint64_t>("version")
#define B200WKV_BTDM .Attr<uint64_t>("B").Attr<uint64_t>("T").Attr<uint64_t>("D").Attr<uint64_t>("M")
#define B200WKV_STEP .Attr<uint64_t>("B").Attr<uint64_t>("H").Attr<uint64_t>("L").Attr<uint64_t>("layer")

// the symbols jaxrwkv registers (rwkv7.py:461-465, rwkv4.py:396-400)
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7FwdF32, Wkv7Fwd<B200WKV_F32>, (bind_buffers<9, 3>() B200WKV_BTH));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7FwdBF16, Wkv7Fwd<B200WKV_BF16>, (bind_buffers<9, 3>() B200WKV_BTH));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7BwdF32, Wkv7Bwd<B200WKV_F32>, (bind_buffers<12, 8>() B200WKV_BTH));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7BwdBF16, Wkv7Bwd<B200WKV_BF16>, (bind_buffers<12, 8>() B200WKV_BTH));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV4FwdF32, Wkv4Fwd<B200WKV_F32>, (bind_buffers<7, 3>() B200WKV_BTC));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV4FwdBF16, Wkv4Fwd<B200WKV_BF16>, (bind_buffers<7, 3>() B200WKV_BTC));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV4BwdF32, Wkv4Bwd<B200WKV_F32>, (bind_buffers<10, 5>() B200WKV_BTC));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV4BwdBF16, Wkv4Bwd<B200WKV_BF16>, (bind_buffers<10, 5>() B200WKV_BTC));
// additions without a counterpart in jaxrwkv
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7InferF32, Wkv7Infer<B200WKV_F32>, (bind_buffers<9, 2>() B200WKV_BTH));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7InferBF16, Wkv7Infer<B200WKV_BF16>, (bind_buffers<9, 2>() B200WKV_BTH));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7StepF32, Wkv7Step<B200WKV_F32>, (bind_buffers<9, 2>() B200WKV_STEP));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV7StepBF16, Wkv7Step<B200WKV_BF16>, (bind_buffers<9, 2>() B200WKV_STEP));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV6FwdF32, Wkv6Fwd<B200WKV_F32>, (bind_buffers<8, 3>() B200WKV_BTHV));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV6FwdBF16, Wkv6Fwd<B200WKV_BF16>, (bind_buffers<8, 3>() B200WKV_BTHV));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV6BwdF32, Wkv6Bwd<B200WKV_F32>, (bind_buffers<11, 7>() B200WKV_BTHV));
XLA_FFI_DEFINE_HANDLER_SYMBOL(WKV6BwdBF16, Wkv6Bwd<B200WKV_BF16>, (bind_buffers<11, 7>() B200WKV_BTHV));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TokenShiftFwdF32, ShiftFwd<B200WKV_F32>, (bind_buffers<5, 2>() B200WKV_BTDM));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TokenShiftFwdBF16, ShiftFwd<B200WKV_BF16>, (bind_buffers<5, 2>() B200WKV_BTDM));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TokenShiftBwdF32, ShiftBwd<B200WKV_F32>, (bind_buffers<7, 3>() B200WKV_BTDM));
XLA_FFI_DEFINE_HANDLER_SYMBOL(TokenShiftBwdBF16, ShiftBwd<B200WKV_BF16>, (bind_buffers<7, 3>() B200WKV_BTDM));

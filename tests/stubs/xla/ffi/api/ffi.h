// Stand-in for the XLA FFI header (xla/ffi/api/ffi.h), for TESTS ONLY: the real header ships with
// jaxlib and is not available where the CPU test-suite runs.  It declares the small part of the API
// surface that csrc/xla_ffi_adapter.cc uses, with the same spelling, and its binding builder checks
// that every handler can be invoked with the argument list its binding describes (stream, then one
// AnyBuffer per operand, one Result<AnyBuffer> per result, one value per attribute).  It executes
// nothing; it only lets `g++ -fsyntax-only` type-check the adapter.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <type_traits>
#include <utility>
#include <vector>

namespace xla {
namespace ffi {

enum class DataType { PRED, U8, U32, F32, BF16 };

class Error {
public:
    static Error Success() { return Error(); }
    static Error InvalidArgument(std::string) { return Error(); }
    static Error Internal(std::string) { return Error(); }
};

template <typename T>
class Span {
public:
    size_t size() const { return v_.size(); }
    const T& back() const { return v_.back(); }
private:
    std::vector<T> v_;
};

class AnyBuffer {
public:
    void* untyped_data() const { return nullptr; }
    size_t size_bytes() const { return 0; }
    DataType element_type() const { return DataType::F32; }
    Span<int64_t> dimensions() const { return {}; }
};

template <typename T>
class Result {
public:
    T* operator->() { return &t_; }
private:
    T t_;
};

template <typename T>
struct PlatformStream {};

template <typename... Ts>
class Binding {
public:
    template <typename C> auto Ctx() && { return Binding<Ts..., typename CtxType<C>::type>(); }
    template <typename A> auto Arg() && { return Binding<Ts..., A>(); }
    template <typename R> auto Ret() && { return Binding<Ts..., Result<R>>(); }
    template <typename A> auto Attr(const char*) && { return Binding<Ts..., A>(); }
    template <typename F> int To(F&&) && {
        static_assert(std::is_invocable_r<Error, F, Ts...>::value, "handler signature does not match its binding");
        return 0;
    }
private:
    template <typename C> struct CtxType;
    template <typename S> struct CtxType<PlatformStream<S>> { using type = S; };
};

struct Ffi {
    static Binding<> Bind() { return Binding<>(); }
};

}  // namespace ffi
}  // namespace xla

#define XLA_FFI_DEFINE_HANDLER_SYMBOL(name, impl, binding) \
    extern "C" int name(void*) { static int h = (binding).To(impl); return h; }

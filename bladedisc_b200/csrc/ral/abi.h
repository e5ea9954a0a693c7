// Type-erased calling convention of RAL custom calls, re-expressed.
//
// A DISC-compiled executable calls every runtime function as
//   f(ctx, "name___device___T1_T2..___R", void** args)
// where args[i] points at the i-th flattened argument: scalars take one slot,
// a rank-N memref takes 3 + 2N slots (base pointer, aligned pointer, offset,
// N sizes, N strides) and the slot after the last argument points at storage
// for the result (one slot per element when the result is a tuple).  The
// convention is defined by tao_compiler/mlir/ral/ral_helper.h:46-60 (memref
// layout), :65-152 (name mangling) and :160-252 (unpacking); the producer side
// is tao_compiler/mlir/disc/transforms/disc_to_llvm.cc:73-167, 302-365.
//
// This header derives mangled name and unpacking thunk from an ordinary C++
// function signature.
#pragma once
#include <array>
#include <cstdint>
#include <string>
#include <tuple>
#include <type_traits>
#include <utility>

namespace disc_b200 {
namespace ral {

struct ExecContext;

struct f16_t {
  uint16_t bits;
};
struct bf16_t {
  uint16_t bits;
};

// Same object layout as an MLIR memref descriptor.
template <typename T, int N>
struct MemRef {
  T* base;
  T* data;
  int64_t offset;
  int64_t sizes[N];
  int64_t strides[N];
};
template <typename T>
struct MemRef<T, 0> {
  T* base;
  T* data;
  int64_t offset;
};

template <typename T, int N>
inline int64_t memref_numel(const MemRef<T, N>& m) {
  int64_t n = 1;
  if constexpr (N > 0) {
    for (int i = 0; i < N; ++i) n *= m.sizes[i];
  }
  return n;
}

// Dense row-major descriptor over `data` with the given sizes.
template <typename T, int N>
inline MemRef<T, N> make_memref(T* data, const int64_t* sizes) {
  MemRef<T, N> m;
  m.base = data;
  m.data = data;
  m.offset = 0;
  if constexpr (N > 0) {
    int64_t stride = 1;
    for (int i = N - 1; i >= 0; --i) {
      m.sizes[i] = sizes[i];
      m.strides[i] = stride;
      stride *= sizes[i];
    }
  }
  return m;
}

// ------------------------------------------------------------ type names
template <typename T, typename = void>
struct TypeTag;
#define DISC_B200_TYPE_TAG(T, S)                   \
  template <>                                      \
  struct TypeTag<T, void> {                        \
    static std::string str() { return S; }         \
  };
DISC_B200_TYPE_TAG(bool, "i1")
DISC_B200_TYPE_TAG(uint8_t, "ui8")
DISC_B200_TYPE_TAG(int8_t, "i8")
DISC_B200_TYPE_TAG(uint16_t, "ui16")
DISC_B200_TYPE_TAG(int16_t, "i16")
DISC_B200_TYPE_TAG(bf16_t, "bf16")
DISC_B200_TYPE_TAG(f16_t, "f16")
DISC_B200_TYPE_TAG(uint32_t, "ui32")
DISC_B200_TYPE_TAG(int32_t, "i32")
DISC_B200_TYPE_TAG(int64_t, "i64")
DISC_B200_TYPE_TAG(uint64_t, "i64")
DISC_B200_TYPE_TAG(float, "f32")
DISC_B200_TYPE_TAG(double, "f64")
DISC_B200_TYPE_TAG(void, "void")
DISC_B200_TYPE_TAG(void**, "ppvoid")
#undef DISC_B200_TYPE_TAG
// Every other pointer (context, stream handle, strings, attribute blobs) is "pvoid".
template <typename T>
struct TypeTag<T*, std::enable_if_t<!std::is_same_v<T*, void**>>> {
  static std::string str() { return "pvoid"; }
};
template <typename T, int N>
struct TypeTag<MemRef<T, N>, void> {
  static std::string str() { return "m" + std::to_string(N) + "d" + TypeTag<T>::str(); }
};
template <typename... Ts>
struct TypeTag<std::tuple<Ts...>, void> {
  static std::string str() {
    std::string s;
    bool first = true;
    ((s += (first ? "" : "_") + TypeTag<Ts>::str(), first = false), ...);
    return s;
  }
};

template <typename R, typename... A>
std::string mangle(const std::string& api, const std::string& device, R (*)(A...)) {
  std::string args;
  bool first = true;
  ((args += (first ? "" : "_") + TypeTag<std::decay_t<A>>::str(), first = false), ...);
  return api + "___" + device + "___" + args + "___" + TypeTag<R>::str();
}

// --------------------------------------------------------------- unpacking
template <typename T>
struct Slots {
  static constexpr int n = 1;
  static T read(void** a) { return *static_cast<T*>(a[0]); }
};
template <typename T, int N>
struct Slots<MemRef<T, N>> {
  static constexpr int n = 3 + 2 * N;
  static MemRef<T, N> read(void** a) {
    MemRef<T, N> m;
    m.base = *static_cast<T**>(a[0]);
    m.data = *static_cast<T**>(a[1]);
    m.offset = *static_cast<int64_t*>(a[2]);
    if constexpr (N > 0) {
      for (int i = 0; i < N; ++i) m.sizes[i] = *static_cast<int64_t*>(a[3 + i]);
      for (int i = 0; i < N; ++i) m.strides[i] = *static_cast<int64_t*>(a[3 + N + i]);
    }
    return m;
  }
};

template <typename... A>
constexpr std::array<int, sizeof...(A) + 1> slot_offsets() {
  std::array<int, sizeof...(A) + 1> off{};
  const int n[] = {Slots<std::decay_t<A>>::n..., 0};
  int acc = 0;
  for (size_t i = 0; i < sizeof...(A); ++i) {
    off[i] = acc;
    acc += n[i];
  }
  off[sizeof...(A)] = acc;
  return off;
}

template <typename R>
struct ResultSlot {
  static void write(void** a, R&& r) { *static_cast<R*>(a[0]) = std::move(r); }
};
template <typename... Rs>
struct ResultSlot<std::tuple<Rs...>> {
  static void write(void** a, std::tuple<Rs...>&& r) { put(a, r, std::index_sequence_for<Rs...>{}); }
  template <size_t... I>
  static void put(void** a, std::tuple<Rs...>& r, std::index_sequence<I...>) {
    ((*static_cast<Rs*>(a[I]) = std::get<I>(r)), ...);
  }
};

using ApiFn = void (*)(void** args);

template <auto Fn>
struct Thunk;
template <typename R, typename... A, R (*Fn)(A...)>
struct Thunk<Fn> {
  static void call(void** args) { run(args, std::index_sequence_for<A...>{}); }
  template <size_t... I>
  static void run(void** args, std::index_sequence<I...>) {
    constexpr auto off = slot_offsets<A...>();
    if constexpr (std::is_void_v<R>) {
      Fn(Slots<std::decay_t<A>>::read(args + off[I])...);
    } else {
      ResultSlot<R>::write(args + off[sizeof...(A)], Fn(Slots<std::decay_t<A>>::read(args + off[I])...));
    }
  }
};

// Registry of custom calls: full mangled name -> thunk.  As in the reference
// (tao_compiler/mlir/ral/ral_helper.cc:43-51) the bare api name is also
// registered as a nickname and the first registration keeps it.
bool registry_add(const std::string& mangled, const std::string& nickname, ApiFn fn);
ApiFn registry_find(const std::string& name);
int registry_size();
const char* registry_name_at(int i);

template <auto Fn>
struct Registrar {
  Registrar(const char* api, const char* device) {
    registry_add(mangle(api, device, Fn), api, &Thunk<Fn>::call);
  }
};

#define DISC_B200_CAT2(a, b) a##b
#define DISC_B200_CAT(a, b) DISC_B200_CAT2(a, b)
#define DISC_B200_RAL_API(api, device, ...) \
  static ::disc_b200::ral::Registrar<&__VA_ARGS__> DISC_B200_CAT(disc_b200_reg_, __COUNTER__)(api, device)

}  // namespace ral
}  // namespace disc_b200

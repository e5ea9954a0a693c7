// Reshapes / aliases ("inc_ref") and typed memref copies ("h2d", "d2h", "d2d") of
// generated code.  Host code only.
//
// A memref descriptor has the same layout for every element type, and neither a
// reshape nor an alias looks at the elements, so one function per (rank in, rank
// out) serves every type: it is registered under each type's mangled name.  The
// copies need the element size only: one function per (size, rank).
#include <cuda_runtime.h>

#include <cstring>
#include <string>
#include <utility>

#include "abi.h"
#include "context.h"

namespace disc_b200 {
namespace ral {
namespace {

cudaStream_t stream_of(ExecContext* ctx) { return ctx->ctx->stream; }

bool check_stream_handle(ExecContext* ctx, void* handle) {
  if (reinterpret_cast<intptr_t>(handle) != 0) {
    ctx->signal_error("not a valid stream idx");
    return false;
  }
  return true;
}

// "inc_ref": the result describes the same buffer (with the shape operand's sizes and
// dense strides, when one is given) and the buffer's owner count goes up, so that a
// later dealloc of either name keeps it alive for the other
// (tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc:517-625,
// base/cpu/cpu_context_impl.cc:234-330).  Buffers this execution does not own --
// inputs, constants, persistent buffers -- are never freed by dealloc here, so nothing
// has to be counted for them; a pointer that is none of these is an error.
template <bool kHost>
bool retain(ExecContext* ctx, void* p) {
  if (!p) return true;
  auto& counts = kHost ? ctx->host_refcount : ctx->refcount;
  auto it = counts.find(p);
  if (it != counts.end()) {
    ++it->second;
    return true;
  }
  if (ctx->input_ptrs.count(p)) return true;
  std::shared_ptr<ConstStore> consts;
  {
    std::lock_guard<std::mutex> l(ctx->ctx->mu);
    if ((kHost ? ctx->ctx->host_persistent : ctx->ctx->persistent).count(p)) return true;
    consts = ctx->ctx->consts;
  }
  if (consts) {
    std::lock_guard<std::mutex> l(consts->mu);
    for (const auto& kv : (kHost ? consts->host_consts : consts->device_consts)) {
      if (kv.second.ptr == p) return true;
    }
  }
  ctx->signal_error("inc_ref: buffer is neither an input, a constant nor owned by this execution");
  return false;
}

using Byte = uint8_t;  // stands for any element type

template <int N, bool kHost>
MemRef<Byte, N> ral_alias(ExecContext* ctx, void* stream_handle, MemRef<Byte, N> input) {
  retain<kHost>(ctx, input.data);
  return input;
}

template <int N, int M, bool kHost>
MemRef<Byte, M> ral_reshape(ExecContext* ctx, void* stream_handle, MemRef<Byte, N> input,
                            MemRef<int64_t, 1> shape) {
  MemRef<Byte, M> m;
  std::memset(&m, 0, sizeof(m));
  if constexpr (M > 0) {
    if (!shape.data || shape.sizes[0] < M) {
      ctx->signal_error("inc_ref: shape operand shorter than the result rank");
      return m;
    }
    m = make_memref<Byte, M>(input.data, shape.data);  // the shape operand lives in host memory
  }
  m.base = input.base;
  m.data = input.data;
  m.offset = 0;
  retain<kHost>(ctx, input.data);
  return m;
}

// "h2d" / "d2h" / "d2d": copies between two dense memrefs of one shape, on the context's
// stream (tao_compiler/mlir/ral/context/common_context_impl_cuda.cc:380-460).
template <typename U, int N, cudaMemcpyKind kKind>
void ral_copy_memref(ExecContext* ctx, void* stream_handle, MemRef<U, N> from, MemRef<U, N> to) {
  if (!check_stream_handle(ctx, stream_handle)) return;
  const int64_t n = memref_numel(from);
  if (n != memref_numel(to)) {
    ctx->signal_error("memref copy: operand sizes differ");
    return;
  }
  if (n == 0) return;
  const cudaError_t st = cudaMemcpyAsync(to.data, from.data, static_cast<size_t>(n) * sizeof(U), kKind, stream_of(ctx));
  if (st != cudaSuccess) ctx->signal_error(std::string("memref copy: ") + cudaGetErrorString(st));
}

// element types: the reference's (cuda_context_impl.cc:686-760, common_context_impl_cuda.cc:460-520)
// and the 8-bit ones of the quantized path
struct ElemTag {
  const char* tag;
  int bytes;
};
constexpr ElemTag kElems[] = {{"f32", 4}, {"f64", 8}, {"f16", 2}, {"bf16", 2}, {"i8", 1},
                              {"ui8", 1}, {"i32", 4}, {"i64", 8}, {"i1", 1}};

std::string memref_tag(int rank, const char* elem) { return "m" + std::to_string(rank) + "d" + elem; }

template <int N, bool kHost, size_t... M>
void register_reshapes(std::index_sequence<M...>) {
  const std::string dev = kHost ? "cpu" : "gpu";
  for (const ElemTag& e : kElems) {
    (registry_add("inc_ref___" + dev + "___pvoid_pvoid_" + memref_tag(N, e.tag) + "_m1di64___" +
                      memref_tag(static_cast<int>(M), e.tag),
                  "inc_ref", &Thunk<&ral_reshape<N, static_cast<int>(M), kHost>>::call),
     ...);
  }
}
template <bool kHost, size_t... N>
void register_views(std::index_sequence<N...>) {
  const std::string dev = kHost ? "cpu" : "gpu";
  for (const ElemTag& e : kElems) {
    (registry_add("inc_ref___" + dev + "___pvoid_pvoid_" + memref_tag(static_cast<int>(N), e.tag) + "___" +
                      memref_tag(static_cast<int>(N), e.tag),
                  "inc_ref", &Thunk<&ral_alias<static_cast<int>(N), kHost>>::call),
     ...);
  }
  (register_reshapes<static_cast<int>(N), kHost>(std::make_index_sequence<9>{}), ...);
}

template <typename U, int N>
void register_copies_of(const char* tag) {
  const std::string args = "___gpu___pvoid_pvoid_" + memref_tag(N, tag) + "_" + memref_tag(N, tag) + "___void";
  registry_add("h2d" + args, "h2d", &Thunk<&ral_copy_memref<U, N, cudaMemcpyHostToDevice>>::call);
  registry_add("d2h" + args, "d2h", &Thunk<&ral_copy_memref<U, N, cudaMemcpyDeviceToHost>>::call);
  registry_add("d2d" + args, "d2d", &Thunk<&ral_copy_memref<U, N, cudaMemcpyDeviceToDevice>>::call);
}
template <size_t... N>
void register_copies(std::index_sequence<N...>) {
  for (const ElemTag& e : kElems) {
    switch (e.bytes) {
      case 1: (register_copies_of<uint8_t, static_cast<int>(N)>(e.tag), ...); break;
      case 2: (register_copies_of<uint16_t, static_cast<int>(N)>(e.tag), ...); break;
      case 4: (register_copies_of<uint32_t, static_cast<int>(N)>(e.tag), ...); break;
      default: (register_copies_of<uint64_t, static_cast<int>(N)>(e.tag), ...); break;
    }
  }
}

const bool g_registered = [] {
  register_views<false>(std::make_index_sequence<9>{});
  register_views<true>(std::make_index_sequence<9>{});
  register_copies(std::make_index_sequence<9>{});
  return true;
}();

}  // namespace
}  // namespace ral
}  // namespace disc_b200

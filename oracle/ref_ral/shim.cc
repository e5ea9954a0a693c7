// TEST INFRASTRUCTURE.  Linked together with the reference's own RAL core
// (ral_api.cc, ral_context.cc, ral_helper.cc, ral_logging.cc, ral_metadata.cc,
// compiled from the reference tree where it lies) into oracle/_ref/libref_ral.so.
//
// It registers recording stubs, with the reference's registration macro and
// the reference's C++ signatures, for the custom calls our library implements
// under reference names.  Tests then (1) compare the names the reference
// mangles with the names our registry holds and (2) send one packed argument
// array through the reference's tao_ral_call_impl and read back what its
// unpacking produced, which pins the packing our own tests use.  (3) The
// reference's metadata file emitter and loader are exported as they are, so
// that files written by either side can be read by the other.  (4) The reference's
// parser of custom_attrs blobs (context/pdll_util.cc) renders what it understood of a
// blob, so that the writer and the parser of this repository are checked against it.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "mlir/ral/ral_api.h"
#include "mlir/ral/ral_context.h"
#include "mlir/ral/ral_helper.h"
#include "mlir/ral/context/pdll_util.h"
#include "mlir/ral/ral_metadata.h"

using tao::ral::ExecutionContext;
using tao::ral::MemRefType;

namespace {

std::vector<int64_t> g_record;
std::vector<std::string> g_names;

void rec(int64_t v) { g_record.push_back(v); }
void rec_ptr(const void* p) { g_record.push_back(static_cast<int64_t>(reinterpret_cast<intptr_t>(p))); }
template <typename T, int N>
void rec_memref(const MemRefType<T, N>& m) {
  rec_ptr(m.basePtr);
  rec_ptr(m.data);
  rec(m.offset);
  for (int i = 0; i < N; ++i) rec(m.sizes[i]);
  for (int i = 0; i < N; ++i) rec(m.strides[i]);
}
template <typename T>
void rec_memref(const MemRefType<T, 0>& m) {
  rec_ptr(m.basePtr);
  rec_ptr(m.data);
  rec(m.offset);
}

template <int N, typename BiasT>
MemRefType<int8_t, N> stub_pdll_qgemm(ExecutionContext* ctx, void* stream, MemRefType<int8_t, N> input,
                                      MemRefType<int8_t, 2> weight, MemRefType<BiasT, 1> bias,
                                      MemRefType<float, 0> in_s, MemRefType<int32_t, 0> in_zp,
                                      MemRefType<float, 0> w_s, MemRefType<int32_t, 0> w_zp,
                                      MemRefType<float, 0> out_s, MemRefType<int32_t, 0> out_zp,
                                      void* attrs) {
  g_record.clear();
  rec_ptr(ctx);
  rec_ptr(stream);
  rec_memref(input);
  rec_memref(weight);
  rec_memref(bias);
  rec_memref(in_s);
  rec_memref(in_zp);
  rec_memref(w_s);
  rec_memref(w_zp);
  rec_memref(out_s);
  rec_memref(out_zp);
  rec_ptr(attrs);
  MemRefType<int8_t, N> r;
  r.basePtr = reinterpret_cast<int8_t*>(0x1000);
  r.data = reinterpret_cast<int8_t*>(0x1040);
  r.offset = 7;
  for (int i = 0; i < N; ++i) {
    r.sizes[i] = 100 + i;
    r.strides[i] = 200 + i;
  }
  return r;
}

template <int N>
MemRefType<int8_t, N> stub_pdll_qgemm_pc(ExecutionContext* ctx, void* stream, MemRefType<int8_t, N> input,
                                         MemRefType<int8_t, 2> weight, MemRefType<int8_t, 1> bias,
                                         MemRefType<float, 1> in_s, MemRefType<int32_t, 1> in_zp,
                                         MemRefType<float, 1> w_s, MemRefType<int32_t, 1> w_zp,
                                         MemRefType<float, 1> out_s, MemRefType<int32_t, 1> out_zp,
                                         void* attrs) {
  g_record.clear();
  rec_ptr(ctx);
  rec_ptr(stream);
  rec_memref(input);
  rec_memref(weight);
  rec_memref(bias);
  rec_memref(in_s);
  rec_memref(in_zp);
  rec_memref(w_s);
  rec_memref(w_zp);
  rec_memref(out_s);
  rec_memref(out_zp);
  rec_ptr(attrs);
  MemRefType<int8_t, N> r;
  std::memset(&r, 0, sizeof(r));
  return r;
}

void stub_qgemm(ExecutionContext* ctx, void* stream, MemRefType<int8_t, 2> input,
                MemRefType<int8_t, 2> weight, MemRefType<float, 0> in_s, MemRefType<int32_t, 0> in_zp,
                MemRefType<float, 0> w_s, MemRefType<int32_t, 0> w_zp, MemRefType<float, 0> out_s,
                MemRefType<int32_t, 0> out_zp, MemRefType<int8_t, 2> result, bool tp_a, bool tp_b,
                bool weight_is_const) {
  g_record.clear();
  rec_ptr(ctx);
  rec_ptr(stream);
  rec_memref(input);
  rec_memref(weight);
  rec_memref(in_s);
  rec_memref(in_zp);
  rec_memref(w_s);
  rec_memref(w_zp);
  rec_memref(out_s);
  rec_memref(out_zp);
  rec_memref(result);
  rec(tp_a);
  rec(tp_b);
  rec(weight_is_const);
}

// Driver-set signatures (tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc).
void* stub_alloc(ExecutionContext* ctx, size_t bytes) {
  g_record.clear();
  rec_ptr(ctx);
  rec(static_cast<int64_t>(bytes));
  return reinterpret_cast<void*>(0x2000);
}
void stub_dealloc(ExecutionContext* ctx, void* p) {
  g_record.clear();
  rec_ptr(ctx);
  rec_ptr(p);
}
void* stub_alloc_persistent(ExecutionContext*, size_t) { return nullptr; }
void stub_memset(ExecutionContext*, void*, void*, int, size_t) {}
void* stub_get_stream(ExecutionContext*, int32_t) { return nullptr; }
void* stub_as_cu_stream(ExecutionContext*, void*) { return nullptr; }
void stub_d2d(ExecutionContext*, void*, void*, void*, size_t) {}
void stub_h2d(ExecutionContext*, void*, const void*, void*, size_t) {}
void stub_d2h(ExecutionContext*, void*, void*, void*, size_t) {}
void stub_sync_on_stream(ExecutionContext*, void*) {}
void stub_sync_all(ExecutionContext*) {}
void stub_launch(ExecutionContext*, void**, size_t, const char*, intptr_t, intptr_t, intptr_t, intptr_t,
                 intptr_t, intptr_t, int32_t, void*, int32_t, void**) {}
template <typename T, int N>
MemRefType<T, N> stub_recv_input(ExecutionContext*, int64_t) {
  MemRefType<T, N> m;
  std::memset(&m, 0, sizeof(m));
  return m;
}
template <typename T, int N>
void stub_send_output(ExecutionContext*, int64_t, MemRefType<T, N>) {}

// The collective calls of tao_compiler/mlir/ral/collective.cu.cc:60-440, with
// that file's signatures (it cannot be compiled here: CUDA, NCCL and
// TensorFlow headers), so that the names its registrations mangle are known.
template <typename T, int N>
MemRefType<T, N> stub_collective(ExecutionContext*, void*, MemRefType<T, N> input, void*) {
  return input;
}

// ral_const with the signature of ral_base_cuda_const_host / _cuda
// (tao_compiler/mlir/ral/context/common_context_impl.cc:279-283; the file needs
// the whole runtime to compile, so only its signature is restated).
template <typename T, int N>
MemRefType<T, N> stub_const(ExecutionContext*, void*, const char*, int32_t) {
  return MemRefType<T, N>();
}

// ral_qconv with the signature of gpu_conv_impl::ral_qconv<int8_t, 4>
// (tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:1831-1841; that file needs
// TensorFlow's StreamExecutor and cuDNN, so only the signature is restated).
void stub_qconv(ExecutionContext*, void*, MemRefType<int8_t, 4>, MemRefType<int8_t, 4>, MemRefType<int32_t, 1>,
                MemRefType<float, 0>, MemRefType<int32_t, 0>, MemRefType<float, 1>, MemRefType<int32_t, 1>,
                MemRefType<float, 0>, MemRefType<int32_t, 0>, MemRefType<int8_t, 4>, MemRefType<int32_t, 1>) {}

// "inc_ref" (alias and reshape) and the memref copies, with the signatures of
// tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc:544-625 and
// common_context_impl_cuda.cc:380-420 (files that need the whole CUDA runtime of the reference).
template <typename T, int N>
MemRefType<T, N> stub_alias(ExecutionContext*, void*, MemRefType<T, N> input) {
  return input;
}
template <typename T, int N, int M>
MemRefType<T, M> stub_reshape(ExecutionContext*, void*, MemRefType<T, N>, MemRefType<int64_t, 1>) {
  return MemRefType<T, M>();
}
template <typename T, int N>
void stub_copy(ExecutionContext*, void*, MemRefType<T, N>, MemRefType<T, N>) {}

// What the reference's parser made of a blob, as text: keys sorted, strings quoted,
// floats with 17 significant digits, dense tensors as dense<type bits[shape]:bytes B>.
void render_ref(tao::ral::PDLAttr& a, std::string& o) {
  const std::string& t = a.getType();
  if (t == "dict") {
    auto& items = a.as<tao::ral::DictPDLAttr>().getValue();
    std::vector<std::string> keys;
    for (auto& kv : items) keys.push_back(kv.first);
    std::sort(keys.begin(), keys.end());
    o += "{";
    for (size_t i = 0; i < keys.size(); ++i) {
      o += (i ? ", " : "") + keys[i] + ": ";
      render_ref(*items[keys[i]], o);
    }
    o += "}";
  } else if (t == "str") {
    o += "\"" + a.as<tao::ral::StrPDLAttr>().getValue() + "\"";
  } else if (t == "bool") {
    o += a.as<tao::ral::BoolPDLAttr>().getValue() ? "true" : "false";
  } else if (t == "int") {
    o += std::to_string(a.as<tao::ral::IntPDLAttr>().getValue());
  } else if (t == "float") {
    char buf[64];
    snprintf(buf, sizeof(buf), "%.17g", a.as<tao::ral::FloatPDLAttr>().getValue());
    o += buf;
  } else if (t == "intArray") {
    auto& v = a.as<tao::ral::IntArrayPDLAttr>().getValue();
    o += "[";
    for (size_t i = 0; i < v.size(); ++i) o += (i ? ", " : "") + std::to_string(v[i]);
    o += "]";
  } else if (t == "array") {
    auto& v = a.as<tao::ral::ArrayPDLAttr>().getValue();
    o += "[";
    for (size_t i = 0; i < v.size(); ++i) {
      if (i) o += ", ";
      render_ref(*v[i], o);
    }
    o += "]";
  } else if (t == "denseElementsAttr") {
    auto& d = a.as<tao::ral::DenseElementsPDLAttr>();
    o += "dense<" + d.getElementType() + std::to_string(d.getNumBits()) + "[";
    auto shape = d.getShape();
    for (size_t i = 0; i < shape.size(); ++i) o += (i ? "x" : "") + std::to_string(shape[i]);
    o += "]:" + std::to_string(d.getRawData().size()) + "B>";
  } else {
    o += "?" + t;
  }
}

template <typename F>
void note(const char* api, const char* device, F f) {
  g_names.push_back(
      tao::ral::TaoRalApiFuncNameHelper<F>::Invoke(std::string(api) + "___" + std::string(device)));
}

}  // namespace

#define REF_STUB2(api, device, line, ...)        \
  TAO_RAL_API(api, device, __VA_ARGS__);         \
  static bool disc_note_##line = (note(api, device, &__VA_ARGS__), true)
#define REF_STUB1(api, device, line, ...) REF_STUB2(api, device, line, __VA_ARGS__)
#define REF(api, device, ...) REF_STUB1(api, device, __COUNTER__, __VA_ARGS__)

REF("ral_pdll_qgemm", "gpu", stub_pdll_qgemm<2, int8_t>);
REF("ral_pdll_qgemm", "gpu", stub_pdll_qgemm<3, int8_t>);
REF("ral_pdll_qgemm", "gpu", stub_pdll_qgemm<2, float>);
REF("ral_pdll_qgemm", "gpu", stub_pdll_qgemm<3, float>);
REF("ral_pdll_qgemm_per_channel", "gpu", stub_pdll_qgemm_pc<2>);
REF("ral_pdll_qgemm_per_channel", "gpu", stub_pdll_qgemm_pc<3>);
REF("ral_qgemm", "gpu", stub_qgemm);
REF("alloc", "gpu", stub_alloc);
REF("dealloc", "gpu", stub_dealloc);
REF("ral_gpu_alloc_persistent", "gpu", stub_alloc_persistent);
REF("ral_gpu_memset", "gpu", stub_memset);
REF("ral_gpu_get_stream", "gpu", stub_get_stream);
REF("ral_gpu_as_cu_stream", "gpu", stub_as_cu_stream);
REF("d2d_", "gpu", stub_d2d);
REF("h2d_", "gpu", stub_h2d);
REF("d2h_", "gpu", stub_d2h);
REF("sync_on_stream", "gpu", stub_sync_on_stream);
REF("ral_gpu_sync_all", "gpu", stub_sync_all);
REF("ral_kernel_launch", "gpu", stub_launch);
REF("ral_recv_input", "cpu", stub_recv_input<float, 2>);
REF("ral_recv_input", "cpu", stub_recv_input<int8_t, 3>);
REF("ral_send_output", "cpu", stub_send_output<float, 2>);
REF("ral_send_output", "cpu", stub_send_output<int8_t, 3>);
REF("ral_recv_input", "cpu", stub_recv_input<uint8_t, 2>);
REF("ral_recv_input", "cpu", stub_recv_input<double, 8>);
REF("ral_send_output", "cpu", stub_send_output<bool, 5>);
REF("ral_send_output", "cpu", stub_send_output<int64_t, 0>);

#define REF_COLLECTIVES(T)                                              \
  REF("ral_all_reduce", "gpu", stub_collective<T, 0>);                    \
  REF("ral_all_reduce", "gpu", stub_collective<T, 1>);                    \
  REF("ral_all_reduce", "gpu", stub_collective<T, 2>);                    \
  REF("ral_all_reduce", "gpu", stub_collective<T, 3>);                    \
  REF("ral_all_reduce", "gpu", stub_collective<T, 4>);                    \
  REF("ral_all_gather", "gpu", stub_collective<T, 1>);                    \
  REF("ral_all_gather", "gpu", stub_collective<T, 2>);                    \
  REF("ral_all_gather", "gpu", stub_collective<T, 3>);                    \
  REF("ral_all_gather", "gpu", stub_collective<T, 4>);                    \
  REF("ral_async_collective_done", "gpu", stub_collective<T, 0>);         \
  REF("ral_async_collective_done", "gpu", stub_collective<T, 1>);         \
  REF("ral_async_collective_done", "gpu", stub_collective<T, 2>);         \
  REF("ral_async_collective_done", "gpu", stub_collective<T, 3>);         \
  REF("ral_async_collective_done", "gpu", stub_collective<T, 4>)
REF_COLLECTIVES(float);
REF_COLLECTIVES(tao::ral::float16);
REF_COLLECTIVES(tao::ral::bfloat16);

REF("ral_qconv", "gpu", stub_qconv);
REF("inc_ref", "gpu", stub_alias<float, 2>);
REF("inc_ref", "gpu", stub_alias<tao::ral::float16, 0>);
REF("inc_ref", "cpu", stub_alias<int64_t, 1>);
REF("inc_ref", "gpu", stub_reshape<float, 3, 2>);
REF("inc_ref", "gpu", stub_reshape<tao::ral::bfloat16, 8, 1>);
REF("inc_ref", "gpu", stub_reshape<bool, 1, 0>);
REF("inc_ref", "cpu", stub_reshape<int32_t, 0, 4>);
REF("h2d", "gpu", stub_copy<float, 2>);
REF("d2h", "gpu", stub_copy<int64_t, 0>);
REF("d2d", "gpu", stub_copy<double, 8>);

#define REF_CONSTS(T)                             \
  REF("ral_const", "cpu", stub_const<T, 0>);        \
  REF("ral_const", "cpu", stub_const<T, 1>);        \
  REF("ral_const", "cpu", stub_const<T, 2>);        \
  REF("ral_const", "cpu", stub_const<T, 8>);        \
  REF("ral_const", "gpu", stub_const<T, 0>);        \
  REF("ral_const", "gpu", stub_const<T, 1>);        \
  REF("ral_const", "gpu", stub_const<T, 2>);        \
  REF("ral_const", "gpu", stub_const<T, 4>);        \
  REF("ral_const", "gpu", stub_const<T, 8>)
REF_CONSTS(double);
REF_CONSTS(float);
REF_CONSTS(tao::ral::float16);
REF_CONSTS(tao::ral::bfloat16);
REF_CONSTS(int8_t);
REF_CONSTS(uint8_t);
REF_CONSTS(int16_t);
REF_CONSTS(uint16_t);
REF_CONSTS(int32_t);
REF_CONSTS(uint32_t);
REF_CONSTS(int64_t);
REF_CONSTS(bool);

extern "C" {

int ref_num_names() { return static_cast<int>(g_names.size()); }
const char* ref_name(int i) { return g_names[i].c_str(); }

// Dispatches through the reference's own entry point with a reference
// Context / ExecutionContext; returns the number of recorded values.
int ref_dispatch(const char* name, void** args) {
  static tao::ral::Context* ctx = new tao::ral::Context;
  tao::ral::ExecutionContext exec(ctx);
  // The generated stub overwrites the first argument with the real context.
  *static_cast<void**>(args[0]) = &exec;
  tao_ral_call_impl(&exec, const_cast<char*>(name), args);
  return static_cast<int>(g_record.size());
}
int64_t ref_recorded(int i) { return g_record[i]; }

// The reference's parser on a custom_attrs blob (context/pdll_util.cc:20-170): length of the
// rendering, -1 if it could not parse; the text is copied into out when it fits.
int ref_attrs_describe(const void* blob, char* out, int capacity) {
  uint8_t* cur = const_cast<uint8_t*>(static_cast<const uint8_t*>(blob));
  auto attr = tao::ral::parsePDLAttr(cur);
  if (!attr) return -1;
  std::string text;
  render_ref(*attr, text);
  if (static_cast<int>(text.size()) < capacity) std::memcpy(out, text.c_str(), text.size() + 1);
  return static_cast<int>(text.size());
}

// The reference's emitter (ral_metadata.cc:117-167): header, constants, tailer.
// Values are the hexadecimal strings the compiler would have produced.
int ref_metadata_write(const char* path, int n, const char* const* names, const int* is_host,
                       const char* const* hex_values) {
  tao::ral::MetadataFileEmitter emitter(path);
  if (!emitter.emitHeader()) return 1;
  for (int i = 0; i < n; ++i) {
    const bool ok = is_host[i] ? emitter.emitHostConstant(names[i], hex_values[i])
                               : emitter.emitDeviceConstant(names[i], hex_values[i]);
    if (!ok) return 2;
  }
  return emitter.emitTailer() ? 0 : 3;
}

// The reference's loader (ral_metadata.cc:65-115): length of the value, or -1 if
// the file does not load, -2 if there is no such constant; the value is copied
// into buf when it fits.
int64_t ref_metadata_get(const char* path, const char* name, int is_host, char* buf, int64_t cap) {
  auto file = tao::ral::MetadataFile::loadFromFile(path);
  if (!file) return -1;
  const std::string* value = nullptr;
  const bool found = is_host ? file->getHostConstant(name, value) : file->getDeviceConstant(name, value);
  if (!found || !value) return -2;
  if (static_cast<int64_t>(value->size()) <= cap) std::memcpy(buf, value->data(), value->size());
  return static_cast<int64_t>(value->size());
}
}

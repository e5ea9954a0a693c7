// Custom calls registered with the dispatcher.
//
// Part 1 is the driver set a compiled executable and the kernels rely on
// (reference: tao_compiler/mlir/ral/device/gpu/gpu_driver.cc:29-43 names,
// tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc:258-510,627-764
// behaviour, tao_compiler/mlir/ral/context/base/base_context.cc:136-235 I/O).
// Part 2 is the quantized GEMM family with the reference's names, operand
// order and result ownership (tao_compiler/mlir/ral/context/
// quantized_gpu_kernel_impl.cc:197-481, stream_executor_based_impl.cc:427-483).
// Part 3 registers the fused forms and the bandwidth kernels under new names a
// PDLL pattern can target (any registered name is reachable from a
// custom_call_v2: docs/developers/add_custom_call.md of the reference).
#include <cstring>
#include <memory>
#include <tuple>

#include "../kernels/qconv.h"
#include "../kernels/qgemm.h"
#include "../kernels/rowops.h"
#include "../kernels/woq_gemm.h"
#include "abi.h"
#include "context.h"
#include "conv_plan.h"
#include "cu_driver_dyn.h"
#include "nccl_dyn.h"
#include "pdl_attr.h"

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

void report(ExecContext* ctx, cudaError_t st, const char* what, const char* detail) {
  if (st == cudaSuccess) return;
  std::string m = std::string(what) + ": " + (detail ? detail : cudaGetErrorString(st));
  ctx->signal_error(m);
}

// ------------------------------------------------------------ 1. drivers
void* ral_alloc(ExecContext* ctx, uint64_t bytes) { return ctx->alloc(bytes); }
void ral_dealloc(ExecContext* ctx, void* p) { ctx->dealloc(p); }
void* ral_alloc_persistent(ExecContext* ctx, uint64_t bytes) {
  void* p = ctx->ctx->raw_alloc(bytes);
  if (!p) {
    ctx->signal_error("persistent device allocation failed");
    return nullptr;
  }
  std::lock_guard<std::mutex> l(ctx->ctx->mu);
  ctx->ctx->persistent.insert(p);
  return p;
}
void ral_memset(ExecContext* ctx, void* handle, void* p, int32_t value, uint64_t bytes) {
  if (!p) return;
  report(ctx, cudaMemsetAsync(p, value, bytes, stream_of(ctx)), "memset", nullptr);
}
void* ral_get_stream(ExecContext* ctx, int32_t idx) {
  if (idx < 0) {
    ctx->signal_error("not a valid stream_id");
    return nullptr;
  }
  if (idx > 0) {
    ctx->signal_error("multi-stream not supported");
    return nullptr;
  }
  return nullptr;  // handle of stream 0 is the integer 0
}
void* ral_as_cu_stream(ExecContext* ctx, void* handle) { return stream_of(ctx); }
void ral_d2d(ExecContext* ctx, void* handle, void* from, void* to, uint64_t bytes) {
  if (!check_stream_handle(ctx, handle)) return;
  report(ctx, cudaMemcpyAsync(to, from, bytes, cudaMemcpyDeviceToDevice, stream_of(ctx)), "d2d", nullptr);
}
void ral_h2d(ExecContext* ctx, void* handle, const void* from, void* to, uint64_t bytes) {
  report(ctx, cudaMemcpyAsync(to, from, bytes, cudaMemcpyHostToDevice, stream_of(ctx)), "h2d", nullptr);
}
void ral_d2h(ExecContext* ctx, void* handle, void* from, void* to, uint64_t bytes) {
  report(ctx, cudaMemcpyAsync(to, from, bytes, cudaMemcpyDeviceToHost, stream_of(ctx)), "d2h", nullptr);
}
void ral_sync_on_stream(ExecContext* ctx, void* handle) {
  if (!check_stream_handle(ctx, handle)) return;
  report(ctx, cudaStreamSynchronize(stream_of(ctx)), "StreamSync", nullptr);
}
void ral_sync_all(ExecContext* ctx) { report(ctx, cudaDeviceSynchronize(), "DeviceSync", nullptr); }

// A kernel the compiler generated (kLoop / kStitch fusions and everything else
// that is not a library call), embedded in the executable as one or several
// device images.  Same selection, caching and launch as the reference
// (cuda_context_impl.cc:348-445).  Images built for sm_60..sm_86 carry no code a
// B200 can run; what runs here is the PTX of image 0, compiled by the driver on
// first use, or an image a newer compiler built for sm_100.  The quantized path
// itself does not come through here: its kernels are the custom calls of part 3.
void ral_kernel_launch(ExecContext* ctx, void** blobs, uint64_t num_blobs, const char* name,
                       int64_t gx, int64_t gy, int64_t gz, int64_t bx, int64_t by, int64_t bz,
                       int32_t smem, void* stream, int32_t num_args, void** params) {
  if (!gx || !gy || !gz || !bx || !by || !bz) return;  // empty tensor: nothing to launch (:356-359)
  if (!blobs || !name || num_blobs == 0) {
    ctx->signal_error("ral_kernel_launch: no device image or no kernel name");
    return;
  }
  if (gx < 0 || gy < 0 || gz < 0 || bx < 0 || by < 0 || bz < 0 || smem < 0 || bx * by * bz > 1024) {
    ctx->signal_error(std::string("ral_kernel_launch: invalid launch dimensions for ") + name);
    return;
  }
  const CuDriverApi& cu = cu_driver_api();
  if (!cu.ok) {
    ctx->signal_error("ral_kernel_launch: CUDA driver unavailable: " + cu.error);
    return;
  }
  Context* c = ctx->ctx;
  void* function = nullptr;
  {
    std::lock_guard<std::mutex> l(c->mu);
    if (c->cc_major == 0) {
      cudaFree(nullptr);  // binds the device's primary context to this thread for the driver calls
      cudaDeviceGetAttribute(&c->cc_major, cudaDevAttrComputeCapabilityMajor, c->device);
      cudaDeviceGetAttribute(&c->cc_minor, cudaDevAttrComputeCapabilityMinor, c->device);
    }
    const int pick = select_blob(num_blobs, c->cc_major, c->cc_minor);
    const void* image = blobs[pick];
    auto key = std::make_pair(image, std::string(name));
    auto it = c->kernels.find(key);
    if (it == c->kernels.end()) {
      auto mod = c->modules.find(image);
      if (mod == c->modules.end()) {
        void* module = nullptr;
        const int st = image ? cu.ModuleLoadData(&module, image) : 1;
        if (st != 0 || !module) {
          const std::string why = "ral_kernel_launch: ModuleLoad of image " + std::to_string(pick) + " of " +
                                  std::to_string(num_blobs) + " for kernel '" + name + "': " + cu.describe(st) +
                                  " (device is sm_" + std::to_string(c->cc_major) + std::to_string(c->cc_minor) +
                                  "; the image needs code for it or PTX the driver can compile)";
          if (c->status == 0) {  // mu is held
            c->status = 1;
            c->message = why;
          }
          return;
        }
        mod = c->modules.emplace(image, module).first;
      }
      void* fn = nullptr;
      const int st = cu.ModuleGetFunction(&fn, mod->second, name);
      if (st != 0 || !fn) {
        if (c->status == 0) {
          c->status = 1;
          c->message = std::string("ral_kernel_launch: GetFunction '") + name + "': " + cu.describe(st);
        }
        return;
      }
      if (smem > 48 * 1024) cu.FuncSetAttribute(fn, kCuFuncAttrMaxDynamicShared, smem);
      it = c->kernels.emplace(key, fn).first;
    }
    function = it->second;
  }
  const int st = cu.LaunchKernel(function, static_cast<unsigned>(gx), static_cast<unsigned>(gy),
                                 static_cast<unsigned>(gz), static_cast<unsigned>(bx), static_cast<unsigned>(by),
                                 static_cast<unsigned>(bz), static_cast<unsigned>(smem), stream_of(ctx), params,
                                 nullptr);
  if (st != 0) ctx->signal_error(std::string("ral_kernel_launch: LaunchKernel '") + name + "': " + cu.describe(st));
}

DISC_B200_RAL_API("alloc", "gpu", ral_alloc);
DISC_B200_RAL_API("dealloc", "gpu", ral_dealloc);
DISC_B200_RAL_API("ral_gpu_alloc_persistent", "gpu", ral_alloc_persistent);
DISC_B200_RAL_API("ral_gpu_memset", "gpu", ral_memset);
DISC_B200_RAL_API("ral_gpu_get_stream", "gpu", ral_get_stream);
DISC_B200_RAL_API("ral_gpu_as_cu_stream", "gpu", ral_as_cu_stream);
DISC_B200_RAL_API("d2d_", "gpu", ral_d2d);
DISC_B200_RAL_API("h2d_", "gpu", ral_h2d);
DISC_B200_RAL_API("d2h_", "gpu", ral_d2h);
DISC_B200_RAL_API("sync_on_stream", "gpu", ral_sync_on_stream);
DISC_B200_RAL_API("ral_gpu_sync_all", "gpu", ral_sync_all);
DISC_B200_RAL_API("ral_kernel_launch", "gpu", ral_kernel_launch);

// Host buffers of generated code (cpu_context_impl.cc:120-215: "alloc", "dealloc" and
// "ral_cpu_alloc_persistent" on "cpu").
void* ral_host_alloc(ExecContext* ctx, uint64_t bytes) { return ctx->host_alloc(bytes); }
void ral_host_dealloc(ExecContext* ctx, void* p) { ctx->host_dealloc(p); }
void* ral_host_alloc_persistent(ExecContext* ctx, uint64_t bytes) {
  void* p = ctx->host_alloc(bytes);
  if (!p) return nullptr;
  ctx->host_refcount.erase(p);
  std::lock_guard<std::mutex> l(ctx->ctx->mu);
  ctx->ctx->host_persistent.insert(p);
  return p;
}
DISC_B200_RAL_API("alloc", "cpu", ral_host_alloc);
DISC_B200_RAL_API("dealloc", "cpu", ral_host_dealloc);
DISC_B200_RAL_API("ral_cpu_alloc_persistent", "cpu", ral_host_alloc_persistent);

template <typename T, int N>
MemRef<T, N> ral_recv_input(ExecContext* ctx, int64_t idx) {
  MemRef<T, N> m;
  std::memset(&m, 0, sizeof(m));
  auto it = ctx->inputs.find(idx);
  if (it == ctx->inputs.end()) {
    ctx->signal_error("invalid input index");
    return m;
  }
  if (static_cast<int>(it->second.shape.size()) != N) {
    ctx->signal_error("input rank does not match the compiled signature");
    return m;
  }
  return make_memref<T, N>(static_cast<T*>(it->second.data), it->second.shape.data());
}

template <typename T, int N>
void ral_send_output(ExecContext* ctx, int64_t idx, MemRef<T, N> m) {
  BoundTensor t;
  t.data = m.data;
  if constexpr (N > 0) t.shape.assign(m.sizes, m.sizes + N);
  ctx->outputs[idx] = t;
}

#define DISC_B200_REGISTER_IO(T, N)                                     \
  DISC_B200_RAL_API("ral_recv_input", "cpu", ral_recv_input<T, N>);     \
  DISC_B200_RAL_API("ral_send_output", "cpu", ral_send_output<T, N>)
// ranks 0..8 and the element types of the reference (base_context.cc:222-300), plus the
// 16-bit floats at every rank (the reference has them for rank 0 only, and in its CUDA build)
#define DISC_B200_REGISTER_IO_RANKS(T) \
  DISC_B200_REGISTER_IO(T, 0);         \
  DISC_B200_REGISTER_IO(T, 1);         \
  DISC_B200_REGISTER_IO(T, 2);         \
  DISC_B200_REGISTER_IO(T, 3);         \
  DISC_B200_REGISTER_IO(T, 4);         \
  DISC_B200_REGISTER_IO(T, 5);         \
  DISC_B200_REGISTER_IO(T, 6);         \
  DISC_B200_REGISTER_IO(T, 7);         \
  DISC_B200_REGISTER_IO(T, 8)
DISC_B200_REGISTER_IO_RANKS(float);
DISC_B200_REGISTER_IO_RANKS(double);
DISC_B200_REGISTER_IO_RANKS(f16_t);
DISC_B200_REGISTER_IO_RANKS(bf16_t);
DISC_B200_REGISTER_IO_RANKS(int8_t);
DISC_B200_REGISTER_IO_RANKS(uint8_t);
DISC_B200_REGISTER_IO_RANKS(int32_t);
DISC_B200_REGISTER_IO_RANKS(int64_t);
DISC_B200_REGISTER_IO_RANKS(bool);

// ------------------------------------------------------------ attr cache
struct AttrCache {
  struct Entry {
    std::unique_ptr<Attr> attr;
    std::string bytes;  // the blob as it was when parsed
  };
  std::mutex mu;
  std::unordered_map<void*, Entry> map;
  std::vector<std::unique_ptr<Attr>> retired;  // replaced entries stay alive: a caller may still hold one
};
AttrCache& attr_cache() {
  static AttrCache* c = new AttrCache;
  return *c;
}
// Parsed once per blob address, like the reference (pdll_util.h:190-220).  In a
// compiled executable a blob is constant data; a host that builds blobs at run
// time may reuse an address for other content, so a hit also compares the bytes.
const Attr* attrs_of(ExecContext* ctx, void* blob) {
  static const Attr kEmpty = [] {
    Attr a;
    a.kind = Attr::kDict;
    return a;
  }();
  if (!blob) return &kEmpty;
  AttrCache& c = attr_cache();
  std::lock_guard<std::mutex> l(c.mu);
  auto it = c.map.find(blob);
  if (it != c.map.end()) {
    // Byte by byte, stopping at the first difference: the blob's own length is not known before
    // it is parsed, and a well-formed blob that agrees with the cached one on all of its bytes
    // has the cached one's length (every length is part of the bytes), so nothing past it is read.
    const char* now = static_cast<const char*>(blob);
    const std::string& was = it->second.bytes;
    size_t i = 0;
    while (i < was.size() && now[i] == was[i]) ++i;
    if (i == was.size()) return it->second.attr.get();
  }
  const uint8_t* cur = static_cast<const uint8_t*>(blob);
  auto a = parse_attr(&cur);
  if (!a || a->kind != Attr::kDict) {
    ctx->signal_error("fail to parse custom_attrs");
    return nullptr;
  }
  AttrCache::Entry e;
  e.attr = std::move(a);
  e.bytes.assign(static_cast<const char*>(blob), static_cast<size_t>(cur - static_cast<const uint8_t*>(blob)));
  if (it != c.map.end()) {
    c.retired.push_back(std::move(it->second.attr));
    it->second = std::move(e);
  } else {
    it = c.map.emplace(blob, std::move(e)).first;
  }
  return it->second.attr.get();
}

// ---------------------------------------------------- 2. reference qgemm
template <int N>
int64_t leading_rows(const MemRef<int8_t, N>& in, int64_t* result_sizes, int64_t n) {
  int64_t m = 1;
  for (int i = 0; i < N - 1; ++i) {
    m *= in.sizes[i];
    result_sizes[i] = in.sizes[i];
  }
  result_sizes[N - 1] = n;
  return m;
}

bool run_qgemm(ExecContext* ctx, QGemmParams& p) {
  if (p.M <= 128) {
    const int64_t need = qgemm_splitk_ws_bytes(p.M, p.N, p.K);
    int64_t have = 0;
    p.splitk_ws = static_cast<int32_t*>(ctx->ctx->get_splitk_ws(need, &have));
    p.splitk_ws_bytes = p.splitk_ws ? have : 0;
  }
  const char* detail = nullptr;
  cudaError_t st = qgemm_launch(p, stream_of(ctx), &detail);
  if (st != cudaSuccess) {
    report(ctx, st, "qgemm", detail);
    return false;
  }
  return true;
}

QGemmParams base_params(const int8_t* a, const int8_t* w, void* out, int64_t m, int64_t n,
                        int64_t k) {
  QGemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.a = a;
  p.w = w;
  p.out = out;
  p.M = m;
  p.N = n;
  p.K = k;
  p.lda = k;
  p.ldw = k;
  p.ldo = n;
  return p;
}

// out_i8 = sat(rne(acc * (s_x * s_w / s_out) + bias)), zero points ignored
// (symmetric), result allocated here and owned by the caller.
template <int N, typename BiasT>
MemRef<int8_t, N> pdll_qgemm_per_tensor(ExecContext* ctx, void* stream_handle,
                                        MemRef<int8_t, N> input, MemRef<int8_t, 2> weight,
                                        MemRef<BiasT, 1> bias, MemRef<float, 0> in_scale,
                                        MemRef<int32_t, 0> in_zp, MemRef<float, 0> w_scale,
                                        MemRef<int32_t, 0> w_zp, MemRef<float, 0> out_scale,
                                        MemRef<int32_t, 0> out_zp, void* custom_attrs) {
  const int64_t k = weight.sizes[1];
  const int64_t n = weight.sizes[0];
  int64_t rs[N];
  const int64_t m = leading_rows<N>(input, rs, n);
  if (memref_numel(input) == 0 || memref_numel(weight) == 0) {
    return make_memref<int8_t, N>(nullptr, rs);
  }
  if (input.sizes[N - 1] != k) {
    ctx->signal_error("ral_pdll_qgemm: input and weight disagree on K");
    return make_memref<int8_t, N>(nullptr, rs);
  }
  int8_t* out = static_cast<int8_t*>(ctx->alloc(static_cast<size_t>(m * n)));
  auto result = make_memref<int8_t, N>(out, rs);
  if (!out) return result;
  QGemmParams p = base_params(input.data, weight.data, out, m, n, k);
  p.x_scale = in_scale.data;
  p.w_scale = w_scale.data;
  p.out_scale = out_scale.data;
  p.x_scale_kind = kScaleScalar;
  p.w_scale_kind = kScaleScalar;
  p.out_scale_kind = kScaleScalar;
  p.fold_out_scale = 1;
  p.bias = bias.data;
  p.bias_kind = std::is_same_v<BiasT, float> ? kBiasF32 : kBiasI8;
  p.out_dtype = kOutI8;
  run_qgemm(ctx, p);
  return result;
}

// Per-channel form produced by the QKV-merge pass: every scale operand has N
// entries, bias is int8.
template <int N>
MemRef<int8_t, N> pdll_qgemm_per_channel(ExecContext* ctx, void* stream_handle,
                                         MemRef<int8_t, N> input, MemRef<int8_t, 2> weight,
                                         MemRef<int8_t, 1> bias, MemRef<float, 1> in_scale,
                                         MemRef<int32_t, 1> in_zp, MemRef<float, 1> w_scale,
                                         MemRef<int32_t, 1> w_zp, MemRef<float, 1> out_scale,
                                         MemRef<int32_t, 1> out_zp, void* custom_attrs) {
  const int64_t k = weight.sizes[1];
  const int64_t n = weight.sizes[0];
  int64_t rs[N];
  const int64_t m = leading_rows<N>(input, rs, n);
  if (memref_numel(input) == 0 || memref_numel(weight) == 0) {
    return make_memref<int8_t, N>(nullptr, rs);
  }
  if (input.sizes[N - 1] != k || in_scale.sizes[0] != n || w_scale.sizes[0] != n ||
      out_scale.sizes[0] != n || bias.sizes[0] != n) {
    ctx->signal_error("ral_pdll_qgemm_per_channel: operand extents disagree");
    return make_memref<int8_t, N>(nullptr, rs);
  }
  int8_t* out = static_cast<int8_t*>(ctx->alloc(static_cast<size_t>(m * n)));
  auto result = make_memref<int8_t, N>(out, rs);
  if (!out) return result;
  QGemmParams p = base_params(input.data, weight.data, out, m, n, k);
  p.x_scale = in_scale.data;
  p.w_scale = w_scale.data;
  p.out_scale = out_scale.data;
  p.x_scale_kind = kScalePerCol;
  p.w_scale_kind = kScalePerCol;
  p.out_scale_kind = kScalePerCol;
  p.fold_out_scale = 1;
  p.bias = bias.data;
  p.bias_kind = kBiasI8;
  p.out_dtype = kOutI8;
  run_qgemm(ctx, p);
  return result;
}

// Older form: result buffer passed in, no bias.  The GPU rewriter lays the
// weight out as [N, K] (tp_b = true); other layouts are not produced for GPU.
void ral_qgemm_gpu(ExecContext* ctx, void* stream_handle, MemRef<int8_t, 2> input,
                   MemRef<int8_t, 2> weight, MemRef<float, 0> in_scale, MemRef<int32_t, 0> in_zp,
                   MemRef<float, 0> w_scale, MemRef<int32_t, 0> w_zp, MemRef<float, 0> out_scale,
                   MemRef<int32_t, 0> out_zp, MemRef<int8_t, 2> result, bool tp_a, bool tp_b,
                   bool weight_is_const) {
  if (memref_numel(input) == 0 || memref_numel(weight) == 0 || memref_numel(result) == 0) return;
  if (tp_a || !tp_b) {
    ctx->signal_error("ral_qgemm: only input [M,K] x weight [N,K] (tp_a = false, tp_b = true)");
    return;
  }
  const int64_t m = input.sizes[0], k = input.sizes[1], n = weight.sizes[0];
  if (weight.sizes[1] != k || result.sizes[0] != m || result.sizes[1] != n) {
    ctx->signal_error("ral_qgemm: operand extents disagree");
    return;
  }
  QGemmParams p = base_params(input.data, weight.data, result.data, m, n, k);
  p.x_scale = in_scale.data;
  p.w_scale = w_scale.data;
  p.out_scale = out_scale.data;
  p.x_scale_kind = kScaleScalar;
  p.w_scale_kind = kScaleScalar;
  p.out_scale_kind = kScaleScalar;
  p.fold_out_scale = 1;
  p.bias_kind = kBiasNone;
  p.out_dtype = kOutI8;
  run_qgemm(ctx, p);
}

DISC_B200_RAL_API("ral_pdll_qgemm", "gpu", pdll_qgemm_per_tensor<2, int8_t>);
DISC_B200_RAL_API("ral_pdll_qgemm", "gpu", pdll_qgemm_per_tensor<3, int8_t>);
DISC_B200_RAL_API("ral_pdll_qgemm", "gpu", pdll_qgemm_per_tensor<2, float>);
DISC_B200_RAL_API("ral_pdll_qgemm", "gpu", pdll_qgemm_per_tensor<3, float>);
DISC_B200_RAL_API("ral_pdll_qgemm_per_channel", "gpu", pdll_qgemm_per_channel<2>);
DISC_B200_RAL_API("ral_pdll_qgemm_per_channel", "gpu", pdll_qgemm_per_channel<3>);
DISC_B200_RAL_API("ral_qgemm", "gpu", ral_qgemm_gpu);

// ------------------------------------------------------- 3. fused forms
int act_from(const Attr* a) {
  const std::string s = a->get_str("activation", "none");
  if (s == "gelu") return kActGelu;
  if (s == "silu") return kActSilu;
  return kActNone;
}

template <typename T>
constexpr int elem_type_of() {
  return std::is_same_v<T, float> ? kF32 : kF16;
}

// y = act(acc * s_x * s_w[n] + bias[n]) as f16, or requantized to int8 at
// out_scale: dequantize + bias + activation (+ quantize) of the reference
// graph in the GEMM epilogue.  XS is MemRef<float,0> (static activation scale)
// or MemRef<float,1> (one scale per row, from disc_b200_dynamic_quantize).
template <int N, typename OutT, typename XS>
MemRef<OutT, N> fused_qgemm(ExecContext* ctx, void* stream_handle, MemRef<int8_t, N> input,
                            MemRef<int8_t, 2> weight, MemRef<float, 1> bias, XS x_scale,
                            MemRef<float, 1> w_scale, MemRef<float, 0> out_scale,
                            void* custom_attrs) {
  const int64_t k = weight.sizes[1];
  const int64_t n = weight.sizes[0];
  int64_t rs[N];
  const int64_t m = leading_rows<N>(input, rs, n);
  if (memref_numel(input) == 0 || memref_numel(weight) == 0) {
    return make_memref<OutT, N>(nullptr, rs);
  }
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<OutT, N>(nullptr, rs);
  if (input.sizes[N - 1] != k || w_scale.sizes[0] != n) {
    ctx->signal_error("disc_b200_qgemm: operand extents disagree");
    return make_memref<OutT, N>(nullptr, rs);
  }
  OutT* out = static_cast<OutT*>(ctx->alloc(static_cast<size_t>(m * n) * sizeof(OutT)));
  auto result = make_memref<OutT, N>(out, rs);
  if (!out) return result;
  QGemmParams p = base_params(input.data, weight.data, out, m, n, k);
  p.x_scale = x_scale.data;
  p.x_scale_kind = std::is_same_v<XS, MemRef<float, 0>> ? kScaleScalar : kScalePerRow;
  p.w_scale = w_scale.data;
  p.w_scale_kind = kScalePerCol;
  p.bias = memref_numel(bias) == n ? bias.data : nullptr;
  p.bias_kind = p.bias ? kBiasF32 : kBiasNone;
  p.act = act_from(at);
  if constexpr (std::is_same_v<OutT, int8_t>) {
    p.out_scale = out_scale.data;
    p.out_scale_kind = kScaleScalar;
    p.div_out_scale = 1;
    p.div_exact = at->get_bool("exact_division", false) ? 1 : 0;
    p.out_dtype = kOutI8;
  } else {
    p.out_dtype = kOutF16;
  }
  run_qgemm(ctx, p);
  return result;
}

DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<2, f16_t, MemRef<float, 0>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<3, f16_t, MemRef<float, 0>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<2, int8_t, MemRef<float, 0>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<3, int8_t, MemRef<float, 0>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<2, f16_t, MemRef<float, 1>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<3, f16_t, MemRef<float, 1>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<2, int8_t, MemRef<float, 1>>);
DISC_B200_RAL_API("disc_b200_qgemm", "gpu", fused_qgemm<3, int8_t, MemRef<float, 1>>);

template <typename T, int N>
MemRef<int8_t, N> quantize_call(ExecContext* ctx, void* stream_handle, MemRef<T, N> x,
                                MemRef<float, 0> scale, MemRef<int32_t, 0> zp, void* custom_attrs) {
  const int64_t numel = memref_numel(x);
  if (numel == 0) return make_memref<int8_t, N>(nullptr, x.sizes);
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<int8_t, N>(nullptr, x.sizes);
  int8_t* q = static_cast<int8_t*>(ctx->alloc(static_cast<size_t>(numel)));
  auto result = make_memref<int8_t, N>(q, x.sizes);
  if (!q) return result;
  QuantizeParams p;
  p.x = x.data;
  p.q = q;
  p.numel = numel;
  p.in_type = elem_type_of<T>();
  p.scale = scale.data;
  p.zero_point = zp.data;
  p.channels = 1;
  p.inner = 1;
  p.qmin = static_cast<int>(at->get_int("quant_min", -128));
  p.qmax = static_cast<int>(at->get_int("quant_max", 127));
  const char* detail = nullptr;
  const cudaError_t launch_st = quantize_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "quantize", detail);
  return result;
}

template <typename T, int N>
std::tuple<MemRef<int8_t, N>, MemRef<float, 1>> dynamic_quantize_call(ExecContext* ctx,
                                                                      void* stream_handle,
                                                                      MemRef<T, N> x,
                                                                      void* custom_attrs) {
  const int64_t cols = x.sizes[N - 1];
  const int64_t numel = memref_numel(x);
  const int64_t rows = cols > 0 ? numel / cols : 0;
  int64_t rsz[1] = {rows};
  if (numel == 0) {
    return std::make_tuple(make_memref<int8_t, N>(nullptr, x.sizes), make_memref<float, 1>(nullptr, rsz));
  }
  int8_t* q = static_cast<int8_t*>(ctx->alloc(static_cast<size_t>(numel)));
  float* s = static_cast<float*>(ctx->alloc(static_cast<size_t>(rows) * sizeof(float)));
  auto r0 = make_memref<int8_t, N>(q, x.sizes);
  auto r1 = make_memref<float, 1>(s, rsz);
  if (!q || !s) return std::make_tuple(r0, r1);
  DynQuantParams p;
  p.x = x.data;
  p.q = q;
  p.row_scale = s;
  p.rows = rows;
  p.cols = cols;
  p.in_type = elem_type_of<T>();
  const char* detail = nullptr;
  const cudaError_t launch_st = dynamic_quantize_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "dynamic_quantize", detail);
  return std::make_tuple(r0, r1);
}

template <typename T, int N>
MemRef<T, N> dequantize_call(ExecContext* ctx, void* stream_handle, MemRef<int8_t, N> q,
                             MemRef<float, 0> scale, MemRef<int32_t, 0> zp, void* custom_attrs) {
  const int64_t numel = memref_numel(q);
  if (numel == 0) return make_memref<T, N>(nullptr, q.sizes);
  T* y = static_cast<T*>(ctx->alloc(static_cast<size_t>(numel) * sizeof(T)));
  auto result = make_memref<T, N>(y, q.sizes);
  if (!y) return result;
  DequantizeParams p;
  p.q = q.data;
  p.y = y;
  p.numel = numel;
  p.out_type = elem_type_of<T>();
  p.scale = scale.data;
  p.zero_point = zp.data;
  p.channels = 1;
  p.inner = 1;
  const char* detail = nullptr;
  const cudaError_t launch_st = dequantize_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "dequantize", detail);
  return result;
}

template <typename T, int N>
NormParams norm_params(const MemRef<T, N>& x, const T* residual, const T* gamma, const T* beta,
                       float eps, int rms) {
  NormParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = x.data;
  p.residual = residual;
  p.gamma = gamma;
  p.beta = beta;
  p.cols = x.sizes[N - 1];
  p.rows = p.cols > 0 ? memref_numel(x) / p.cols : 0;
  p.eps = eps;
  p.type = elem_type_of<T>();
  p.rms = rms;
  return p;
}

template <typename T, int N>
MemRef<T, N> layernorm_call(ExecContext* ctx, void* stream_handle, MemRef<T, N> x,
                            MemRef<T, 1> gamma, MemRef<T, 1> beta, void* custom_attrs) {
  if (memref_numel(x) == 0) return make_memref<T, N>(nullptr, x.sizes);
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<T, N>(nullptr, x.sizes);
  T* y = static_cast<T*>(ctx->alloc(static_cast<size_t>(memref_numel(x)) * sizeof(T)));
  auto result = make_memref<T, N>(y, x.sizes);
  if (!y) return result;
  NormParams p = norm_params<T, N>(x, nullptr, gamma.data, beta.data,
                                   static_cast<float>(at->get_float("eps", 1e-5)), 0);
  p.y = y;
  const char* detail = nullptr;
  const cudaError_t launch_st = norm_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "layernorm", detail);
  return result;
}

template <typename T, int N>
MemRef<T, N> add_layernorm_call(ExecContext* ctx, void* stream_handle, MemRef<T, N> x,
                                MemRef<T, N> residual, MemRef<T, 1> gamma, MemRef<T, 1> beta,
                                void* custom_attrs) {
  if (memref_numel(x) == 0) return make_memref<T, N>(nullptr, x.sizes);
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<T, N>(nullptr, x.sizes);
  if (memref_numel(residual) != memref_numel(x)) {
    ctx->signal_error("disc_b200_add_layernorm: residual shape differs");
    return make_memref<T, N>(nullptr, x.sizes);
  }
  T* y = static_cast<T*>(ctx->alloc(static_cast<size_t>(memref_numel(x)) * sizeof(T)));
  auto result = make_memref<T, N>(y, x.sizes);
  if (!y) return result;
  NormParams p = norm_params<T, N>(x, residual.data, gamma.data, beta.data,
                                   static_cast<float>(at->get_float("eps", 1e-5)), 0);
  p.y = y;
  const char* detail = nullptr;
  const cudaError_t launch_st = norm_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "add_layernorm", detail);
  return result;
}

// LayerNorm(x + residual) with a second, int8 output at a static scale.
template <typename T, int N>
std::tuple<MemRef<T, N>, MemRef<int8_t, N>> add_layernorm_quant_call(
    ExecContext* ctx, void* stream_handle, MemRef<T, N> x, MemRef<T, N> residual,
    MemRef<T, 1> gamma, MemRef<T, 1> beta, MemRef<float, 0> q_scale, void* custom_attrs) {
  auto empty = std::make_tuple(make_memref<T, N>(nullptr, x.sizes), make_memref<int8_t, N>(nullptr, x.sizes));
  if (memref_numel(x) == 0) return empty;
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return empty;
  if (memref_numel(residual) != memref_numel(x)) {
    ctx->signal_error("disc_b200_add_layernorm_quant: residual shape differs");
    return empty;
  }
  const size_t numel = static_cast<size_t>(memref_numel(x));
  T* y = static_cast<T*>(ctx->alloc(numel * sizeof(T)));
  int8_t* q = static_cast<int8_t*>(ctx->alloc(numel));
  auto result = std::make_tuple(make_memref<T, N>(y, x.sizes), make_memref<int8_t, N>(q, x.sizes));
  if (!y || !q) return result;
  NormParams p = norm_params<T, N>(x, residual.data, gamma.data, beta.data,
                                   static_cast<float>(at->get_float("eps", 1e-5)), 0);
  p.y = y;
  p.q_out = q;
  p.q_scale = q_scale.data;
  const char* detail = nullptr;
  const cudaError_t launch_st = norm_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "add_layernorm_quant", detail);
  return result;
}

template <typename T, int N>
MemRef<T, N> rmsnorm_call(ExecContext* ctx, void* stream_handle, MemRef<T, N> x, MemRef<T, 1> gamma,
                          void* custom_attrs) {
  if (memref_numel(x) == 0) return make_memref<T, N>(nullptr, x.sizes);
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<T, N>(nullptr, x.sizes);
  T* y = static_cast<T*>(ctx->alloc(static_cast<size_t>(memref_numel(x)) * sizeof(T)));
  auto result = make_memref<T, N>(y, x.sizes);
  if (!y) return result;
  NormParams p = norm_params<T, N>(x, nullptr, gamma.data, nullptr,
                                   static_cast<float>(at->get_float("eps", 1e-6)), 1);
  p.y = y;
  const char* detail = nullptr;
  const cudaError_t launch_st = norm_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "rmsnorm", detail);
  return result;
}

template <typename T, int N>
MemRef<T, N> softmax_impl(ExecContext* ctx, MemRef<T, N> x, const int32_t* lens, int64_t batches,
                          void* custom_attrs) {
  if (memref_numel(x) == 0) return make_memref<T, N>(nullptr, x.sizes);
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<T, N>(nullptr, x.sizes);
  T* y = static_cast<T*>(ctx->alloc(static_cast<size_t>(memref_numel(x)) * sizeof(T)));
  auto result = make_memref<T, N>(y, x.sizes);
  if (!y) return result;
  SoftmaxParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = x.data;
  p.y = y;
  p.cols = x.sizes[N - 1];
  p.rows = memref_numel(x) / p.cols;
  p.rows_per_batch = (lens && batches > 0) ? p.rows / batches : p.rows;
  p.lens = lens;
  p.scale = static_cast<float>(at->get_float("scale", 1.0));
  p.type = elem_type_of<T>();
  p.log_softmax = at->get_bool("log", false) ? 1 : 0;
  const char* detail = nullptr;
  const cudaError_t launch_st = softmax_launch(p, stream_of(ctx), &detail);
  report(ctx, launch_st, "softmax", detail);
  return result;
}

template <typename T, int N>
MemRef<T, N> softmax_call(ExecContext* ctx, void* stream_handle, MemRef<T, N> x, void* custom_attrs) {
  return softmax_impl<T, N>(ctx, x, nullptr, 0, custom_attrs);
}

// Rows of batch b (the leading axis) keep only their first lens[b] columns.
template <typename T, int N>
MemRef<T, N> masked_softmax_call(ExecContext* ctx, void* stream_handle, MemRef<T, N> x,
                                 MemRef<int32_t, 1> lens, void* custom_attrs) {
  if (lens.sizes[0] != x.sizes[0]) {
    ctx->signal_error("disc_b200_masked_softmax: one length per leading index expected");
    return make_memref<T, N>(nullptr, x.sizes);
  }
  return softmax_impl<T, N>(ctx, x, lens.data, x.sizes[0], custom_attrs);
}

#define DISC_B200_REGISTER_ROWOPS(T, N)                                                  \
  DISC_B200_RAL_API("disc_b200_quantize", "gpu", quantize_call<T, N>);                   \
  DISC_B200_RAL_API("disc_b200_dynamic_quantize", "gpu", dynamic_quantize_call<T, N>);   \
  DISC_B200_RAL_API("disc_b200_dequantize", "gpu", dequantize_call<T, N>);               \
  DISC_B200_RAL_API("disc_b200_layernorm", "gpu", layernorm_call<T, N>);                 \
  DISC_B200_RAL_API("disc_b200_add_layernorm", "gpu", add_layernorm_call<T, N>);         \
  DISC_B200_RAL_API("disc_b200_add_layernorm_quant", "gpu", add_layernorm_quant_call<T, N>); \
  DISC_B200_RAL_API("disc_b200_rmsnorm", "gpu", rmsnorm_call<T, N>);                     \
  DISC_B200_RAL_API("disc_b200_softmax", "gpu", softmax_call<T, N>)
DISC_B200_REGISTER_ROWOPS(float, 2);
DISC_B200_REGISTER_ROWOPS(float, 3);
DISC_B200_REGISTER_ROWOPS(f16_t, 2);
DISC_B200_REGISTER_ROWOPS(f16_t, 3);
DISC_B200_RAL_API("disc_b200_softmax", "gpu", softmax_call<float, 4>);
DISC_B200_RAL_API("disc_b200_softmax", "gpu", softmax_call<f16_t, 4>);
DISC_B200_RAL_API("disc_b200_masked_softmax", "gpu", masked_softmax_call<float, 4>);
DISC_B200_RAL_API("disc_b200_masked_softmax", "gpu", masked_softmax_call<f16_t, 4>);
DISC_B200_RAL_API("disc_b200_masked_softmax", "gpu", masked_softmax_call<float, 3>);
DISC_B200_RAL_API("disc_b200_masked_softmax", "gpu", masked_softmax_call<f16_t, 3>);


// ------------------------------------------------------- 4. collectives
// The column-parallel split of a linear over the GPUs of one box ends in an
// all-gather.  ral_all_gather / ral_all_reduce / ral_async_collective_done keep
// the reference's names, attributes and result ownership
// (tao_compiler/mlir/ral/collective.cu.cc:60-309,398-440, registered :444-504).
// Differences: a failure is recorded instead of ignored, a call that is not
// asynchronous runs on the compute stream (the reference issues it on the
// communication stream without ordering it behind the producer), bf16 is sent
// as bf16 (the reference maps it to ncclHalf, harmless for a gather and wrong
// for a sum).
template <typename T>
constexpr int nccl_type_of() {
  if constexpr (std::is_same_v<T, float>) return kNcclFloat32;
  if constexpr (std::is_same_v<T, f16_t>) return kNcclFloat16;
  if constexpr (std::is_same_v<T, bf16_t>) return kNcclBfloat16;
  if constexpr (std::is_same_v<T, int32_t>) return kNcclInt32;
  return kNcclInt8;
}

struct CollectiveEnv {
  const NcclApi* api = nullptr;
  void* comm = nullptr;
  cudaStream_t compute = nullptr;
  cudaStream_t comm_stream = nullptr;
  int size = 0;
  int rank = 0;
};

bool collective_env(ExecContext* ctx, CollectiveEnv* env) {
  int size = 0, rank = 0;
  if (!ctx->ctx->comm_info(&size, &rank)) return false;
  env->api = &nccl_api();
  env->comm = ctx->ctx->nccl_comm;
  env->compute = stream_of(ctx);
  env->comm_stream = ctx->ctx->comm_stream ? ctx->ctx->comm_stream : env->compute;
  env->size = size;
  env->rank = rank;
  return true;
}

// Makes `later` wait for everything queued on `earlier` so far.
bool order_streams(ExecContext* ctx, cudaStream_t earlier, cudaStream_t later) {
  if (earlier == later) return true;
  cudaEvent_t ev = nullptr;
  cudaError_t st = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  const bool created = st == cudaSuccess;
  if (st == cudaSuccess) st = cudaEventRecord(ev, earlier);
  if (st == cudaSuccess) st = cudaStreamWaitEvent(later, ev, 0);
  if (created) cudaEventDestroy(ev);  // the queued wait keeps what it needs
  if (st != cudaSuccess) {
    report(ctx, st, "stream ordering for a collective", nullptr);
    return false;
  }
  return true;
}

// Leaves an event on the communication stream under `key`;
// ral_async_collective_done makes the compute stream wait for it.
bool leave_token(ExecContext* ctx, const CollectiveEnv& env, int64_t key) {
  cudaEvent_t ev;
  cudaError_t st = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
  if (st == cudaSuccess) st = cudaEventRecord(ev, env.comm_stream);
  if (st != cudaSuccess) {
    report(ctx, st, "completion event of a collective", nullptr);
    return false;
  }
  auto it = ctx->async_tokens.find(key);
  if (it != ctx->async_tokens.end()) cudaEventDestroy(it->second);
  ctx->async_tokens[key] = ev;
  return true;
}

// Group size named by the replica_groups attribute ([groups, ranks per group]);
// the communicator's size when the attribute is absent.
int64_t group_size_of(const Attr* at, int comm_size) {
  const Attr* rg = at->find("replica_groups");
  if (rg && rg->kind == Attr::kDense && rg->shape.size() == 2) return rg->shape[1];
  return comm_size;
}

// in-place capable gather of `count` elements per rank on the stream the
// attributes select; returns false after recording the error.
bool run_all_gather(ExecContext* ctx, const CollectiveEnv& env, const Attr* at, const void* send,
                    void* recv, size_t count, int dtype) {
  const bool is_async = at->get_bool("is_async", false);
  cudaStream_t s = env.compute;
  if (is_async) {
    if (!order_streams(ctx, env.compute, env.comm_stream)) return false;
    s = env.comm_stream;
  }
  const int st = env.api->AllGather(send, recv, count, dtype, env.comm, s);
  if (st != 0) {
    ctx->signal_error("ncclAllGather failed: " + env.api->describe(st));
    return false;
  }
  if (is_async) return leave_token(ctx, env, at->get_int("async_token_key", 0));
  return true;
}

template <typename T, int N>
MemRef<T, N> ral_all_gather(ExecContext* ctx, void* stream_handle, MemRef<T, N> input,
                            void* custom_attrs) {
  int64_t sizes[N];
  for (int i = 0; i < N; ++i) sizes[i] = input.sizes[i];
  MemRef<T, N> none = make_memref<T, N>(nullptr, sizes);
  if (!check_stream_handle(ctx, stream_handle)) return none;
  const Attr* at = attrs_of(ctx, custom_attrs);
  CollectiveEnv env;
  if (!at || !collective_env(ctx, &env)) return none;
  const int64_t dim = at->get_int("all_gather_dim", 0);
  const int64_t group = group_size_of(at, env.size);
  if (dim < 0 || dim >= N) {
    ctx->signal_error("ral_all_gather: all_gather_dim out of range");
    return none;
  }
  if (group != env.size) {
    ctx->signal_error("ral_all_gather: replica group of " + std::to_string(group) +
                      " ranks but the communicator has " + std::to_string(env.size));
    return none;
  }
  // As in the reference the data arrives rank-major whatever the dimension:
  // the result holds rank 0's buffer, then rank 1's, ...
  sizes[dim] *= group;
  const int64_t count = memref_numel(input);
  if (count == 0) return make_memref<T, N>(nullptr, sizes);
  T* out = static_cast<T*>(ctx->alloc(static_cast<size_t>(count * group) * sizeof(T)));
  MemRef<T, N> result = make_memref<T, N>(out, sizes);
  if (!out) return result;
  run_all_gather(ctx, env, at, input.data, out, static_cast<size_t>(count), nccl_type_of<T>());
  return result;
}

int nccl_op_of(const std::string& kind) {
  if (kind == "prod") return kNcclProd;
  if (kind == "min") return kNcclMin;
  if (kind == "max") return kNcclMax;
  return kNcclSum;  // the reference's default for anything else (collective.cu.cc:52-58)
}

template <typename T, int N>
MemRef<T, N> ral_all_reduce(ExecContext* ctx, void* stream_handle, MemRef<T, N> input,
                            void* custom_attrs) {
  MemRef<T, N> result = input;
  result.base = result.data = nullptr;
  if (!check_stream_handle(ctx, stream_handle)) return result;
  const Attr* at = attrs_of(ctx, custom_attrs);
  CollectiveEnv env;
  if (!at || !collective_env(ctx, &env)) return result;
  const int64_t count = memref_numel(input);
  if (count == 0) return result;
  T* out = static_cast<T*>(ctx->alloc(static_cast<size_t>(count) * sizeof(T)));
  if (!out) return result;
  result.base = result.data = out;
  result.offset = 0;
  if constexpr (N > 0) {
    int64_t stride = 1;
    for (int i = N - 1; i >= 0; --i) {
      result.strides[i] = stride;
      stride *= result.sizes[i];
    }
  }
  const bool is_async = at->get_bool("is_async", false);
  cudaStream_t s = env.compute;
  if (is_async) {
    if (!order_streams(ctx, env.compute, env.comm_stream)) return result;
    s = env.comm_stream;
  }
  const int st = env.api->AllReduce(input.data, out, static_cast<size_t>(count), nccl_type_of<T>(),
                                    nccl_op_of(at->get_str("reduction_kind", "sum")), env.comm, s);
  if (st != 0) {
    ctx->signal_error("ncclAllReduce failed: " + env.api->describe(st));
    return result;
  }
  if (is_async) leave_token(ctx, env, at->get_int("async_token_key", 0));
  return result;
}

// The consumer side of an asynchronous collective: the compute stream waits for
// the event the collective left; the buffer passes through with one more
// reference, as in the reference (collective.cu.cc:411-416), so that the
// dealloc of the collective's own result does not free what this call returns.
template <typename T, int N>
MemRef<T, N> ral_async_collective_done(ExecContext* ctx, void* stream_handle, MemRef<T, N> input,
                                       void* custom_attrs) {
  if (!check_stream_handle(ctx, stream_handle)) return input;
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return input;
  auto rc = ctx->refcount.find(input.data);
  if (rc != ctx->refcount.end()) ++rc->second;
  if (!at->get_bool("is_async", false)) return input;
  const int64_t key = at->get_int("async_token_key", 0);
  auto it = ctx->async_tokens.find(key);
  if (it == ctx->async_tokens.end()) {
    ctx->signal_error("ral_async_collective_done: no collective in flight under token " +
                      std::to_string(key));
    return input;
  }
  report(ctx, cudaStreamWaitEvent(stream_of(ctx), it->second, 0), "wait for a collective", nullptr);
  cudaEventDestroy(it->second);
  ctx->async_tokens.erase(it);
  return input;
}

#define DISC_B200_REGISTER_COLLECTIVES(T)                                              \
  DISC_B200_RAL_API("ral_all_reduce", "gpu", ral_all_reduce<T, 0>);                    \
  DISC_B200_RAL_API("ral_all_reduce", "gpu", ral_all_reduce<T, 1>);                    \
  DISC_B200_RAL_API("ral_all_reduce", "gpu", ral_all_reduce<T, 2>);                    \
  DISC_B200_RAL_API("ral_all_reduce", "gpu", ral_all_reduce<T, 3>);                    \
  DISC_B200_RAL_API("ral_all_reduce", "gpu", ral_all_reduce<T, 4>);                    \
  DISC_B200_RAL_API("ral_all_gather", "gpu", ral_all_gather<T, 1>);                    \
  DISC_B200_RAL_API("ral_all_gather", "gpu", ral_all_gather<T, 2>);                    \
  DISC_B200_RAL_API("ral_all_gather", "gpu", ral_all_gather<T, 3>);                    \
  DISC_B200_RAL_API("ral_all_gather", "gpu", ral_all_gather<T, 4>);                    \
  DISC_B200_RAL_API("ral_async_collective_done", "gpu", ral_async_collective_done<T, 0>); \
  DISC_B200_RAL_API("ral_async_collective_done", "gpu", ral_async_collective_done<T, 1>); \
  DISC_B200_RAL_API("ral_async_collective_done", "gpu", ral_async_collective_done<T, 2>); \
  DISC_B200_RAL_API("ral_async_collective_done", "gpu", ral_async_collective_done<T, 3>); \
  DISC_B200_RAL_API("ral_async_collective_done", "gpu", ral_async_collective_done<T, 4>)
DISC_B200_REGISTER_COLLECTIVES(float);
DISC_B200_REGISTER_COLLECTIVES(f16_t);
DISC_B200_REGISTER_COLLECTIVES(bf16_t);
// int8 results of the fused call below travel through the same "done" call.
DISC_B200_RAL_API("ral_async_collective_done", "gpu", ral_async_collective_done<int8_t, 3>);

// One column-parallel shard of a quantized linear and its all-gather in one
// call.  Rank r holds rows [r * N/g, (r + 1) * N/g) of the weight with their
// scales and bias; its GEMM epilogue writes straight into slot r of the result
// [g, M, N/g] and NCCL gathers in place (send buffer = slot r of the receive
// buffer), so no copy sits between the kernel and the collective.  The result
// keeps the rank-major layout the gather produces; the next linear reads it as
// its activation without a re-layout (input rank 3 here = such a buffer).
// Attributes: activation, and is_async / async_token_key as for ral_all_gather
// (asynchronous: the gather runs on the communication stream and overlaps the
// caller's next independent kernels until ral_async_collective_done).
template <int NIN, typename OutT, typename XS>
MemRef<OutT, 3> qgemm_all_gather(ExecContext* ctx, void* stream_handle, MemRef<int8_t, NIN> input,
                                 MemRef<int8_t, 2> weight, MemRef<float, 1> bias, XS x_scale,
                                 MemRef<float, 1> w_scale, MemRef<float, 0> out_scale,
                                 void* custom_attrs) {
  static_assert(NIN == 2 || NIN == 3, "row-major [M, K] or gathered [g, M, K / g]");
  const int64_t k = weight.sizes[1];
  const int64_t n_local = weight.sizes[0];
  const int64_t m = input.sizes[NIN - 2];
  int64_t rs[3] = {0, m, n_local};
  if (!check_stream_handle(ctx, stream_handle)) return make_memref<OutT, 3>(nullptr, rs);
  const Attr* at = attrs_of(ctx, custom_attrs);
  CollectiveEnv env;
  if (!at || !collective_env(ctx, &env)) return make_memref<OutT, 3>(nullptr, rs);
  rs[0] = env.size;
  const int64_t k_in = NIN == 2 ? input.sizes[1] : input.sizes[0] * input.sizes[2];
  if (k_in != k || w_scale.sizes[0] != n_local) {
    ctx->signal_error("disc_b200_qgemm_all_gather: operand extents disagree");
    return make_memref<OutT, 3>(nullptr, rs);
  }
  if (m == 0 || n_local == 0 || k == 0) return make_memref<OutT, 3>(nullptr, rs);
  const int64_t slot = m * n_local;
  OutT* out = static_cast<OutT*>(ctx->alloc(static_cast<size_t>(slot * env.size) * sizeof(OutT)));
  auto result = make_memref<OutT, 3>(out, rs);
  if (!out) return result;
  OutT* mine = out + slot * env.rank;
  QGemmParams p = base_params(input.data, weight.data, mine, m, n_local, k);
  if constexpr (NIN == 3) {
    p.a_slabs = static_cast<int>(input.sizes[0]);
    p.a_slab_cols = input.sizes[2];
    p.a_slab_stride = input.sizes[1] * input.sizes[2];
    p.lda = input.sizes[2];
  }
  p.x_scale = x_scale.data;
  p.x_scale_kind = std::is_same_v<XS, MemRef<float, 0>> ? kScaleScalar : kScalePerRow;
  p.w_scale = w_scale.data;
  p.w_scale_kind = kScalePerCol;
  p.bias = memref_numel(bias) == n_local ? bias.data : nullptr;
  p.bias_kind = p.bias ? kBiasF32 : kBiasNone;
  p.act = act_from(at);
  if constexpr (std::is_same_v<OutT, int8_t>) {
    p.out_scale = out_scale.data;
    p.out_scale_kind = kScaleScalar;
    p.div_out_scale = 1;
    p.div_exact = at->get_bool("exact_division", false) ? 1 : 0;
    p.out_dtype = kOutI8;
  } else {
    p.out_dtype = kOutF16;
  }
  if (!run_qgemm(ctx, p)) return result;
  // bytes, so that int8 and f16 results share one code path
  run_all_gather(ctx, env, at, mine, out, static_cast<size_t>(slot) * sizeof(OutT), kNcclInt8);
  return result;
}

#define DISC_B200_REGISTER_QGEMM_AG(NIN)                                                        \
  DISC_B200_RAL_API("disc_b200_qgemm_all_gather", "gpu", qgemm_all_gather<NIN, f16_t, MemRef<float, 0>>);  \
  DISC_B200_RAL_API("disc_b200_qgemm_all_gather", "gpu", qgemm_all_gather<NIN, f16_t, MemRef<float, 1>>);  \
  DISC_B200_RAL_API("disc_b200_qgemm_all_gather", "gpu", qgemm_all_gather<NIN, int8_t, MemRef<float, 0>>); \
  DISC_B200_RAL_API("disc_b200_qgemm_all_gather", "gpu", qgemm_all_gather<NIN, int8_t, MemRef<float, 1>>)
DISC_B200_REGISTER_QGEMM_AG(2);
DISC_B200_REGISTER_QGEMM_AG(3);


// --------------------------------------------------------- 5. constants
// ral_const: the constants of the compiled graph (for the quantized path the
// int8 weights, scale vectors and biases) by unique name, decoded from the
// metadata file on first use; device constants are uploaded once and live as
// long as the context.  Reference: ral_base_cuda_const_host / _cuda
// (tao_compiler/mlir/ral/context/common_context_impl.cc:279-420,
// common_context_impl_cuda.cc:61-200), both registered as "ral_const".
template <typename T, int N, bool kDevice>
MemRef<T, N> ral_const(ExecContext* ctx, void* stream_handle, const char* unique_name,
                       int32_t unique_index_in_module) {
  int64_t zeros[N > 0 ? N : 1] = {0};
  MemRef<T, N> none = make_memref<T, N>(nullptr, zeros);
  const ConstEntry* e = ctx->ctx->get_const(kDevice, unique_name, unique_index_in_module);
  if (!e) return none;
  if (static_cast<int>(e->shape.size()) != N) {
    ctx->signal_error("unexpected shape string in unique_name");
    return none;
  }
  return make_memref<T, N>(static_cast<T*>(e->ptr), e->shape.data());
}

#define DISC_B200_REGISTER_CONST(T, N)                                   \
  DISC_B200_RAL_API("ral_const", "cpu", ral_const<T, N, false>);          \
  DISC_B200_RAL_API("ral_const", "gpu", ral_const<T, N, true>)
// ranks 0..8 and the element types the reference instantiates
// (common_context_impl.cc:392-480 and :985-1000, common_context_impl_cuda.cc:177-290)
#define DISC_B200_REGISTER_CONST_RANKS(T) \
  DISC_B200_REGISTER_CONST(T, 0);         \
  DISC_B200_REGISTER_CONST(T, 1);         \
  DISC_B200_REGISTER_CONST(T, 2);         \
  DISC_B200_REGISTER_CONST(T, 3);         \
  DISC_B200_REGISTER_CONST(T, 4);         \
  DISC_B200_REGISTER_CONST(T, 5);         \
  DISC_B200_REGISTER_CONST(T, 6);         \
  DISC_B200_REGISTER_CONST(T, 7);         \
  DISC_B200_REGISTER_CONST(T, 8)
DISC_B200_REGISTER_CONST_RANKS(double);
DISC_B200_REGISTER_CONST_RANKS(float);
DISC_B200_REGISTER_CONST_RANKS(f16_t);
DISC_B200_REGISTER_CONST_RANKS(bf16_t);
DISC_B200_REGISTER_CONST_RANKS(int8_t);
DISC_B200_REGISTER_CONST_RANKS(uint8_t);
DISC_B200_REGISTER_CONST_RANKS(int16_t);
DISC_B200_REGISTER_CONST_RANKS(uint16_t);
DISC_B200_REGISTER_CONST_RANKS(int32_t);
DISC_B200_REGISTER_CONST_RANKS(uint32_t);
DISC_B200_REGISTER_CONST_RANKS(int64_t);
DISC_B200_REGISTER_CONST_RANKS(bool);


// ------------------------------------------------- 6. weight-only qgemm
// ral_pdll_weight_only_qgemm(input, weight [K, N] ui8, [bias,] weight_scale [N],
// weight_zero_point [N]) -> input @ ((weight - zp) * scale) [+ bias]: the call the
// pattern pytorch_blade/tests/disc/pdl/pdll_files/gpu/weight_only_qgemm.pdll:2-106
// emits (operand order :27 and :90); f16 is what the reference's weight pass
// expects, f32 what its front-end test produces
// (test_torchscipt_to_mhlo/test_quantization.py:501-618).  The weights are used
// as the pattern leaves them.  weight_should_be_reordered = false means the
// compiler has already permuted them for its sm_75/80 kernel
// (disc_transform_weight_data_layout_for_weight_only_gemm.cc): that layout is
// refused, the pass has to stay off for this runtime.
template <typename T, int N, bool kBias>
MemRef<T, N> weight_only_qgemm_impl(ExecContext* ctx, void* stream_handle, MemRef<T, N> input,
                                    MemRef<uint8_t, 2> weight, const T* bias, int64_t bias_len,
                                    MemRef<T, 1> scale, MemRef<int32_t, 1> zp, void* custom_attrs) {
  static_assert(N == 2 || N == 3, "rank 2 or 3 input");
  int64_t rs[N];
  int64_t m = 1;
  for (int i = 0; i < N - 1; ++i) {
    rs[i] = input.sizes[i];
    m *= input.sizes[i];
  }
  const int64_t k = weight.sizes[0];
  const int64_t n = weight.sizes[1];
  rs[N - 1] = n;
  if (!check_stream_handle(ctx, stream_handle)) return make_memref<T, N>(nullptr, rs);
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return make_memref<T, N>(nullptr, rs);
  if (!at->get_bool("weight_should_be_reordered", true)) {
    ctx->signal_error(
        "ral_pdll_weight_only_qgemm: weights already permuted by the compiler's weight-layout pass are not "
        "supported; keep weight_should_be_reordered = true (plain [K, N] weights)");
    return make_memref<T, N>(nullptr, rs);
  }
  if (input.sizes[N - 1] != k || scale.sizes[0] != n || zp.sizes[0] != n || (kBias && bias_len != n)) {
    ctx->signal_error("ral_pdll_weight_only_qgemm: operand extents disagree");
    return make_memref<T, N>(nullptr, rs);
  }
  if (m == 0 || n == 0) return make_memref<T, N>(nullptr, rs);
  T* out = static_cast<T*>(ctx->alloc(static_cast<size_t>(m * n) * sizeof(T)));
  auto result = make_memref<T, N>(out, rs);
  if (!out) return result;
  WoqGemmParams p;
  std::memset(&p, 0, sizeof(p));
  p.x = input.data;
  p.w = weight.data;
  p.scale = scale.data;
  p.zp = zp.data;
  p.bias = kBias ? bias : nullptr;
  p.out = out;
  p.M = m;
  p.N = n;
  p.K = k;
  p.ldx = k;
  p.ldw = n;
  p.ldo = n;
  p.type = std::is_same_v<T, float> ? kF32 : kF16;
  const char* detail = nullptr;
  const cudaError_t st = woq_gemm_launch(p, stream_of(ctx), &detail);
  if (st != cudaSuccess) report(ctx, st, "ral_pdll_weight_only_qgemm", detail);
  return result;
}
template <typename T, int N>
MemRef<T, N> weight_only_qgemm(ExecContext* ctx, void* stream_handle, MemRef<T, N> input,
                               MemRef<uint8_t, 2> weight, MemRef<T, 1> scale, MemRef<int32_t, 1> zp,
                               void* custom_attrs) {
  return weight_only_qgemm_impl<T, N, false>(ctx, stream_handle, input, weight, nullptr, 0, scale, zp, custom_attrs);
}
template <typename T, int N>
MemRef<T, N> weight_only_qgemm_bias(ExecContext* ctx, void* stream_handle, MemRef<T, N> input,
                                    MemRef<uint8_t, 2> weight, MemRef<T, 1> bias, MemRef<T, 1> scale,
                                    MemRef<int32_t, 1> zp, void* custom_attrs) {
  return weight_only_qgemm_impl<T, N, true>(ctx, stream_handle, input, weight, bias.data, bias.sizes[0], scale, zp,
                                            custom_attrs);
}
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm<f16_t, 2>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm<f16_t, 3>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm<float, 2>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm<float, 3>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm_bias<f16_t, 2>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm_bias<f16_t, 3>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm_bias<float, 2>);
DISC_B200_RAL_API("ral_pdll_weight_only_qgemm", "gpu", weight_only_qgemm_bias<float, 3>);


// ------------------------------------------------------ 7. quantized conv
// Runs the convolution described by `geo` into `out` (device, preallocated).
bool run_qconv(ExecContext* ctx, const ConvGeometry& geo, const int8_t* x, const int8_t* w, int8_t* out,
               const float* x_scale, const float* w_scale, bool per_channel, const float* out_scale,
               const char* what) {
  QConvParams p;
  p.g = geo;
  p.x = x;
  p.w = w;
  p.out = out;
  p.x_scale = x_scale;
  p.w_scale = w_scale;
  p.w_scale_per_channel = per_channel ? 1 : 0;
  p.out_scale = out_scale;
  p.workspace_bytes = qconv_workspace_bytes(geo);
  p.workspace = ctx->alloc(static_cast<size_t>(p.workspace_bytes));
  if (!p.workspace) return false;
  p.splitk_ws = nullptr;
  p.splitk_ws_bytes = 0;
  const int64_t rows = geo.batch * geo.out_h * geo.out_w;
  if (rows <= 128) {
    const int64_t kp = (geo.k_h * geo.k_w * geo.in_ch + 15) / 16 * 16;
    int64_t have = 0;
    p.splitk_ws = static_cast<int32_t*>(ctx->ctx->get_splitk_ws(qgemm_splitk_ws_bytes(rows, geo.out_ch, kp), &have));
    p.splitk_ws_bytes = p.splitk_ws ? have : 0;
  }
  const char* detail = nullptr;
  const cudaError_t st = qconv_launch(p, stream_of(ctx), &detail);
  // the allocator hands the block out again only to work queued behind these kernels
  ctx->dealloc(p.workspace);
  if (st != cudaSuccess) {
    report(ctx, st, what, detail);
    return false;
  }
  return true;
}

// ral_qconv on "gpu" with the reference's operands
// (tao_compiler/mlir/ral/context/stream_executor_based_impl.cc:1832-1950): output
// preallocated by the caller, padding and metadata in host memory, scales on the
// device.  Like the reference it uses one weight scale (the first) and ignores the
// zero points; unlike it, nothing is read back to the host.
void ral_qconv(ExecContext* ctx, void* stream_handle, MemRef<int8_t, 4> input, MemRef<int8_t, 4> kernel,
               MemRef<int32_t, 1> padding, MemRef<float, 0> input_scale, MemRef<int32_t, 0> input_zp,
               MemRef<float, 1> weight_scale, MemRef<int32_t, 1> weight_zp, MemRef<float, 0> result_scale,
               MemRef<int32_t, 0> result_zp, MemRef<int8_t, 4> output, MemRef<int32_t, 1> metadata) {
  if (!check_stream_handle(ctx, stream_handle)) return;
  if (memref_numel(input) == 0 || memref_numel(kernel) == 0 || memref_numel(output) == 0) return;
  if (padding.sizes[0] != 4 || !padding.data || !metadata.data) {
    ctx->signal_error("ral_qconv: invalid conv params");
    return;
  }
  ConvGeometry geo;
  const std::string why = conv2d_geometry(input.sizes, kernel.sizes, output.sizes, padding.data, metadata.data,
                                          metadata.sizes[0], &geo);
  if (!why.empty()) {
    ctx->signal_error("ral_qconv: " + why);
    return;
  }
  run_qconv(ctx, geo, input.data, kernel.data, output.data, input_scale.data, weight_scale.data, false,
            result_scale.data, "ral_qconv");
}
DISC_B200_RAL_API("ral_qconv", "gpu", ral_qconv);

// ral_pdll_qconv2d with the operands and attributes of the reference's pattern
// (tao_compiler/mlir/disc/tests/pdll/data/quantized_conv2d_i8.pdll; implementation
// for aarch64 hosts: common_context_impl_quantization.cc:363-607): kernel
// [out, y, x, in], per-channel weight scales, attributes data_format / strides /
// dilations / padding / explicit_paddings / weight_is_const; the result is
// allocated here.  The reference registers it on "cpu" only; this is the same
// call for device tensors.
MemRef<int8_t, 4> pdll_qconv2d(ExecContext* ctx, void* stream_handle, MemRef<int8_t, 4> input,
                               MemRef<int8_t, 4> weight, MemRef<float, 0> input_scale,
                               MemRef<int32_t, 0> input_zp, MemRef<float, 1> weight_scale,
                               MemRef<int32_t, 1> weight_zp, MemRef<float, 0> result_scale,
                               MemRef<int32_t, 0> result_zp, void* custom_attrs) {
  int64_t zeros[4] = {0, 0, 0, 0};
  auto none = make_memref<int8_t, 4>(nullptr, zeros);
  if (!check_stream_handle(ctx, stream_handle)) return none;
  if (memref_numel(input) == 0 || memref_numel(weight) == 0) return none;
  const Attr* at = attrs_of(ctx, custom_attrs);
  if (!at) return none;
  auto ints = [&](const char* key) {
    const Attr* a = at->find(key);
    return a && a->kind == Attr::kIntArray ? a->ints : std::vector<int64_t>();
  };
  int32_t padding[4];
  int32_t metadata[17];
  int64_t result_sizes[4];
  const std::string why = plan_conv2d_from_attrs(at->get_str("data_format", "NHWC"), ints("strides"), ints("dilations"),
                                                 at->get_str("padding", ""), ints("explicit_paddings"),
                                                 at->get_bool("weight_is_const", false), input.sizes, weight.sizes,
                                                 padding, result_sizes, metadata);
  if (!why.empty()) {
    ctx->signal_error("ral_pdll_qconv2d: " + why);
    return none;
  }
  ConvGeometry geo;
  const std::string bad = conv2d_geometry(input.sizes, weight.sizes, result_sizes, padding, metadata, 17, &geo);
  if (!bad.empty()) {
    ctx->signal_error("ral_pdll_qconv2d: " + bad);
    return none;
  }
  if (weight_scale.sizes[0] != geo.out_ch && weight_scale.sizes[0] != 1) {
    ctx->signal_error("ral_pdll_qconv2d: one weight scale per output channel (or one in all) expected");
    return none;
  }
  int64_t total = 1;
  for (int i = 0; i < 4; ++i) total *= result_sizes[i];
  if (total == 0) return make_memref<int8_t, 4>(nullptr, result_sizes);
  int8_t* out = static_cast<int8_t*>(ctx->alloc(static_cast<size_t>(total)));
  auto result = make_memref<int8_t, 4>(out, result_sizes);
  if (!out) return result;
  run_qconv(ctx, geo, input.data, weight.data, out, input_scale.data, weight_scale.data,
            weight_scale.sizes[0] == geo.out_ch && geo.out_ch > 1, result_scale.data, "ral_pdll_qconv2d");
  return result;
}
DISC_B200_RAL_API("ral_pdll_qconv2d", "gpu", pdll_qconv2d);

}  // namespace
}  // namespace ral
}  // namespace disc_b200

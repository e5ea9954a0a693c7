// TEST INFRASTRUCTURE.  Linked with the reference's own host runtime
// (ral_api.cc, ral_context.cc, ral_helper.cc, ral_logging.cc, ral_metadata.cc,
// context/common_context_impl.cc, context/base/base_context.cc,
// context/base/cpu/cpu_context_impl.cc, device/cpu/cpu_driver.cc -- compiled from
// the reference tree where it lies, with the two stand-in headers under stubs/)
// into oracle/_ref/libref_host.so.
//
// It runs a compiled executable (a shared object with the entry point "main") on
// the reference's BaseCpuContext the way torch_blade's RalContext::Execute does
// (pytorch_blade/pytorch_blade/compiler/mlir/runtime/ral_context.cpp:293-321), so
// that the tests can run one and the same program on the reference runtime and
// on this repository's and compare what comes out.
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "mlir/ral/context/base/cpu/cpu_context_impl.h"
#include "mlir/ral/context/common_context_impl_quantization.h"
#include "mlir/ral/ral_api.h"
#include "mlir/ral/ral_context.h"

extern "C" {

// Inputs: n_in buffers with rank and sizes (8 slots each).  Outputs: n_out buffers of
// capacity out_caps[i] bytes to copy into, element width out_elem_bytes[i]; receives rank,
// sizes (8 slots each), whether the runtime handed the buffer over as owned, and whether
// the output is the very buffer of input 0..n_in-1 (index) or not (-1).
// Returns 0, or a negative code with a message in err.
int ref_host_run(const char* so_path, const char* metadata_path, int n_in, const void* const* in_data,
                 const int32_t* in_rank, const int64_t* in_sizes8, int n_out, void* const* out_bufs,
                 const int64_t* out_caps, const int32_t* out_elem_bytes, int32_t* out_rank, int64_t* out_sizes8,
                 int32_t* out_owned, int32_t* out_alias_of_input, char* err, int err_cap) {
  auto fail = [&](int code, const std::string& why) {
    if (err && err_cap > 0) {
      std::strncpy(err, why.c_str(), err_cap - 1);
      err[err_cap - 1] = 0;
    }
    return code;
  };
  void* lib = dlopen(so_path, RTLD_NOW | RTLD_LOCAL);
  if (!lib) return fail(-1, std::string("dlopen: ") + dlerror());
  auto entry = reinterpret_cast<void (*)(void**)>(dlsym(lib, kMlirLoweredEntry));
  if (!entry) {
    dlclose(lib);
    return fail(-2, "no entry point");
  }
  int rc = 0;
  {
    tao::ral::BaseContextOption opt;
    opt.metadata_file_path = metadata_path ? metadata_path : "";
    opt.cache_workspace_mem_across_execution = true;
    tao::ral::cpu::BaseCpuContextOption cpu_opt;
    std::unique_ptr<tao::ral::BaseContext> ctx = tao::ral::cpu::MakeBaseCpuContext(opt, cpu_opt);
    {
      auto exec = tao::ral::MakeExecutionContext<tao::ral::cpu::BaseCpuExecutionContext>(ctx.get());
      for (int i = 0; i < n_in; ++i) {
        std::vector<int64_t> shape(in_sizes8 + 8 * i, in_sizes8 + 8 * i + in_rank[i]);
        exec->bindInput(i, const_cast<void*>(in_data[i]), shape);
      }
      void* ctx_struct[] = {exec.get(), reinterpret_cast<void*>(&tao_ral_call_impl)};
      entry(ctx_struct);
      const char* msg = nullptr;
      if (ctx->getLastError(&msg) != 0) {
        rc = fail(-3, msg ? msg : "error");
      } else {
        for (int i = 0; i < n_out && rc == 0; ++i) {
          std::unique_ptr<tao::ral::OutputBufferWrapper> out;
          exec->bindOutput(i, &out);
          if (ctx->getLastError(&msg) != 0 || !out) {
            rc = fail(-4, msg ? msg : "output not found");
            break;
          }
          const auto& shape = out->shape();
          int64_t n = 1;
          out_rank[i] = static_cast<int32_t>(shape.size());
          for (size_t d = 0; d < shape.size() && d < 8; ++d) {
            out_sizes8[8 * i + d] = shape[d];
            n *= shape[d];
          }
          const int64_t bytes = n * out_elem_bytes[i];
          if (bytes > out_caps[i]) {
            rc = fail(-5, "output buffer too small");
            break;
          }
          std::memcpy(out_bufs[i], out->data(), static_cast<size_t>(bytes));
          out_owned[i] = out->owned() ? 1 : 0;
          out_alias_of_input[i] = -1;
          for (int k = 0; k < n_in; ++k) {
            if (out->data() == in_data[k]) out_alias_of_input[i] = k;
          }
        }
      }
    }
  }
  dlclose(lib);
  return rc;
}

// One constant through the reference's own ral_const on "cpu" (ral_base_cuda_const_host,
// context/common_context_impl.cc:279-380): `call` is the full mangled name for the element type
// and rank.  Copies the bytes into out (capacity cap) and the sizes into sizes8.
int ref_host_const(const char* metadata_path, const char* call, const char* unique_name, int32_t index, int rank,
                   int elem_bytes, void* out, int64_t cap, int64_t* sizes8, char* err, int err_cap) {
  auto fail = [&](int code, const std::string& why) {
    if (err && err_cap > 0) {
      std::strncpy(err, why.c_str(), err_cap - 1);
      err[err_cap - 1] = 0;
    }
    return code;
  };
  tao::ral::BaseContextOption opt;
  opt.metadata_file_path = metadata_path;
  tao::ral::cpu::BaseCpuContextOption cpu_opt;
  std::unique_ptr<tao::ral::BaseContext> ctx = tao::ral::cpu::MakeBaseCpuContext(opt, cpu_opt);
  auto exec = tao::ral::MakeExecutionContext<tao::ral::cpu::BaseCpuExecutionContext>(ctx.get());
  void* ctx_slot = exec.get();
  void* stream = nullptr;
  const char* name = unique_name;
  int64_t result[3 + 2 * 8] = {0};  // base, data, offset, sizes, strides of a rank <= 8 memref
  void* args[5] = {&ctx_slot, &stream, &name, &index, result};
  std::string mangled(call);
  tao_ral_call_impl(exec.get(), const_cast<char*>(mangled.c_str()), args);
  const char* msg = nullptr;
  if (ctx->getLastError(&msg) != 0) return fail(-3, msg ? msg : "error");
  int64_t n = 1;
  for (int d = 0; d < rank; ++d) {
    sizes8[d] = result[3 + d];
    n *= result[3 + d];
  }
  if (n * elem_bytes > cap) return fail(-5, "output buffer too small");
  std::memcpy(out, reinterpret_cast<void*>(result[1]), static_cast<size_t>(n * elem_bytes));
  return 0;
}

// The reference's own rules for a convolution's geometry from the attributes of
// ral_pdll_qconv2d (context/common_context_impl_quantization.h:45-215), called exactly as
// ral_pdll_qconv_acl_s8_s8_s8_per_channel calls them (common_context_impl_quantization.cc:393-440).
// Returns 0, or the number of the step that refused the attributes.
int ref_conv_plan(const char* data_format, const int64_t* strides, int n_strides, const int64_t* dilations,
                  int n_dilations, const char* padding_str, const int64_t* explicit_paddings, int n_explicit,
                  int weight_is_const, const int64_t* input_sizes4, const int64_t* weight_sizes4,
                  int32_t* padding_out4, int64_t* result_sizes4, int32_t* metadata_out17) {
  using namespace tao::ral;
  constexpr int NDims = 4;
  MemRefType<int8_t, NDims> input, weight;
  for (int i = 0; i < NDims; ++i) {
    input.sizes[i] = input_sizes4[i];
    weight.sizes[i] = weight_sizes4[i];
  }
  std::vector<int32_t> reorderDims(NDims, 0);
  if (!generateReorderDims<NDims>(data_format, reorderDims)) return 1;
  std::vector<int32_t> st(NDims - 2, 0), dl(NDims - 2, 0);
  if (!generateStrides<NDims>(reorderDims, std::vector<int64_t>(strides, strides + n_strides), st)) return 2;
  if (!generateDilations<NDims>(reorderDims, std::vector<int64_t>(dilations, dilations + n_dilations), dl)) return 3;
  MemRefType<int32_t, 1> padding;
  padding.sizes[0] = (NDims - 2) * 2;
  padding.data = padding_out4;
  for (int i = 0; i < 4; ++i) padding_out4[i] = 0;
  if (std::string(padding_str) == "EXPLICIT") {
    if (!generateExplicitPaddings<NDims>(reorderDims,
                                         std::vector<int64_t>(explicit_paddings, explicit_paddings + n_explicit),
                                         padding))
      return 4;
  } else if (!generatePadding<NDims>(input, weight, padding_str, reorderDims, st, dl, padding)) {
    return 5;
  }
  MemRefType<int32_t, 1> metadata;
  metadata.sizes[0] = NDims * 3 + (NDims - 2) * 2 + 1;
  metadata.data = metadata_out17;
  if (!generateMetadata<NDims>(st, dl, reorderDims, weight_is_const != 0, metadata)) return 6;
  std::vector<int64_t> result(NDims, 0);
  generateResultShape<NDims>(input, weight, reorderDims, padding, st, dl, result);
  for (int i = 0; i < NDims; ++i) result_sizes4[i] = result[i];
  return 0;
}

}  // extern "C"

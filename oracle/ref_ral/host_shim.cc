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

}  // extern "C"

// The few CUDA driver entry points that launching a compiler-generated kernel
// needs (module load, function lookup, launch), reached through dlopen of
// libcuda.so.1: the library then links against the runtime only and still
// loads on a host without a driver (the registry, the metadata reader and the
// host-side calls work there).
// Reference call sites: tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc:348-445.
#pragma once
#include <cstddef>
#include <string>

namespace disc_b200 {
namespace ral {

struct CuDriverApi {
  bool ok = false;
  std::string error;  // why the binding failed

  int (*ModuleLoadData)(void** module, const void* image) = nullptr;
  int (*ModuleUnload)(void* module) = nullptr;
  int (*ModuleGetFunction)(void** function, void* module, const char* name) = nullptr;
  int (*FuncSetAttribute)(void* function, int attribute, int value) = nullptr;
  int (*LaunchKernel)(void* function, unsigned gx, unsigned gy, unsigned gz, unsigned bx, unsigned by,
                      unsigned bz, unsigned smem, void* stream, void** params, void** extra) = nullptr;
  int (*GetErrorString)(int result, const char** str) = nullptr;

  std::string describe(int result) const;
};

// CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES (public driver API value)
constexpr int kCuFuncAttrMaxDynamicShared = 8;

// Binds on first use; never throws.
const CuDriverApi& cu_driver_api();

// Index of the blob to load out of the `num_blobs` images the compiler embedded.
// The compiler emits either one image, or a PTX-bearing image (compute_60) at 0
// followed by cubins in the fixed order sm_70, sm_75, sm_80, sm_86
// (tao_compiler/mlir/ral/context/common_context_impl.cc:209-215, selection at
// cuda_context_impl.cc:375-395); a device that is not in that list,
// every Blackwell part among them, takes image 0 and lets the driver compile
// its PTX.  -1 if num_blobs is 0.
int select_blob(size_t num_blobs, int cc_major, int cc_minor);

}  // namespace ral
}  // namespace disc_b200

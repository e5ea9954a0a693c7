#include "cu_driver_dyn.h"

#include <dlfcn.h>

#include <mutex>

namespace disc_b200 {
namespace ral {
namespace {

template <typename Fn>
bool bind(void* lib, const char* name, Fn* out, std::string* err) {
  void* sym = dlsym(lib, name);
  if (!sym) {
    *err = std::string("CUDA driver symbol missing: ") + name;
    return false;
  }
  *out = reinterpret_cast<Fn>(sym);
  return true;
}

CuDriverApi load() {
  CuDriverApi api;
  void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_NOLOAD);  // the copy the runtime already mapped
  if (!lib) lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    const char* e = dlerror();
    api.error = std::string("libcuda.so.1 not found: ") + (e ? e : "");
    return api;
  }
  if (!bind(lib, "cuModuleLoadData", &api.ModuleLoadData, &api.error) ||
      !bind(lib, "cuModuleUnload", &api.ModuleUnload, &api.error) ||
      !bind(lib, "cuModuleGetFunction", &api.ModuleGetFunction, &api.error) ||
      !bind(lib, "cuFuncSetAttribute", &api.FuncSetAttribute, &api.error) ||
      !bind(lib, "cuLaunchKernel", &api.LaunchKernel, &api.error) ||
      !bind(lib, "cuGetErrorString", &api.GetErrorString, &api.error)) {
    return api;
  }
  api.ok = true;
  return api;
}

}  // namespace

std::string CuDriverApi::describe(int result) const {
  const char* s = nullptr;
  if (GetErrorString && GetErrorString(result, &s) == 0 && s) return s;
  return "CUDA driver error " + std::to_string(result);
}

const CuDriverApi& cu_driver_api() {
  static CuDriverApi api;
  static std::once_flag once;
  std::call_once(once, [] { api = load(); });
  return api;
}

int select_blob(size_t num_blobs, int cc_major, int cc_minor) {
  if (num_blobs == 0) return -1;
  if (num_blobs == 1) return 0;
  static const struct {
    int major, minor;
    size_t index;
  } kOrder[] = {{7, 0, 1}, {7, 5, 2}, {8, 0, 3}, {8, 6, 4}};
  for (const auto& e : kOrder) {
    if (e.major == cc_major && e.minor == cc_minor) return e.index <= num_blobs - 1 ? static_cast<int>(e.index) : 0;
  }
  return 0;
}

}  // namespace ral
}  // namespace disc_b200

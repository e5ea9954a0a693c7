#include "nccl_dyn.h"

#include <dlfcn.h>

#include <mutex>

namespace disc_b200 {
namespace ral {
namespace {

template <typename Fn>
bool bind(void* lib, const char* name, Fn* out, std::string* err) {
  void* sym = dlsym(lib, name);
  if (!sym) {
    *err = std::string("NCCL symbol missing: ") + name;
    return false;
  }
  *out = reinterpret_cast<Fn>(sym);
  return true;
}

NcclApi load() {
  NcclApi api;
  // RTLD_NOLOAD: the copy a host framework already mapped, if any.
  void* lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_LOCAL);
  if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_LOCAL);
  if (!lib) {
    const char* e = dlerror();
    api.error = std::string("libnccl.so.2 not found: ") + (e ? e : "");
    return api;
  }
  int (*get_version)(int*) = nullptr;
  if (!bind(lib, "ncclGetUniqueId", &api.GetUniqueId, &api.error) ||
      !bind(lib, "ncclCommInitRank", &api.CommInitRank, &api.error) ||
      !bind(lib, "ncclCommDestroy", &api.CommDestroy, &api.error) ||
      !bind(lib, "ncclCommCount", &api.CommCount, &api.error) ||
      !bind(lib, "ncclCommUserRank", &api.CommUserRank, &api.error) ||
      !bind(lib, "ncclAllGather", &api.AllGather, &api.error) ||
      !bind(lib, "ncclAllReduce", &api.AllReduce, &api.error) ||
      !bind(lib, "ncclBroadcast", &api.Broadcast, &api.error) ||
      !bind(lib, "ncclGroupStart", &api.GroupStart, &api.error) ||
      !bind(lib, "ncclGroupEnd", &api.GroupEnd, &api.error) ||
      !bind(lib, "ncclGetErrorString", &api.GetErrorString, &api.error) ||
      !bind(lib, "ncclGetVersion", &get_version, &api.error)) {
    return api;
  }
  get_version(&api.version);
  api.ok = true;
  return api;
}

}  // namespace

std::string NcclApi::describe(int result) const {
  if (GetErrorString) return GetErrorString(result);
  return "NCCL result " + std::to_string(result);
}

const NcclApi& nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] { api = load(); });
  return api;
}

}  // namespace ral
}  // namespace disc_b200

#include "context.h"

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>

#include "abi.h"
#include "cu_driver_dyn.h"
#include "nccl_dyn.h"

namespace disc_b200 {
namespace ral {

// ---------------------------------------------------------------- registry
namespace {
struct RegistryState {
  std::mutex mu;
  std::unordered_map<std::string, ApiFn> table;
  std::vector<std::string> full_names;  // mangled names only, in registration order
};
RegistryState& registry() {
  static RegistryState* r = new RegistryState;  // never destroyed: used by static registrars
  return *r;
}
}  // namespace

bool registry_add(const std::string& mangled, const std::string& nickname, ApiFn fn) {
  RegistryState& r = registry();
  std::lock_guard<std::mutex> l(r.mu);
  const bool fresh = r.table.emplace(mangled, fn).second;
  if (fresh) r.full_names.push_back(mangled);
  r.table.emplace(nickname, fn);  // first registration keeps the nickname
  return fresh;
}

ApiFn registry_find(const std::string& name) {
  RegistryState& r = registry();
  std::lock_guard<std::mutex> l(r.mu);
  auto it = r.table.find(name);
  return it == r.table.end() ? nullptr : it->second;
}

int registry_size() {
  RegistryState& r = registry();
  std::lock_guard<std::mutex> l(r.mu);
  return static_cast<int>(r.full_names.size());
}

const char* registry_name_at(int i) {
  RegistryState& r = registry();
  std::lock_guard<std::mutex> l(r.mu);
  if (i < 0 || i >= static_cast<int>(r.full_names.size())) return nullptr;
  return r.full_names[i].c_str();
}

// ----------------------------------------------------------------- context
void* Context::raw_alloc(size_t bytes) {
  if (bytes == 0) bytes = 1;  // as the reference: zero-byte requests still get a pointer
  if (alloc_fn) return alloc_fn(alloc_user, bytes);
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) return nullptr;
  return p;
}

void Context::raw_free(void* p) {
  if (!p) return;
  if (free_fn) {
    free_fn(alloc_user, p);
    return;
  }
  cudaFree(p);
}

void Context::signal_error(int32_t code, const std::string& msg) {
  std::lock_guard<std::mutex> l(mu);
  if (status != 0) return;  // keep the first error
  status = code;
  message = msg;
}

bool Context::ok() {
  std::lock_guard<std::mutex> l(mu);
  return status == 0;
}

void* Context::get_splitk_ws(int64_t bytes, int64_t* have) {
  std::lock_guard<std::mutex> l(mu);
  if (bytes > splitk_ws_bytes) {
    // Another thread may already hold the old block for a launch it has not
    // issued yet, and launches queued on the stream may still use it: the old
    // block is kept until the context dies instead of being freed here.
    if (splitk_ws) retired_splitk_ws.push_back(splitk_ws);
    int64_t want = bytes < (8 << 20) ? (8 << 20) : bytes;
    splitk_ws = raw_alloc(static_cast<size_t>(want));
    splitk_ws_bytes = splitk_ws ? want : 0;
    if (splitk_ws) cudaMemsetAsync(splitk_ws, 0, static_cast<size_t>(want), stream);
  }
  if (have) *have = splitk_ws_bytes;
  return splitk_ws;
}

ConstStore::~ConstStore() {
  for (auto& kv : host_consts) std::free(kv.second.ptr);
  if (shared) {
    for (auto& kv : device_consts) cudaFree(kv.second.ptr);
  }
}

namespace {
struct SharedStores {
  std::mutex mu;
  std::map<std::pair<std::string, int>, std::weak_ptr<ConstStore>> by_file;
};
SharedStores& shared_stores() {
  static SharedStores* s = new SharedStores;  // never destroyed: contexts may die during process exit
  return *s;
}
}  // namespace

std::shared_ptr<ConstStore> shared_const_store(const std::string& path, int device, std::string* error) {
  SharedStores& reg = shared_stores();
  std::lock_guard<std::mutex> l(reg.mu);
  auto key = std::make_pair(path, device);
  auto it = reg.by_file.find(key);
  if (it != reg.by_file.end()) {
    if (auto live = it->second.lock()) return live;
  }
  auto file = MetadataFile::load(path, error);
  if (!file) return nullptr;
  auto store = std::make_shared<ConstStore>();
  store->metadata = std::move(file);
  store->shared = true;
  reg.by_file[key] = store;
  return store;
}

const ConstEntry* Context::get_const(bool on_device, const char* unique_name, int32_t index) {
  auto fail = [&](const std::string& msg) -> const ConstEntry* {
    signal_error(1, msg);
    return nullptr;
  };
  std::shared_ptr<ConstStore> st;
  {
    std::lock_guard<std::mutex> l(mu);
    st = consts;
  }
  if (!st) return fail("ral_const: no metadata file loaded (disc_b200_context_load_metadata)");
  std::lock_guard<std::mutex> l(st->mu);
  auto& by_index = on_device ? st->device_by_index : st->host_by_index;
  if (index >= 0 && index < static_cast<int32_t>(by_index.size()) && by_index[index]) return by_index[index];
  if (!unique_name) return fail("ral_const: null unique_name");
  const std::string key(unique_name);
  auto& store = on_device ? st->device_consts : st->host_consts;
  auto it = store.find(key);
  if (it == store.end()) {
    const std::string_view hex = on_device ? st->metadata->device_constant(key) : st->metadata->host_constant(key);
    if (hex.data() == nullptr) return fail("const unique_name " + key + " not found in metadata file");
    ConstEntry e;
    int64_t width = 0;
    if (!parse_const_name(key, &e.shape, &width)) return fail("unexpected const unique_name format: " + key);
    std::vector<uint8_t> data;
    if (!decode_hex(hex, &data)) return fail("constant " + key + " is not hexadecimal");
    // the shape comes from a string: refuse what cannot be a tensor in memory before multiplying
    constexpr int64_t kMaxConstBytes = int64_t{1} << 40;
    int64_t elems = 1;
    for (int64_t d : e.shape) {
      if (d != 0 && elems > kMaxConstBytes / d) return fail("constant " + key + " is larger than 1 TiB");
      elems *= d;
    }
    if (width != 0 && elems > kMaxConstBytes / width) return fail("constant " + key + " is larger than 1 TiB");
    const int64_t want = elems * width;
    if (static_cast<int64_t>(data.size()) < want) {
      // a splat: the stored element repeats (common_context_impl_cuda.cc:97-105)
      if (data.empty()) return fail("constant " + key + " is empty");
      const std::vector<uint8_t> unit = data;
      data.resize(static_cast<size_t>(want));
      for (int64_t off = static_cast<int64_t>(unit.size()); off < want; off += static_cast<int64_t>(unit.size())) {
        const int64_t n = std::min<int64_t>(static_cast<int64_t>(unit.size()), want - off);
        std::memcpy(data.data() + off, unit.data(), static_cast<size_t>(n));
      }
    }
    e.bytes = static_cast<int64_t>(data.size());
    if (on_device) {
      if (st->shared) {
        if (cudaMalloc(&e.ptr, data.empty() ? 1 : data.size()) != cudaSuccess) e.ptr = nullptr;
      } else {
        e.ptr = raw_alloc(data.size());
      }
      if (!e.ptr) return fail("device allocation of constant " + key + " failed");
      // the staging bytes die with this call: wait for the copy (as the reference does, :116-118);
      // after the wait the constant is visible to every stream, which a shared store relies on
      cudaError_t err = cudaMemcpyAsync(e.ptr, data.data(), data.size(), cudaMemcpyHostToDevice, stream);
      if (err == cudaSuccess) err = cudaStreamSynchronize(stream);
      if (err != cudaSuccess) {
        if (st->shared) {
          cudaFree(e.ptr);
        } else {
          raw_free(e.ptr);
        }
        return fail(std::string("upload of constant ") + key + ": " + cudaGetErrorString(err));
      }
      if (!st->shared) {
        std::lock_guard<std::mutex> lc(mu);
        persistent.insert(e.ptr);  // freed with this context
      }
      st->metadata->release_device(key);
    } else {
      e.ptr = std::malloc(data.empty() ? 1 : data.size());
      if (!e.ptr) return fail("host allocation of constant " + key + " failed");
      std::memcpy(e.ptr, data.data(), data.size());
      st->metadata->release_host(key);
    }
    it = store.emplace(key, std::move(e)).first;
  }
  if (index >= 0 && index < (1 << 20)) {
    if (static_cast<int32_t>(by_index.size()) <= index) by_index.resize(index + 1, nullptr);
    by_index[index] = &it->second;  // unordered_map nodes do not move
  }
  return &it->second;
}

bool Context::comm_info(int* size, int* rank) {
  if (!nccl_comm) {
    signal_error(1, "no NCCL communicator in this context (disc_b200_context_options.nccl_comm)");
    return false;
  }
  if (comm_size == 0) {
    const NcclApi& api = nccl_api();
    if (!api.ok) {
      signal_error(1, "NCCL unavailable: " + api.error);
      return false;
    }
    int n = 0, r = 0;
    int st = api.CommCount(nccl_comm, &n);
    if (st == 0) st = api.CommUserRank(nccl_comm, &r);
    if (st != 0 || n <= 0) {
      signal_error(1, "ncclCommCount / ncclCommUserRank failed: " + api.describe(st));
      return false;
    }
    std::lock_guard<std::mutex> l(mu);
    comm_size = n;
    comm_rank = r;
  }
  *size = comm_size;
  *rank = comm_rank;
  return true;
}

Context::~Context() {
  consts.reset();  // a private store frees its host constants; its device ones are in `persistent`
  for (void* p : host_persistent) std::free(p);
  if (!modules.empty() && cu_driver_api().ok) {
    for (auto& kv : modules) cu_driver_api().ModuleUnload(kv.second);
  }
  for (void* p : persistent) raw_free(p);
  if (splitk_ws) raw_free(splitk_ws);
  for (void* old : retired_splitk_ws) raw_free(old);
  magic = 0;
}

void* ExecContext::alloc(size_t bytes) {
  void* p = ctx->raw_alloc(bytes);
  if (!p) {
    signal_error("device allocation of " + std::to_string(bytes) + " bytes failed");
    return nullptr;
  }
  refcount[p] = 1;
  return p;
}

void ExecContext::dealloc(void* p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> l(ctx->mu);
    if (ctx->persistent.count(p)) return;
  }
  auto it = refcount.find(p);
  if (it == refcount.end()) return;  // not ours (an input, or another context's buffer)
  if (--it->second == 0) {
    refcount.erase(it);
    ctx->raw_free(p);
  }
}

// Host buffers of generated code (shape arithmetic, scalars read back): 64-byte
// aligned, zero-byte requests still get a pointer, counted like device buffers
// (tao_compiler/mlir/ral/context/base/cpu/cpu_context_impl.cc:120-180).
void* ExecContext::host_alloc(size_t bytes) {
  void* p = nullptr;
  const size_t rounded = ((bytes ? bytes : 1) + 63) / 64 * 64;
  if (posix_memalign(&p, 64, rounded) != 0 || !p) {
    signal_error("host allocation of " + std::to_string(bytes) + " bytes failed");
    return nullptr;
  }
  host_refcount[p] = 1;
  return p;
}

void ExecContext::host_dealloc(void* p) {
  if (!p) return;
  {
    std::lock_guard<std::mutex> l(ctx->mu);
    if (ctx->host_persistent.count(p)) return;
  }
  auto it = host_refcount.find(p);
  if (it == host_refcount.end()) return;  // an input or a constant
  if (--it->second == 0) {
    host_refcount.erase(it);
    std::free(p);
  }
}

Context* context_of(void* handle) {
  if (!handle) return nullptr;
  uint32_t magic;
  std::memcpy(&magic, handle, sizeof(magic));
  if (magic == kContextMagic) return static_cast<Context*>(handle);
  if (magic == kExecMagic) return static_cast<ExecContext*>(handle)->ctx;
  return nullptr;
}

}  // namespace ral
}  // namespace disc_b200

// ------------------------------------------------------------------- C ABI
using disc_b200::ral::Context;
using disc_b200::ral::ExecContext;

extern "C" {

const char* const kMlirLoweredEntry = "main";

void tao_ral_call_impl(tao_ral_context_t handle, void* name, void** args) {
  if (!handle) return;
  uint32_t magic;
  std::memcpy(&magic, handle, sizeof(magic));
  if (magic != disc_b200::ral::kExecMagic) return;
  ExecContext* exec = static_cast<ExecContext*>(handle);
  if (!name || !args) {
    exec->signal_error("tao_ral_call_impl: null name or args");
    return;
  }
  // Once a call has failed the following ones are skipped, so that a compiled
  // executable runs through to its end without touching half-made results.
  if (!exec->ctx->ok()) return;
  const char* api = static_cast<const char*>(name);
  disc_b200::ral::ApiFn fn = disc_b200::ral::registry_find(api);
  if (!fn) {
    exec->signal_error(std::string("api_func ") + api + " not found");
    return;
  }
  fn(args);
}

tao_ral_status_t tao_ral_last_error(tao_ral_context_t handle, const char** err_msg) {
  Context* ctx = disc_b200::ral::context_of(handle);
  if (!ctx) {
    if (err_msg) *err_msg = "invalid context handle";
    return 1;
  }
  std::lock_guard<std::mutex> l(ctx->mu);
  if (err_msg) *err_msg = ctx->message.c_str();
  return ctx->status;
}

void tao_ral_clear_error(tao_ral_context_t handle) {
  Context* ctx = disc_b200::ral::context_of(handle);
  if (!ctx) return;
  std::lock_guard<std::mutex> l(ctx->mu);
  ctx->status = 0;
  ctx->message.clear();
}

disc_b200_context* disc_b200_context_create(const disc_b200_context_options* opts) {
  Context* c = new Context;
  if (opts) {
    c->device = opts->device;
    c->stream = static_cast<cudaStream_t>(opts->stream);
    c->alloc_fn = opts->gpu_alloc;
    c->free_fn = opts->gpu_free;
    c->alloc_user = opts->alloc_user;
    c->nccl_comm = opts->nccl_comm;
    c->comm_stream = static_cast<cudaStream_t>(opts->comm_stream ? opts->comm_stream : opts->stream);
  }
  return reinterpret_cast<disc_b200_context*>(c);
}

void disc_b200_context_destroy(disc_b200_context* ctx) { delete reinterpret_cast<Context*>(ctx); }

disc_b200_exec* disc_b200_exec_create(disc_b200_context* ctx) {
  if (!ctx) return nullptr;
  ExecContext* e = new ExecContext;
  e->ctx = reinterpret_cast<Context*>(ctx);
  return reinterpret_cast<disc_b200_exec*>(e);
}

void disc_b200_exec_destroy(disc_b200_exec* handle) {
  ExecContext* e = reinterpret_cast<ExecContext*>(handle);
  if (!e) return;
  std::unordered_set<void*> handed_out;
  for (auto& kv : e->outputs) handed_out.insert(kv.second.data);
  for (auto& kv : e->refcount) {
    if (!handed_out.count(kv.first)) e->ctx->raw_free(kv.first);
  }
  for (auto& kv : e->host_refcount) {
    if (!handed_out.count(kv.first)) std::free(kv.first);
  }
  for (auto& kv : e->async_tokens) cudaEventDestroy(kv.second);
  e->magic = 0;
  delete e;
}

int32_t disc_b200_exec_bind_input(disc_b200_exec* handle, int32_t idx, const void* data,
                                  int32_t rank, const int64_t* sizes) {
  ExecContext* e = reinterpret_cast<ExecContext*>(handle);
  if (!e || rank < 0 || (rank > 0 && !sizes)) return 1;
  disc_b200::ral::BoundTensor t;
  t.data = const_cast<void*>(data);
  if (rank > 0) t.shape.assign(sizes, sizes + rank);
  e->inputs[idx] = t;
  e->input_ptrs.insert(t.data);
  return 0;
}

int32_t disc_b200_exec_get_output(disc_b200_exec* handle, int32_t idx, void** data, int32_t* rank,
                                  int64_t* sizes8, int32_t* owned) {
  ExecContext* e = reinterpret_cast<ExecContext*>(handle);
  if (!e) return 1;
  auto it = e->outputs.find(idx);
  if (it == e->outputs.end()) return 1;
  if (data) *data = it->second.data;
  if (rank) *rank = static_cast<int32_t>(it->second.shape.size());
  if (sizes8) {
    for (size_t i = 0; i < it->second.shape.size() && i < 8; ++i) sizes8[i] = it->second.shape[i];
  }
  if (owned) {
    // An output that aliases an input, a persistent buffer, or a buffer that
    // is also another output with a smaller index stays with its first owner.
    const bool host = e->host_refcount.count(it->second.data) != 0;
    bool mine = host || e->refcount.count(it->second.data) != 0;
    for (auto& kv : e->outputs) {
      if (kv.first < idx && kv.second.data == it->second.data) mine = false;
    }
    *owned = mine ? (host ? 2 : 1) : 0;
  }
  return 0;
}

void disc_b200_exec_free_output(disc_b200_context* ctx, void* data) {
  if (ctx) reinterpret_cast<Context*>(ctx)->raw_free(data);
}

void disc_b200_exec_free_host_output(void* data) { std::free(data); }

int32_t disc_b200_registry_size(void) { return disc_b200::ral::registry_size(); }
const char* disc_b200_registry_name(int32_t i) { return disc_b200::ral::registry_name_at(i); }
int32_t disc_b200_registry_has(const char* n) {
  return n && disc_b200::ral::registry_find(n) != nullptr ? 1 : 0;
}

}  // extern "C"

// Runtime context of the custom calls: the state the reference spreads over
// tao::ral::Context / ExecutionContext (tao_compiler/mlir/ral/ral_context.h:55-199)
// and BaseCudaContextState / BaseCudaExecutionContext
// (tao_compiler/mlir/ral/context/base/cuda/cuda_context_impl.cc:117-166,
//  base_context.h), reduced to what the quantized path touches.
//
// Differences by design: an error is recorded (first one wins) and reported
// through tao_ral_last_error instead of aborting the process
// (tao_compiler/mlir/ral/ral_context.cc:185-191 logs FATAL); the api-name
// lookup is one hash lookup on a string_view, no per-thread cache is needed.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "../../../include/disc_b200_ral.h"
#include "metadata.h"

namespace disc_b200 {
namespace ral {

constexpr uint32_t kContextMagic = 0xD15CB200u;
constexpr uint32_t kExecMagic = 0xD15CE8ECu;

// A constant of the compiled graph once it has been materialised.
struct ConstEntry {
  void* ptr = nullptr;
  std::vector<int64_t> shape;
  int64_t bytes = 0;
};

// The constants of one executable: its metadata file and what has been decoded from it
// (reference: RalGlobalConstantState, tao_compiler/mlir/ral/context/common_context_impl.cc:279-346
// and common_context_impl_cuda.cc:61-132).  Decoded on first use, device ones uploaded once;
// looked up by the module-unique index first, by name otherwise.  A store is private to a
// context, or shared by every context of the process that runs the same file on the same
// device (reference: ProcessLevelConstStore / ConstStoreRegistrar, :152-185, switched on by
// DISC_USE_GLOBAL_CONST_STORE): weights are then uploaded once per process, not per context.
struct ConstStore {
  std::mutex mu;
  std::unique_ptr<MetadataFile> metadata;
  std::unordered_map<std::string, ConstEntry> device_consts, host_consts;
  std::vector<const ConstEntry*> device_by_index, host_by_index;
  // A shared store owns its device constants (cudaMalloc / cudaFree), because it may outlive
  // the context that first asked for one; a private store's live in its context's allocator.
  bool shared = false;
  ~ConstStore();
};
// The process-wide store for (path, device): the live one if any context still holds it, else a
// new one.  nullptr (and `error` filled) if the file does not load.
std::shared_ptr<ConstStore> shared_const_store(const std::string& path, int device, std::string* error);

struct Context {
  uint32_t magic = kContextMagic;
  int device = 0;
  cudaStream_t stream = nullptr;
  disc_b200_alloc_fn alloc_fn = nullptr;
  disc_b200_free_fn free_fn = nullptr;
  void* alloc_user = nullptr;
  void* nccl_comm = nullptr;
  cudaStream_t comm_stream = nullptr;
  int comm_size = 0;  // ranks of nccl_comm, 0 until first asked
  int comm_rank = 0;

  std::mutex mu;
  int32_t status = 0;
  std::string message;
  std::unordered_set<void*> persistent;  // survive executions, freed with the context
  std::unordered_set<void*> host_persistent;  // the same for host buffers
  // Generated kernels: image address -> loaded module, (image, name) -> function
  // (reference: BaseCudaContextState::blobs / kernels, cuda_context_impl.cc:60-75).
  std::unordered_map<const void*, void*> modules;
  std::map<std::pair<const void*, std::string>, void*> kernels;
  int cc_major = 0, cc_minor = 0;  // of `device`, 0 until first asked
  // Scratch of the small-M qgemm path (grown on demand, counters kept zero).
  void* splitk_ws = nullptr;
  int64_t splitk_ws_bytes = 0;
  std::vector<void*> retired_splitk_ws;  // outgrown blocks, freed with the context

  void* raw_alloc(size_t bytes);
  void raw_free(void* p);
  void signal_error(int32_t code, const std::string& msg);
  bool ok();
  // Returns scratch of at least `bytes`, zeroed when (re)allocated.
  // Scratch of at least `bytes`; `have` receives its size (pointer and size are read under one lock).
  void* get_splitk_ws(int64_t bytes, int64_t* have);
  // Size and rank of nccl_comm (queried once); false, with an error signalled,
  // when there is no communicator or NCCL cannot be reached.
  bool comm_info(int* size, int* rank);

  // Constants of the executable; null until a metadata file is attached.
  std::shared_ptr<ConstStore> consts;
  // nullptr after signalling an error
  const ConstEntry* get_const(bool on_device, const char* unique_name, int32_t index);
  ~Context();
};

struct BoundTensor {
  void* data = nullptr;
  std::vector<int64_t> shape;
};

struct ExecContext {
  uint32_t magic = kExecMagic;
  Context* ctx = nullptr;
  std::unordered_map<int64_t, BoundTensor> inputs;
  std::unordered_map<int64_t, BoundTensor> outputs;
  std::unordered_map<void*, int> refcount;  // device buffers allocated during this execution
  std::unordered_map<void*, int> host_refcount;  // host buffers ("alloc" on "cpu"), same rules
  std::unordered_set<void*> input_ptrs;
  // Completion events of asynchronous collectives, by async_token_key
  // (reference: async_pair_tokens, tao_compiler/mlir/ral/collective.cu.cc:134,431).
  std::unordered_map<int64_t, cudaEvent_t> async_tokens;

  void* alloc(size_t bytes);
  void dealloc(void* p);
  void* host_alloc(size_t bytes);
  void host_dealloc(void* p);
  void signal_error(const std::string& msg) { ctx->signal_error(1, msg); }
};

// Either handle kind -> its Context (nullptr if the handle is neither).
Context* context_of(void* handle);

}  // namespace ral
}  // namespace disc_b200

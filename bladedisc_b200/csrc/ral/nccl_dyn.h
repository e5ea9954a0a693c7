// NCCL reached through dlopen, so that the library loads (and the quantized
// path runs) on hosts without NCCL and links against no particular copy of it.
// The copy already mapped into the process wins (a host that created the
// communicator with its own NCCL must be served by the same one); otherwise
// the system's libnccl.so.2 is opened.
//
// Only the entry points the collective custom calls need are bound
// (reference call sites: tao_compiler/mlir/ral/collective.cu.cc:60-309).
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <string>

namespace disc_b200 {
namespace ral {

// Values of ncclDataType_t / ncclRedOp_t (public NCCL API, stable since 2.x).
enum NcclType : int { kNcclInt8 = 0, kNcclUint8 = 1, kNcclInt32 = 2, kNcclFloat16 = 6, kNcclFloat32 = 7, kNcclBfloat16 = 9 };
enum NcclOp : int { kNcclSum = 0, kNcclProd = 1, kNcclMax = 2, kNcclMin = 3 };

constexpr int kNcclUniqueIdBytes = 128;
struct NcclUniqueId {
  char internal[kNcclUniqueIdBytes];
};

struct NcclApi {
  bool ok = false;
  std::string error;  // why the binding failed
  int version = 0;

  int (*GetUniqueId)(NcclUniqueId*) = nullptr;
  int (*CommInitRank)(void** comm, int nranks, NcclUniqueId id, int rank) = nullptr;
  int (*CommDestroy)(void* comm) = nullptr;
  int (*CommCount)(void* comm, int* count) = nullptr;
  int (*CommUserRank)(void* comm, int* rank) = nullptr;
  int (*AllGather)(const void* send, void* recv, size_t sendcount, int dtype, void* comm,
                   cudaStream_t stream) = nullptr;
  int (*AllReduce)(const void* send, void* recv, size_t count, int dtype, int op, void* comm,
                   cudaStream_t stream) = nullptr;
  int (*Broadcast)(const void* send, void* recv, size_t count, int dtype, int root, void* comm,
                   cudaStream_t stream) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;

  std::string describe(int result) const;
};

// Binds on first use; never throws.  `ok == false` means collectives are
// unavailable and `error` says why.
const NcclApi& nccl_api();

}  // namespace ral
}  // namespace disc_b200

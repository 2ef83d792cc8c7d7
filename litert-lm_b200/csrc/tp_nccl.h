// Tensor parallelism over NCCL: the sums of the ranks' partial O and down
// projections.  NCCL is bound at run time (dlopen of libnccl.so.2, the library
// that torch ships and has already loaded in a Python process), so the shared
// library carries no link-time dependency on it and single-GPU users never touch
// it.  Only ncclGetUniqueId / ncclCommInitRank / ncclAllReduce / ncclCommDestroy
// are used; the collective runs on the executor's stream.
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <mutex>
#include <string>

#include "common.cuh"

namespace b200lm {

constexpr int kNcclUniqueIdBytes = 128;

struct NcclApi {
  typedef struct { char internal[kNcclUniqueIdBytes]; } UniqueId;
  typedef void* Comm;
  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int /*dtype*/, int /*op*/, Comm, cudaStream_t) = nullptr;
  int (*CommDestroy)(Comm) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;

  static const NcclApi& get() {
    static NcclApi api;
    static std::once_flag once;
    static std::string failure;
    std::call_once(once, [] {
      void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
      if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
      if (!h) {
        failure = std::string("libnccl.so.2 cannot be loaded (") + dlerror() +
                  "): import torch first or put NCCL on the library path";
        return;
      }
      api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
      api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
      api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
      api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
      api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
      if (!api.GetUniqueId || !api.CommInitRank || !api.AllReduce || !api.CommDestroy) failure = "libnccl.so.2 lacks an expected symbol";
    });
    if (!failure.empty()) throw Error{kFailedPrecondition, failure};
    return api;
  }
  void check(int rc, const char* what) const {
    if (rc != 0)
      throw Error{kInternal, std::string(what) + ": " + (GetErrorString ? GetErrorString(rc) : "NCCL error") + " (" + std::to_string(rc) + ")"};
  }
};

constexpr int kNcclFloat32 = 7;   // ncclFloat32
constexpr int kNcclSum = 0;       // ncclSum

}  // namespace b200lm

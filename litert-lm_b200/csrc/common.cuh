// Shared declarations for the B200 executor library: status codes, error
// plumbing, model geometry and small device helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <mutex>
#include <string>
#include <utility>

namespace b200lm {

// absl::StatusCode integers, the convention of the reference's one dynamic C
// boundary (runtime/components/sampler_factory.cc:30-57).
enum Status : int {
  kOk = 0,
  kCancelled = 1,
  kInvalidArgument = 3,
  kDeadlineExceeded = 4,
  kNotFound = 5,
  kFailedPrecondition = 9,
  kOutOfRange = 11,
  kUnimplemented = 12,
  kInternal = 13,
};

struct Error {
  int code;
  std::string msg;
};

#define B2_CUDA(expr)                                                              \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess)                                                         \
      throw ::b200lm::Error{::b200lm::kInternal, std::string(#expr) + ": " +      \
                                                     cudaGetErrorString(_e)};      \
  } while (0)

#define B2_CHECK(cond, code, text)                          \
  do {                                                      \
    if (!(cond)) throw ::b200lm::Error{(code), (text)};    \
  } while (0)

// The opt-in dynamic shared-memory limit of a kernel is a property of (kernel, device), shared by every
// caller in the process.  It is only ever RAISED here: lowering it for one caller's smaller shape would
// make a later launch that asks for more fail.  Thread-safe.
inline void raise_dyn_smem(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> high;
  int dev = 0;
  B2_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  size_t& h = high[std::make_pair(kernel, dev)];
  if (bytes <= h) return;
  B2_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  h = bytes;
}
template <typename... KArgs>
inline void raise_dyn_smem(void (*kernel)(KArgs...), size_t bytes) {
  raise_dyn_smem(reinterpret_cast<const void*>(kernel), bytes);
}

constexpr int kPage = 256;       // KV positions per page
constexpr int kMaxBuckets = 8;

// Geometry of one decoder, as stored in the weights record.
struct ModelDims {
  int n_layers, d, hq, hkv, hd, ffn, vocab, max_ctx, window, period, kv_dtype;
  int n_buckets;
  int buckets[kMaxBuckets];
  float rope_local, rope_global, eps;
  __host__ __device__ int nq() const { return hq * hd; }
  __host__ __device__ int nkv() const { return hkv * hd; }
  __host__ __device__ int nqkv() const { return (hq + 2 * hkv) * hd; }
  __host__ __device__ int group() const { return hq / hkv; }
  __host__ __device__ bool is_global(int layer) const { return layer % period == period - 1; }
};

// Error word written by device code (bounded waits, range checks); 0 = clean.
enum DeviceError : int {
  kDevOk = 0,
  kDevBarrierTimeout = 1,   // a bounded mbarrier / grid-barrier wait gave up
  kDevBadToken = 2,         // token id outside the vocabulary
  kDevBadPosition = 3,      // position outside the KV capacity
};

#ifdef __CUDACC__
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float gelu_tanh(float x) {
  const float c = 0.7978845608028654f;
  return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}
// Programmatic dependent launch.  A kernel launched with programmatic stream
// serialisation may start while its predecessor in the stream still runs;
// pdl_wait() blocks until the predecessor has completed and its writes are
// visible (a no-op for an ordinary launch).  Nothing before it may touch memory
// the predecessor reads or writes.  pdl_launch_dependents() lets the successor
// start its own set-up once every CTA of this grid has got here.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint4 ldg_nc_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
#endif

}  // namespace b200lm

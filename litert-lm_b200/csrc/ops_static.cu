// Allocation-free variant of the split-KV decode attention (see b200lm_ops.h,
// B200LmOps_AttentionDecodeStatic).  Compiled into the same translation unit
// as ops.cu, whose kernels it launches.
//
// The ordinary entry point allocates device memory for the split partials
// (m, l, unnormalised o per split) on every call.  Some hosts cannot do that:
// a caller that runs inside another runtime's execution callback, a real-time
// serving loop that forbids allocator calls after start-up, or a process whose
// device memory is fully budgeted up front.  For them the partials, the query
// positions and the error word live in ONE file-scope device array of fixed
// size.  Every GPU that loads this library carries that array until the
// process exits.
#include "../../include/b200lm_ops.h"
#include "common.cuh"
#include "decode_ops.cuh"
#include "prefill_ops.cuh"

#include <mutex>

namespace b200lm {

constexpr size_t kStaticScratchBytes = 8u << 20;          // 8 MiB per GPU
constexpr size_t kStaticHeaderBytes = 64u << 10;          // error word + query positions
constexpr int kStaticMaxQueries = (int)(kStaticHeaderBytes / 4) - 16;

// In HOST code this name is only a stand-in for the symbol: it is not a device
// address.  Host code gets the address with cudaGetSymbolAddress (below);
// device code may name the array directly.
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

// Header layout: int[0] = error word, int[16 + i] = position of query i.
__global__ void static_scratch_prepare_kernel(int nq, int pos) {
  int* hdr = reinterpret_cast<int*>(g_attn_static_scratch);
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) hdr[0] = 0;                   // the error word must start at zero
  if (i < nq) hdr[16 + i] = pos;
}

constexpr int kMaxDevices = 64;
static unsigned char* g_static_scratch_addr[kMaxDevices] = {nullptr};
static std::mutex g_static_scratch_mu;     // guards the per-device set-up below

// Device address of the array on `device` (which must be current).  Looked up
// once per device, under a lock: concurrent first calls do the set-up once.
static unsigned char* static_scratch_for(int device) {
  B2_CHECK(device >= 0 && device < kMaxDevices, kInvalidArgument, "device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_static_scratch_mu);
  if (!g_static_scratch_addr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      throw Error{kInternal, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e)};
    // attribute change, not an allocation; done with the set-up so later calls only launch.  The limit is
    // raised to the largest shape the entry point accepts and never lowered by any other caller.
    raise_dyn_smem(attn_decode_kernel, sizeof(float) * ((size_t)(4 + 2) * 256 + (size_t)kDecWarps * 4 * (256 + 2)));
    g_static_scratch_addr[device] = reinterpret_cast<unsigned char*>(p);
  }
  return g_static_scratch_addr[device];
}

// Makes `device` current for the duration of a call and puts the caller's device back afterwards.
struct DeviceScope {
  int prev = -1;
  explicit DeviceScope(int device) {
    if (cudaGetDevice(&prev) != cudaSuccess) { cudaGetLastError(); prev = -1; }
    B2_CUDA(cudaSetDevice(device));
  }
  ~DeviceScope() {
    if (prev >= 0) cudaSetDevice(prev);
  }
};

static int static_fail(char** err, int code, const std::string& msg) {
  if (err) {
    *err = reinterpret_cast<char*>(malloc(msg.size() + 1));
    if (*err) memcpy(*err, msg.c_str(), msg.size() + 1);
  }
  return code;
}

static void require_device(int device) {
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev <= 0) {
    cudaGetLastError();
    throw Error{kFailedPrecondition, "no CUDA device: this backend has no CPU fallback"};
  }
  B2_CHECK(device >= 0 && device < ndev, kInvalidArgument, "device ordinal out of range");
}

}  // namespace b200lm

using namespace b200lm;

extern "C" int B200LmOps_AttentionDecodeStatic(int32_t device, const float* q_dev, const void* k_pages_dev,
                                               const void* v_pages_dev, const int32_t* page_table_dev, int32_t batch,
                                               int32_t s, int32_t hq, int32_t hkv, int32_t hd, int32_t window,
                                               int32_t kv_bf16, int32_t nsplit, float* out_dev, void* stream,
                                               char** err) {
  if (err) *err = nullptr;
  try {
    B2_CHECK(q_dev && k_pages_dev && v_pages_dev && page_table_dev && out_dev, kInvalidArgument, "null pointer");
    B2_CHECK(batch > 0 && s > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, kInvalidArgument, "bad shape");
    const int G = hq / hkv;
    B2_CHECK(G == 1 || G == 2 || G == 4, kUnimplemented, "GQA group size must be 1, 2 or 4");
    B2_CHECK(hd == 32 || hd == 64 || hd == 128 || hd == 256, kUnimplemented, "head_dim must be 32/64/128/256");
    B2_CHECK(nsplit >= 1 && nsplit <= kMaxSplits, kInvalidArgument, "nsplit out of range");
    B2_CHECK(batch <= kStaticMaxQueries, kInvalidArgument,
             "batch exceeds the static scratch: at most " + std::to_string(kStaticMaxQueries) + " queries");
    const size_t part_o_bytes = (size_t)batch * hkv * nsplit * G * hd * sizeof(float);
    const size_t part_ml_bytes = (size_t)batch * hkv * nsplit * G * 2 * sizeof(float);
    B2_CHECK(kStaticHeaderBytes + part_o_bytes + part_ml_bytes <= kStaticScratchBytes, kInvalidArgument,
             "split partials need " + std::to_string(part_o_bytes + part_ml_bytes) + " bytes; the static scratch holds " +
                 std::to_string(kStaticScratchBytes - kStaticHeaderBytes) + " (lower batch or nsplit)");
    require_device(device);
    DeviceScope scope(device);                                  // the caller's current device is restored on return
    unsigned char* scratch = static_scratch_for(device);        // first call on a device does the set-up
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int* hdr = reinterpret_cast<int*>(scratch);
    float* part_o = reinterpret_cast<float*>(scratch + kStaticHeaderBytes);
    float* part_ml = reinterpret_cast<float*>(scratch + kStaticHeaderBytes + part_o_bytes);
    static_scratch_prepare_kernel<<<(batch + 255) / 256, 256, 0, st>>>(batch, s - 1);
    B2_CUDA(cudaGetLastError());
    ModelDims dm{};
    dm.hq = hq; dm.hkv = hkv; dm.hd = hd; dm.d = 64; dm.ffn = 64;
    dm.window = window > 0 ? window : 1 << 30;
    dm.kv_dtype = kv_bf16 ? 1 : 0;
    dm.eps = 1e-6f;
    const int npages = (s + kPage - 1) / kPage;
    dm.max_ctx = npages * kPage;
    AttnJob j;
    memset(&j, 0, sizeof j);
    j.qkv = q_dev;                       // rows of (hq + 2 hkv) * hd floats; only the q part is read
    j.pos = hdr + 16;
    j.page_table = page_table_dev;
    j.pages_per_seq = npages;
    j.seq_stride = 0;
    j.is_global = window > 0 ? 0 : 1;
    j.nsplit = nsplit;
    j.appended = 1;
    j.kv.k = const_cast<void*>(k_pages_dev);
    j.kv.v = const_cast<void*>(v_pages_dev);
    j.part_o = part_o;
    j.part_ml = part_ml;
    j.err = hdr;
    int n_sms = 0;
    B2_CUDA(cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, device));
    const size_t smem_dec = sizeof(float) * ((size_t)(G + 2) * hd + (size_t)kDecWarps * G * (hd + 2));
    const int items = batch * hkv * nsplit;
    const int grid = items < n_sms ? items : n_sms;
    attn_decode_kernel<<<grid, kDecThreads, smem_dec, st>>>(dm, j, batch);
    B2_CUDA(cudaGetLastError());         // a rejected launch must not be followed by a combine of stale partials
    const int total = batch * hq * hd;
    attn_combine_kernel<<<(total + 255) / 256, 256, 0, st>>>(part_o, part_ml, batch, hq, hkv, hd, nsplit, out_dev);
    B2_CUDA(cudaGetLastError());
  } catch (const Error& e_) {
    return static_fail(err, e_.code, e_.msg);
  } catch (...) {
    return static_fail(err, kInternal, "unknown failure");
  }
  return kOk;
}

// Reads back the error word that the kernels of B200LmOps_AttentionDecodeStatic write into the static
// array (a query position outside the cache).  Waits for `stream`, allocates nothing.
extern "C" int B200LmOps_AttentionDecodeStaticStatus(int32_t device, void* stream, int32_t* device_error, char** err) {
  if (err) *err = nullptr;
  try {
    require_device(device);
    DeviceScope scope(device);
    (void)static_scratch_for(device);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    int word = 0;
    B2_CUDA(cudaMemcpyFromSymbolAsync(&word, g_attn_static_scratch, sizeof(int), 0, cudaMemcpyDeviceToHost, st));
    B2_CUDA(cudaStreamSynchronize(st));
    if (device_error) *device_error = word;
    if (word == kDevBadPosition) throw Error{kInvalidArgument, "a query position lay outside the cache"};
    if (word == kDevBarrierTimeout) throw Error{kDeadlineExceeded, "a bounded device-side wait gave up"};
    if (word != kDevOk) throw Error{kInternal, "device error word " + std::to_string(word)};
  } catch (const Error& e_) {
    return static_fail(err, e_.code, e_.msg);
  } catch (...) {
    return static_fail(err, kInternal, "unknown failure");
  }
  return kOk;
}

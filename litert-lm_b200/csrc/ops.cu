// Operator-level C ABI (b200lm_ops.h): thin host wrappers that stage host
// arrays on the device, run ONE kernel family of the executor and copy the
// result back.  Compiled into the same translation unit as executor.cu.
#include <vector>

#include "../../include/b200lm_ops.h"
#include "common.cuh"
#include "decode_ops.cuh"
#include "model_host.h"
#include "prefill_ops.cuh"
#include "runtime.h"

namespace b200lm {

struct DevBuf {
  void* p = nullptr;
  explicit DevBuf(size_t n, bool zero = false) {
    B2_CUDA(cudaMalloc(&p, n ? n : 256));
    if (zero) B2_CUDA(cudaMemset(p, 0, n ? n : 256));
  }
  ~DevBuf() { cudaFree(p); }
  template <typename T>
  T* as() const { return reinterpret_cast<T*>(p); }
  DevBuf(const DevBuf&) = delete;
  DevBuf& operator=(const DevBuf&) = delete;
};

static void need_device(int device) {
  int n = 0;
  cudaError_t r = cudaGetDeviceCount(&n);
  if (r != cudaSuccess || n <= 0) {
    cudaGetLastError();
    throw Error{kFailedPrecondition, "no CUDA device: this backend has no CPU fallback"};
  }
  B2_CHECK(device >= 0 && device < n, kInvalidArgument, "device ordinal out of range");
  B2_CUDA(cudaSetDevice(device));
}

__global__ void unpack_w4t_kernel(const uint4* __restrict__ w, int N, int K, int8_t* __restrict__ out) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)N * K) return;
  int n = (int)(idx / K), k = (int)(idx % K);
  const uint4* tile = w + ((size_t)(n / 16) * (K / 64) + k / 64) * 32;
  out[idx] = (int8_t)w4t_element(tile, n % 16, k % 64);
}

__global__ void f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16(in[i]);
}
__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]);
}

// Stand-alone GEMV: activation slice from global memory, then the same tile
// loop and epilogue as the decode phases.
__global__ void __launch_bounds__(kDecThreads, 1)
gemv_w4_kernel(GemvJob j, const float* __restrict__ x, int ncols, int nterms, ModelDims smem_dims) {
  extern __shared__ __align__(16) unsigned char dsm[];
  DecodeSmem s = carve_smem(dsm, smem_dims, ncols);
  int slice, t0, t1;
  if (!gemv_assignment(j, blockIdx.x, gridDim.x, &slice, &t0, &t1)) return;
  const int Ks = j.K / j.slices;
  for (int col = 0; col < ncols; ++col)
    for (int i = threadIdx.x; i < Ks; i += kDecThreads)
      s.xf[(size_t)col * Ks + i] = x[(size_t)col * j.K + (size_t)slice * Ks + i];
  __syncthreads();
  quantize_cols(s, Ks, ncols, nterms);
  gemv_run(j, s, ncols, nterms, slice, t0, t1, nullptr, nullptr);
}

// Combine of split-KV partials into normalised outputs (the log-sum-exp merge
// that phase C of the decode step performs in its prologue).
__global__ void attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int nq,
                                    int hq, int hkv, int hd, int nsplit, float* __restrict__ out) {
  int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= nq * hq * hd) return;
  int e = idx % hd, h = (idx / hd) % hq, qi = idx / (hd * hq);
  int G = hq / hkv, kvh = h / G, g = h % G;
  size_t base = (((size_t)qi * hkv + kvh) * nsplit) * G + g;
  float M = -INFINITY;
  for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, part_ml[(base + (size_t)sp * G) * 2]);
  float L = 0.f, O = 0.f;
  for (int sp = 0; sp < nsplit; ++sp) {
    size_t pi = base + (size_t)sp * G;
    float f = __expf(part_ml[pi * 2] - M);
    L += part_ml[pi * 2 + 1] * f;
    O += part_o[pi * hd + e] * f;
  }
  out[idx] = L > 0.f ? O / L : 0.f;
}

// Split-KV decode attention over a batch of single-token queries.
__global__ void __launch_bounds__(kDecThreads, 1)
attn_decode_kernel(ModelDims dm, AttnJob job, int nq) {
  extern __shared__ __align__(16) float attn_sm2[];
  int items = nq * dm.hkv * job.nsplit;
  for (int it = blockIdx.x; it < items; it += gridDim.x) {
    int split = it % job.nsplit, rest = it / job.nsplit;
    int kvh = rest % dm.hkv, qi = rest / dm.hkv;
    attn_dispatch(dm, job, attn_sm2, qi, kvh, split);
  }
}

template <typename T>
__global__ void fill_pages_kernel(const float* __restrict__ src, T* __restrict__ dst, int S, int hkv, int hd) {
  // src [S][hkv][hd] -> pages [page][hkv][kPage][hd]
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)S * hkv * hd) return;
  int e = (int)(idx % hd), h = (int)((idx / hd) % hkv), s = (int)(idx / ((int64_t)hd * hkv));
  size_t off = (((size_t)(s / kPage) * hkv + h) * kPage + (s % kPage)) * hd + e;
  if constexpr (sizeof(T) == 4) dst[off] = src[idx];
  else dst[off] = __float2bfloat16(src[idx]);
}

// src [S][hkv][hd] -> transposed bf16 pages [page][hkv][hd][kPage]
__global__ void fill_pages_vt_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int S, int hkv, int hd) {
  int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)S * hkv * hd) return;
  int e = (int)(idx % hd), h = (int)((idx / hd) % hkv), s = (int)(idx / ((int64_t)hd * hkv));
  size_t off = (((size_t)(s / kPage) * hkv + h) * hd + e) * kPage + (s % kPage);
  dst[off] = __float2bfloat16(src[idx]);
}
__global__ void scale_to_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, int64_t n, float scale) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16(src[i] * scale);
}

}  // namespace b200lm

using namespace b200lm;

static int ops_fail(char** err, int code, const std::string& msg) {
  if (err) {
    *err = reinterpret_cast<char*>(malloc(msg.size() + 1));
    if (*err) memcpy(*err, msg.c_str(), msg.size() + 1);
  }
  return code;
}
#define OPS_BEGIN \
  if (err) *err = nullptr; \
  try {
#define OPS_END                                                              \
  }                                                                          \
  catch (const Error& e_) { return ops_fail(err, e_.code, e_.msg); }         \
  catch (const std::exception& e_) { return ops_fail(err, kInternal, e_.what()); } \
  return kOk;

static void check_matrix(int64_t n, int64_t k) {
  B2_CHECK(n > 0 && k > 0 && k % 64 == 0, kInvalidArgument, "k must be a positive multiple of 64");
}

extern "C" {

int B200LmOps_RepackW4T(const uint8_t* packed, int64_t n, int64_t k, uint8_t* out, char** err) {
  OPS_BEGIN
  B2_CHECK(packed && out, kInvalidArgument, "null pointer");
  check_matrix(n, k);
  int64_t np = (n + 15) / 16 * 16;
  repack_w4t(packed, np, k, [n](int64_t r) { return r < n ? r : (int64_t)-1; }, reinterpret_cast<uint32_t*>(out));
  OPS_END
}

int B200LmOps_RepackW4G(const uint8_t* packed, int64_t n, int64_t k, uint8_t* out, char** err) {
  OPS_BEGIN
  B2_CHECK(packed && out, kInvalidArgument, "null pointer");
  check_matrix(n, k);
  int64_t tiles = (n + 127) / 128;
  repack_w4g(packed, tiles, k, [n](int64_t r) { return r < n ? r : (int64_t)-1; }, reinterpret_cast<uint32_t*>(out));
  OPS_END
}

int B200LmOps_UnpackW4(int32_t device, const uint8_t* packed, int64_t n, int64_t k, int8_t* out, char** err) {
  OPS_BEGIN
  B2_CHECK(packed && out, kInvalidArgument, "null pointer");
  check_matrix(n, k);
  B2_CHECK(n % 16 == 0, kInvalidArgument, "n must be a multiple of 16");
  need_device(device);
  std::vector<uint32_t> host((size_t)n * k / 8);
  repack_w4t(packed, n, k, [](int64_t r) { return r; }, host.data());
  DevBuf w(host.size() * 4), o((size_t)n * k);
  B2_CUDA(cudaMemcpy(w.p, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
  int64_t total = n * k;
  unpack_w4t_kernel<<<(unsigned)((total + 255) / 256), 256>>>(w.as<uint4>(), (int)n, (int)k, o.as<int8_t>());
  B2_CUDA(cudaGetLastError());
  B2_CUDA(cudaMemcpy(out, o.p, (size_t)total, cudaMemcpyDeviceToHost));
  OPS_END
}

int B200LmOps_GemvW4(int32_t device, const uint8_t* packed, const float* scale, int64_t n, int64_t k, const float* x,
                     int32_t ncols, int32_t nterms, int32_t kslices, float* y, char** err) {
  OPS_BEGIN
  B2_CHECK(packed && scale && x && y, kInvalidArgument, "null pointer");
  check_matrix(n, k);
  B2_CHECK(n % 16 == 0, kInvalidArgument, "n must be a multiple of 16");
  B2_CHECK(ncols >= 1 && ncols <= kMaxCols && nterms >= 1 && nterms <= 3 && ncols * nterms <= kQCols,
           kInvalidArgument, "ncols * nterms must fit one 8-column MMA tile");
  B2_CHECK(kslices >= 1 && (k / 64) % kslices == 0, kInvalidArgument, "kslices must divide k/64");
  need_device(device);
  cudaDeviceProp prop;
  B2_CUDA(cudaGetDeviceProperties(&prop, device));
  std::vector<uint32_t> host((size_t)n * k / 8);
  repack_w4t(packed, n, k, [](int64_t r) { return r; }, host.data());
  DevBuf w(host.size() * 4), sc((size_t)n * 4), xd((size_t)ncols * k * 4), yd((size_t)kslices * ncols * n * 4, true);
  B2_CUDA(cudaMemcpy(w.p, host.data(), host.size() * 4, cudaMemcpyHostToDevice));
  B2_CUDA(cudaMemcpy(sc.p, scale, (size_t)n * 4, cudaMemcpyHostToDevice));
  B2_CUDA(cudaMemcpy(xd.p, x, (size_t)ncols * k * 4, cudaMemcpyHostToDevice));
  ModelDims dm{};
  dm.d = (int)k; dm.ffn = (int)k; dm.hq = 1; dm.hkv = 1; dm.hd = 32;
  size_t smem = dec_smem_bytes(dm, ncols);
  B2_CHECK(smem <= (size_t)prop.sharedMemPerBlockOptin, kInvalidArgument, "k too large for the shared-memory staging");
  raise_dyn_smem(gemv_w4_kernel, (size_t)(smem));
  GemvJob j{w.as<uint4>(), sc.as<float>(), (int)n, (int)k, kslices, yd.as<float>(), kEpiPlain};
  gemv_w4_kernel<<<prop.multiProcessorCount, kDecThreads, smem>>>(j, xd.as<float>(), ncols, nterms, dm);
  B2_CUDA(cudaGetLastError());
  B2_CUDA(cudaDeviceSynchronize());
  std::vector<float> parts((size_t)kslices * ncols * n);
  B2_CUDA(cudaMemcpy(parts.data(), yd.p, parts.size() * 4, cudaMemcpyDeviceToHost));
  for (int64_t i = 0; i < (int64_t)ncols * n; ++i) {
    float acc = 0.f;
    for (int s = 0; s < kslices; ++s) acc += parts[(size_t)s * ncols * n + i];
    y[i] = acc;
  }
  OPS_END
}

static void run_gemm_common(int device, int mode, const uint8_t* packed_rows, const float* scales, int64_t n_logical,
                            int64_t k, bool geglu, int64_t ffn, const float* a, int t, int ksplit, int repeat,
                            float* out, float* ms_out) {
  need_device(device);
  cudaDeviceProp prop;
  B2_CUDA(cudaGetDeviceProperties(&prop, device));
  const int tp = (t + kGemmBM - 1) / kGemmBM * kGemmBM;
  DevBuf a32((size_t)t * k * 4), a16((size_t)tp * k * 2, true);
  B2_CUDA(cudaMemcpy(a32.p, a, (size_t)t * k * 4, cudaMemcpyHostToDevice));
  int64_t na = (int64_t)t * k;
  f32_to_bf16_kernel<<<(unsigned)((na + 255) / 256), 256>>>(a32.as<float>(), a16.as<__nv_bfloat16>(), na);
  // weights in both layouts
  const int64_t n = n_logical;
  std::vector<uint32_t> t4((size_t)n * k / 8);
  std::vector<float> st((size_t)n);
  int64_t tiles = geglu ? ffn / 64 : (n + 127) / 128;
  std::vector<uint32_t> g4((size_t)tiles * 128 * k / 8);
  std::vector<float> sg((size_t)tiles * 128, 1.0f);
  if (geglu) {
    auto mapt = [ffn](int64_t r) { int64_t tile = r / 16, pair = tile / 2; return (tile & 1 ? ffn : (int64_t)0) + pair * 16 + (r % 16); };
    auto mapg = [ffn](int64_t r) { int64_t j = r / 128, c = r % 128; return (c & 1 ? ffn : (int64_t)0) + j * 64 + (c >> 1); };
    repack_w4t(packed_rows, n, k, mapt, t4.data());
    repack_w4g(packed_rows, tiles, k, mapg, g4.data());
    for (int64_t r = 0; r < n; ++r) st[r] = scales[mapt(r)];
    for (int64_t r = 0; r < tiles * 128; ++r) sg[r] = scales[mapg(r)];
  } else {
    B2_CHECK(n % 16 == 0, kInvalidArgument, "n must be a multiple of 16");
    repack_w4t(packed_rows, n, k, [](int64_t r) { return r; }, t4.data());
    repack_w4g(packed_rows, tiles, k, [n](int64_t r) { return r < n ? r : (int64_t)-1; }, g4.data());
    std::copy(scales, scales + n, st.begin());
    std::copy(scales, scales + n, sg.begin());
  }
  DevBuf wt(t4.size() * 4), wg(g4.size() * 4), dst((size_t)n * 4), dsg(sg.size() * 4), errw(4, true);
  B2_CUDA(cudaMemcpy(wt.p, t4.data(), t4.size() * 4, cudaMemcpyHostToDevice));
  B2_CUDA(cudaMemcpy(wg.p, g4.data(), g4.size() * 4, cudaMemcpyHostToDevice));
  B2_CUDA(cudaMemcpy(dst.p, st.data(), st.size() * 4, cudaMemcpyHostToDevice));
  B2_CUDA(cudaMemcpy(dsg.p, sg.data(), sg.size() * 4, cudaMemcpyHostToDevice));
  const int64_t out_cols = geglu ? ffn : n;
  DevBuf of((size_t)std::max(ksplit, 1) * t * n * 4, true), ob((size_t)t * out_cols * 2, true);
  ActMap tm{};
  if (mode == B200LM_GEMM_TCGEN05) tm = make_activation_map(a16.as<__nv_bfloat16>(), tp, (int)k);
  cudaEvent_t e0, e1;
  B2_CUDA(cudaEventCreate(&e0));
  B2_CUDA(cudaEventCreate(&e1));
  auto run = [&]() {
    launch_gemm(nullptr, mode, tm, a16.as<__nv_bfloat16>(), wt.as<uint4>(), dst.as<float>(), wg.as<uint8_t>(),
                dsg.as<float>(), t, (int)n, (int)k, ksplit, geglu, of.as<float>(), ob.as<__nv_bfloat16>(),
                errw.as<int>(), nullptr);
  };
  run();
  B2_CUDA(cudaDeviceSynchronize());
  if (repeat > 1) {
    B2_CUDA(cudaEventRecord(e0));
    for (int r = 0; r < repeat; ++r) run();
    B2_CUDA(cudaEventRecord(e1));
    B2_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    B2_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (ms_out) *ms_out = ms / repeat;
  } else if (ms_out) {
    *ms_out = 0.f;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  int errv = 0;
  B2_CUDA(cudaMemcpy(&errv, errw.p, 4, cudaMemcpyDeviceToHost));
  B2_CHECK(errv == 0, kDeadlineExceeded, "a bounded device-side wait gave up in the GEMM kernel");
  if (geglu) {
    DevBuf o32((size_t)t * out_cols * 4);
    int64_t no = (int64_t)t * out_cols;
    bf16_to_f32_kernel<<<(unsigned)((no + 255) / 256), 256>>>(ob.as<__nv_bfloat16>(), o32.as<float>(), no);
    B2_CUDA(cudaMemcpy(out, o32.p, (size_t)no * 4, cudaMemcpyDeviceToHost));
  } else {
    std::vector<float> parts((size_t)ksplit * t * n);
    B2_CUDA(cudaMemcpy(parts.data(), of.p, parts.size() * 4, cudaMemcpyDeviceToHost));
    for (int64_t i = 0; i < (int64_t)t * n; ++i) {
      float acc = 0.f;
      for (int s = 0; s < ksplit; ++s) acc += parts[(size_t)s * t * n + i];
      out[i] = acc;
    }
  }
}

int B200LmOps_GemmW4(int32_t device, int32_t mode, const uint8_t* packed, const float* scale, int64_t n, int64_t k,
                     const float* a, int32_t t, int32_t ksplit, int32_t repeat, float* out, float* ms_out, char** err) {
  OPS_BEGIN
  B2_CHECK(packed && scale && a && out, kInvalidArgument, "null pointer");
  check_matrix(n, k);
  B2_CHECK(t > 0, kInvalidArgument, "t must be positive");
  B2_CHECK(mode == B200LM_GEMM_CHECK || mode == B200LM_GEMM_TCGEN05, kInvalidArgument, "unknown GEMM mode");
  B2_CHECK(ksplit >= 1 && (k / 64) % ksplit == 0, kInvalidArgument, "ksplit must divide k/64");
  B2_CHECK(mode == B200LM_GEMM_TCGEN05 || ksplit == 1, kInvalidArgument, "the check GEMM does not split K");
  run_gemm_common(device, mode, packed, scale, n, k, false, 0, a, t, ksplit, repeat, out, ms_out);
  OPS_END
}

int B200LmOps_GemmGegluW4(int32_t device, int32_t mode, const uint8_t* gate_packed, const float* gate_scale,
                          const uint8_t* up_packed, const float* up_scale, int64_t ffn, int64_t k, const float* a,
                          int32_t t, float* out, char** err) {
  OPS_BEGIN
  B2_CHECK(gate_packed && gate_scale && up_packed && up_scale && a && out, kInvalidArgument, "null pointer");
  check_matrix(ffn, k);
  B2_CHECK(ffn % 64 == 0 && t > 0, kInvalidArgument, "ffn must be a multiple of 64");
  B2_CHECK(mode == B200LM_GEMM_CHECK || mode == B200LM_GEMM_TCGEN05, kInvalidArgument, "unknown GEMM mode");
  std::vector<uint8_t> rows((size_t)2 * ffn * k / 2);
  memcpy(rows.data(), gate_packed, (size_t)ffn * k / 2);
  memcpy(rows.data() + (size_t)ffn * k / 2, up_packed, (size_t)ffn * k / 2);
  std::vector<float> sc((size_t)2 * ffn);
  std::copy(gate_scale, gate_scale + ffn, sc.begin());
  std::copy(up_scale, up_scale + ffn, sc.begin() + ffn);
  run_gemm_common(device, mode, rows.data(), sc.data(), 2 * ffn, k, true, ffn, a, t, 1, 1, out, nullptr);
  OPS_END
}

int B200LmOps_Attention(int32_t device, const float* q, const float* k, const float* v, int32_t t, int32_t s,
                        int32_t hq, int32_t hkv, int32_t hd, int32_t qpos0, int32_t window, int32_t kv_bf16,
                        int32_t nsplit, int32_t repeat, float* out, float* ms_out, char** err) {
  OPS_BEGIN
  B2_CHECK(q && k && v && out, kInvalidArgument, "null pointer");
  B2_CHECK(t > 0 && s > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, kInvalidArgument, "bad shape");
  int G = hq / hkv;
  B2_CHECK(G == 1 || G == 2 || G == 4, kUnimplemented, "GQA group size must be 1, 2 or 4");
  B2_CHECK(hd == 32 || hd == 64 || hd == 128 || hd == 256, kUnimplemented, "head_dim must be 32/64/128/256");
  B2_CHECK(nsplit >= 1 && nsplit <= kMaxSplits, kInvalidArgument, "nsplit out of range");
  need_device(device);
  cudaDeviceProp prop;
  B2_CUDA(cudaGetDeviceProperties(&prop, device));
  ModelDims dm{};
  dm.hq = hq; dm.hkv = hkv; dm.hd = hd; dm.d = 64; dm.ffn = 64;
  dm.window = window > 0 ? window : 1 << 30;
  dm.kv_dtype = (kv_bf16 & 1) ? 1 : 0;
  dm.eps = 1e-6f;
  const bool decode = nsplit > 1;
  const bool priv = decode && (kv_bf16 & 2);     // every query reads its own physical copy of the cache
  const int kv_bf16_flags = kv_bf16;             // bit 2: the streaming kernel instead of the register-resident split kernel
  kv_bf16 &= 1;
  const int npages = (s + kPage - 1) / kPage;
  dm.max_ctx = npages * kPage;
  const size_t esz = kv_bf16 ? 2 : 4;
  const size_t pool = (size_t)npages * hkv * kPage * hd;
  const int ncopies = priv ? t : 1;
  B2_CHECK((double)pool * esz * 2 * ncopies <= 16e9, kInvalidArgument, "private caches would exceed 16 GB");
  DevBuf kp(pool * esz * ncopies, true), vp(pool * esz * ncopies, true), src((size_t)s * hkv * hd * 4);
  int64_t nkv = (int64_t)s * hkv * hd;
  for (int pass = 0; pass < 2; ++pass) {
    B2_CUDA(cudaMemcpy(src.p, pass ? v : k, (size_t)nkv * 4, cudaMemcpyHostToDevice));
    void* dstp = pass ? vp.p : kp.p;
    if (kv_bf16) fill_pages_kernel<__nv_bfloat16><<<(unsigned)((nkv + 255) / 256), 256>>>(src.as<float>(), reinterpret_cast<__nv_bfloat16*>(dstp), s, hkv, hd);
    else fill_pages_kernel<float><<<(unsigned)((nkv + 255) / 256), 256>>>(src.as<float>(), reinterpret_cast<float*>(dstp), s, hkv, hd);
    for (int c = 1; c < ncopies; ++c)
      B2_CUDA(cudaMemcpyAsync(reinterpret_cast<unsigned char*>(dstp) + (size_t)c * pool * esz, dstp, pool * esz,
                              cudaMemcpyDeviceToDevice, 0));
    B2_CUDA(cudaDeviceSynchronize());
  }
  // queries laid out like a QKV projection row: [q heads | k | v]; only q is read
  const int nqkv = (hq + 2 * hkv) * hd;
  std::vector<float> rows((size_t)t * nqkv, 0.f);
  for (int i = 0; i < t; ++i) memcpy(rows.data() + (size_t)i * nqkv, q + (size_t)i * hq * hd, sizeof(float) * hq * hd);
  DevBuf qd(rows.size() * 4), ptab(sizeof(int) * npages * ncopies), posd(sizeof(int) * t), errw(4, true);
  B2_CUDA(cudaMemcpy(qd.p, rows.data(), rows.size() * 4, cudaMemcpyHostToDevice));
  std::vector<int> pt((size_t)npages * ncopies), pos(t);
  for (int c = 0; c < ncopies; ++c)
    for (int i = 0; i < npages; ++i) pt[(size_t)c * npages + i] = c * npages + i;
  for (int i = 0; i < t; ++i) pos[i] = decode ? s - 1 : qpos0 + i;
  B2_CUDA(cudaMemcpy(ptab.p, pt.data(), sizeof(int) * pt.size(), cudaMemcpyHostToDevice));
  B2_CUDA(cudaMemcpy(posd.p, pos.data(), sizeof(int) * t, cudaMemcpyHostToDevice));
  DevBuf po((size_t)t * hkv * nsplit * G * hd * 4, true), pml((size_t)t * hkv * nsplit * G * 2 * 4, true);
  DevBuf od((size_t)t * hq * hd * 4, true);
  AttnJob j;
  memset(&j, 0, sizeof j);
  j.qkv = qd.as<float>();
  j.pos = posd.as<int>();
  j.page_table = ptab.as<int>();
  j.pages_per_seq = npages;
  j.seq_stride = priv ? 1 : 0;
  j.is_global = window > 0 ? 0 : 1;
  j.nsplit = nsplit;
  j.appended = 1;
  j.kv.k = kp.p;
  j.kv.v = vp.p;
  j.err = errw.as<int>();
  cudaEvent_t e0, e1;
  B2_CUDA(cudaEventCreate(&e0));
  B2_CUDA(cudaEventCreate(&e1));
  size_t smem_pf = sizeof(float) * ((size_t)(G + 2) * hd + (size_t)8 * G * (hd + 2));
  size_t smem_dec = sizeof(float) * ((size_t)(G + 2) * hd + (size_t)kDecWarps * G * (hd + 2));
  raise_dyn_smem(pf_attn_kernel, (size_t)(smem_pf));
  raise_dyn_smem(attn_decode_kernel, (size_t)(smem_dec));
  // decode, on request: the streaming kernel (K / V blocks by bulk copies into a shared-memory ring) + its combine
  DevBuf wpart((size_t)t * hkv * nsplit * G * (hd + 2) * 4, true);
  WideAttnArgs wa{qd.as<float>(), posd.as<int>(), ptab.as<int>(), npages, window > 0 ? 0 : 1, nsplit, 0, nullptr, nullptr, nullptr,
                  nullptr, LayerKv{kp.p, vp.p, nullptr, nullptr}, wpart.as<float>(), nullptr, errw.as<int>(), priv ? 1 : 0, 1,
                  nullptr, 2};
  const bool stream_decode = decode && (kv_bf16_flags & 4);
  auto run = [&]() {
    if (stream_decode) {
      launch_wide_attn(nullptr, dm, t, (size_t)prop.sharedMemPerBlockOptin, wa);
      wide_attn_combine_kernel<<<t * hq, 128>>>(wpart.as<float>(), nsplit, hq, hkv, hd, nullptr, od.as<float>());
    } else if (decode) {
      j.part_o = po.as<float>();
      j.part_ml = pml.as<float>();
      int items = t * hkv * nsplit;
      int grid = std::min(items, prop.multiProcessorCount);
      attn_decode_kernel<<<grid, kDecThreads, smem_dec>>>(dm, j, t);
      int total = t * hq * hd;
      attn_combine_kernel<<<(total + 255) / 256, 256>>>(po.as<float>(), pml.as<float>(), t, hq, hkv, hd, nsplit,
                                                        od.as<float>());
    } else {
      j.out_f32 = od.as<float>();
      pf_attn_kernel<<<t * hkv, 256, smem_pf>>>(dm, j);
    }
  };
  run();
  B2_CUDA(cudaGetLastError());
  B2_CUDA(cudaDeviceSynchronize());
  if (repeat > 1) {
    B2_CUDA(cudaEventRecord(e0));
    for (int r = 0; r < repeat; ++r) run();
    B2_CUDA(cudaEventRecord(e1));
    B2_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    B2_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (ms_out) *ms_out = ms / repeat;
  } else if (ms_out) {
    *ms_out = 0.f;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  B2_CUDA(cudaMemcpy(out, od.p, (size_t)t * hq * hd * 4, cudaMemcpyDeviceToHost));
  OPS_END
}

int B200LmOps_AttentionPrefillTc(int32_t device, const float* q, const float* k, const float* v, int32_t s, int32_t hq,
                                 int32_t hkv, int32_t hd, int32_t window, int32_t repeat, float* out, float* ms_out,
                                 char** err) {
  OPS_BEGIN
  B2_CHECK(q && k && v && out, kInvalidArgument, "null pointer");
  B2_CHECK(s > 0 && hq > 0 && hkv > 0 && hq % hkv == 0, kInvalidArgument, "bad shape");
  const int G = hq / hkv;
  B2_CHECK(G == 1 || G == 2 || G == 4, kUnimplemented, "GQA group size must be 1, 2 or 4");
  B2_CHECK(hd == 128 || hd == 256, kUnimplemented, "the tensor-core kernel takes head_dim 128 or 256");
  need_device(device);
  // static softmax shift: |q.k| / sqrt(hd) <= max|q| max|k| / sqrt(hd)
  double mq = 0.0, mk = 0.0;
  for (int64_t i = 0; i < (int64_t)s * hq; ++i) {
    double a = 0.0;
    for (int e = 0; e < hd; ++e) a += (double)q[i * hd + e] * q[i * hd + e];
    mq = std::max(mq, a);
  }
  for (int64_t i = 0; i < (int64_t)s * hkv; ++i) {
    double a = 0.0;
    for (int e = 0; e < hd; ++e) a += (double)k[i * hd + e] * k[i * hd + e];
    mk = std::max(mk, a);
  }
  const float bound = (float)(std::sqrt(mq) * std::sqrt(mk) / std::sqrt((double)hd) * 1.02);
  B2_CHECK(bound <= kFaMaxBound, kFailedPrecondition,
           "scores can reach " + std::to_string(bound) + ": beyond the static softmax shift of the tensor-core kernel");
  const int npages = (s + kPage - 1) / kPage;
  const int tp = (s + 127) / 128 * 128;
  const size_t pool = (size_t)npages * hkv * kPage * hd;
  DevBuf src((size_t)s * std::max(hq, hkv) * hd * 4), qb((size_t)tp * hq * hd * 2, true), kb(pool * 2, true),
      vtb(pool * 2, true), ob((size_t)tp * hq * hd * 2, true), o32((size_t)s * hq * hd * 4), ptab(sizeof(int) * npages),
      errw(4, true);
  const int64_t nq = (int64_t)s * hq * hd, nkv = (int64_t)s * hkv * hd;
  B2_CUDA(cudaMemcpy(src.p, q, (size_t)nq * 4, cudaMemcpyHostToDevice));
  scale_to_bf16_kernel<<<(unsigned)((nq + 255) / 256), 256>>>(src.as<float>(), qb.as<__nv_bfloat16>(), nq,
                                                            1.0f / std::sqrt((float)hd));
  B2_CUDA(cudaDeviceSynchronize());
  B2_CUDA(cudaMemcpy(src.p, k, (size_t)nkv * 4, cudaMemcpyHostToDevice));
  fill_pages_kernel<__nv_bfloat16><<<(unsigned)((nkv + 255) / 256), 256>>>(src.as<float>(), kb.as<__nv_bfloat16>(), s, hkv, hd);
  B2_CUDA(cudaDeviceSynchronize());
  B2_CUDA(cudaMemcpy(src.p, v, (size_t)nkv * 4, cudaMemcpyHostToDevice));
  fill_pages_vt_kernel<<<(unsigned)((nkv + 255) / 256), 256>>>(src.as<float>(), vtb.as<__nv_bfloat16>(), s, hkv, hd);
  B2_CUDA(cudaDeviceSynchronize());
  std::vector<int> pt(npages);
  for (int i = 0; i < npages; ++i) pt[i] = i;
  B2_CUDA(cudaMemcpy(ptab.p, pt.data(), sizeof(int) * npages, cudaMemcpyHostToDevice));
  CUtensorMap tm_q, tm_k, tm_vt;
  {
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)hq, (cuuint64_t)tp};
    cuuint64_t str[2] = {(cuuint64_t)hd * 2, (cuuint64_t)hq * hd * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(128 / G)};
    tm_q = make_bf16_map(qb.p, 3, dims, str, box);
    const cuuint64_t rows = (cuuint64_t)npages * hkv * kPage;
    cuuint64_t kd[2] = {(cuuint64_t)hd, rows};
    cuuint64_t ks[1] = {(cuuint64_t)hd * 2};
    cuuint32_t kbx[2] = {64, (cuuint32_t)kFaBN};
    tm_k = make_bf16_map(kb.p, 2, kd, ks, kbx);
    cuuint64_t vd[2] = {(cuuint64_t)kPage, (cuuint64_t)npages * hkv * hd};
    cuuint64_t vs[1] = {(cuuint64_t)kPage * 2};
    cuuint32_t vbx[2] = {(cuuint32_t)kFaBN, (cuuint32_t)hd};
    tm_vt = make_bf16_map(vtb.p, 2, vd, vs, vbx);
  }
  FaArgs fa{s, 0, hq, hkv, window > 0 ? window : 1 << 30, window > 0 ? 0 : 1, ptab.as<int>(), ob.as<__nv_bfloat16>(), bound,
            errw.as<int>()};
  const int TT = 128 / G;
  dim3 grid((s + TT - 1) / TT, hkv);
  if (hd == 256)
    raise_dyn_smem(flash_prefill_tc_kernel<256>, (size_t)(FaSmem<256>::kTotal));
  else
    raise_dyn_smem(flash_prefill_tc_kernel<128>, (size_t)(FaSmem<128>::kTotal));
  auto run = [&]() {
    if (hd == 256) flash_prefill_tc_kernel<256><<<grid, kFaThreads, FaSmem<256>::kTotal>>>(tm_q, tm_k, tm_vt, fa);
    else flash_prefill_tc_kernel<128><<<grid, kFaThreads, FaSmem<128>::kTotal>>>(tm_q, tm_k, tm_vt, fa);
  };
  run();
  B2_CUDA(cudaGetLastError());
  B2_CUDA(cudaDeviceSynchronize());
  if (repeat > 1) {
    cudaEvent_t e0, e1;
    B2_CUDA(cudaEventCreate(&e0));
    B2_CUDA(cudaEventCreate(&e1));
    B2_CUDA(cudaEventRecord(e0));
    for (int r = 0; r < repeat; ++r) run();
    B2_CUDA(cudaEventRecord(e1));
    B2_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    B2_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (ms_out) *ms_out = ms / repeat;
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  } else if (ms_out) {
    *ms_out = 0.f;
  }
  int errv = 0;
  B2_CUDA(cudaMemcpy(&errv, errw.p, 4, cudaMemcpyDeviceToHost));
  B2_CHECK(errv == 0, kDeadlineExceeded, "a bounded device-side wait gave up in the attention kernel");
  bf16_to_f32_kernel<<<(unsigned)((nq + 255) / 256), 256>>>(ob.as<__nv_bfloat16>(), o32.as<float>(), nq);
  B2_CUDA(cudaMemcpy(out, o32.p, (size_t)nq * 4, cudaMemcpyDeviceToHost));
  OPS_END
}

}  // extern "C"

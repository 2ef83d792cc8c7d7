// The B200 executor: model upload, paged KV cache, the reference's executor
// state machine (token hold-back, step counter, bucketed work groups) and the
// kernel orchestration for prefill and decode, behind the C ABI of b200lm.h.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>

#include <algorithm>
#include <cmath>
#include <fstream>
#include <memory>
#include <string>
#include <vector>

#include "../../include/b200lm.h"
#include "common.cuh"
#include "decode_ops.cuh"
#include "decode_stream.cuh"
#include "decode_fused.cuh"
#include "model_host.h"
#include "prefill_ops.cuh"
#include "prefill_gemm_ts.cuh"
#include "prefill_attn_tc.cuh"
#include "runtime.h"

namespace b200lm {

// ------------------------------------------------------------------ the model

Model::~Model() {
  cudaSetDevice(device);
  for (void* p : allocations) cudaFree(p);
}

void* Model::alloc(size_t bytes) {
  void* p = nullptr;
  B2_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 256)));
  allocations.push_back(p);
  return p;
}

template <typename T>
static T* upload(Model& m, const T* host, size_t count) {
  T* d = reinterpret_cast<T*>(m.alloc(count * sizeof(T)));
  B2_CUDA(cudaMemcpy(d, host, count * sizeof(T), cudaMemcpyHostToDevice));
  return d;
}

static const uint4* upload_w4t(Model& m, const uint8_t* packed, int64_t rows, int64_t K) {
  std::vector<uint32_t> buf((size_t)rows * K / 8);
  repack_w4t(packed, rows, K, [](int64_t r) { return r; }, buf.data());
  return reinterpret_cast<const uint4*>(upload(m, buf.data(), buf.size()));
}

// Host-side W4T tiles of a matrix.
template <typename RowMap>
static std::vector<uint32_t> w4t_host(const uint8_t* packed, int64_t rows, int64_t K, RowMap map) {
  std::vector<uint32_t> buf((size_t)rows * K / 8);
  repack_w4t(packed, rows, K, map, buf.data());
  return buf;
}
// Row-tile records: the KT tiles of a 16-row tile followed by its 16 scales.
static const unsigned char* upload_w4ts(Model& m, const std::vector<uint32_t>& w4t, const float* scale_tile_order, int64_t rows,
                                        int64_t K) {
  const int64_t RT = rows / 16, KT = K / 64, rec = KT * 512 + 64;
  std::vector<unsigned char> out((size_t)RT * rec);
  const unsigned char* src = reinterpret_cast<const unsigned char*>(w4t.data());
  for (int64_t rt = 0; rt < RT; ++rt) {
    memcpy(out.data() + rt * rec, src + rt * KT * 512, (size_t)KT * 512);
    memcpy(out.data() + rt * rec + KT * 512, scale_tile_order + rt * 16, 64);
  }
  return upload(m, out.data(), out.size());
}
// Tiles reordered [k_tile][row_tile].
static const uint4* upload_w4t_kmajor(Model& m, const std::vector<uint32_t>& w4t, int64_t rows, int64_t K) {
  const int64_t RT = rows / 16, KT = K / 64;
  std::vector<uint32_t> out(w4t.size());
  for (int64_t rt = 0; rt < RT; ++rt)
    for (int64_t kt = 0; kt < KT; ++kt) memcpy(out.data() + (kt * RT + rt) * 128, w4t.data() + (rt * KT + kt) * 128, 512);
  return reinterpret_cast<const uint4*>(upload(m, out.data(), out.size()));
}
// Tiles reordered [k slice][row_tile][k_tile within the slice].
static const uint4* upload_w4t_sliced(Model& m, const std::vector<uint32_t>& w4t, int64_t rows, int64_t K, int slices) {
  const int64_t RT = rows / 16, KT = K / 64, ktc = KT / slices;
  std::vector<uint32_t> out(w4t.size());
  for (int64_t sl = 0; sl < slices; ++sl)
    for (int64_t rt = 0; rt < RT; ++rt)
      memcpy(out.data() + ((sl * RT + rt) * ktc) * 128, w4t.data() + (rt * KT + sl * ktc) * 128, (size_t)ktc * 512);
  return reinterpret_cast<const uint4*>(upload(m, out.data(), out.size()));
}
static const float* upload_pair(Model& m, const float* a, const float* b, size_t n) {
  std::vector<float> v(2 * n, 0.f);
  memcpy(v.data(), a, n * 4);
  if (b) memcpy(v.data() + n, b, n * 4);
  return upload(m, v.data(), v.size());
}

// W4G with rows padded to 128; scales padded with 1.0.
static void upload_w4g(Model& m, const uint8_t* packed, const float* scale, int64_t rows, int64_t K,
                       const uint8_t** w_out, const float** s_out) {
  int64_t tiles = (rows + 127) / 128;
  std::vector<uint32_t> buf((size_t)tiles * 128 * K / 8);
  repack_w4g(packed, tiles, K, [rows](int64_t r) { return r < rows ? r : (int64_t)-1; }, buf.data());
  std::vector<float> sc((size_t)tiles * 128, 1.0f);
  std::copy(scale, scale + rows, sc.begin());
  *w_out = reinterpret_cast<const uint8_t*>(upload(m, buf.data(), buf.size()));
  *s_out = upload(m, sc.data(), sc.size());
}

std::shared_ptr<Model> Model::load(const uint8_t* image, size_t n, int device, bool want_tc) {
  WeightsRecord rec = locate_weights(image, n);
  auto m = std::make_shared<Model>();
  m->device = device;
  m->dims = rec.dims;
  const ModelDims& d = m->dims;
  B2_CUDA(cudaSetDevice(device));
  auto bytes = [&](const TensorEntry& e) { return rec.base + e.offset; };
  auto fvec = [&](const std::string& nm, size_t count) {
    const TensorEntry& e = rec.need(nm, 1);
    B2_CHECK(e.nbytes == count * 4, kInvalidArgument, "tensor has the wrong size: " + nm);
    return upload(*m, reinterpret_cast<const float*>(bytes(e)), count);
  };
  auto qmat = [&](const std::string& nm, int64_t rows, int64_t K) -> const TensorEntry& {
    const TensorEntry& e = rec.need(nm + ".q", 0);
    B2_CHECK((int64_t)e.rows == rows && (int64_t)e.cols == K && (int64_t)e.nbytes == rows * K / 2,
             kInvalidArgument, "matrix has the wrong shape: " + nm);
    return e;
  };
  // tied embedding: canonical rows for the gather, mma tiles for the head
  {
    const TensorEntry& e = qmat("embed", d.vocab, d.d);
    m->embed_rows = upload(*m, bytes(e), (size_t)e.nbytes);
    m->embed_scale = fvec("embed.scale", d.vocab);
    if (want_tc) {
      const TensorEntry& es = rec.need("embed.scale", 1);
      upload_w4g(*m, bytes(e), reinterpret_cast<const float*>(bytes(es)), d.vocab, d.d, &m->head_g, &m->head_gs);
    }
    auto ht = w4t_host(bytes(e), d.vocab, d.d, [](int64_t r) { return r; });
    m->head_w = reinterpret_cast<const uint4*>(upload(*m, ht.data(), ht.size()));
    m->head_ws = upload_w4ts(*m, ht, reinterpret_cast<const float*>(bytes(rec.need("embed.scale", 1))), d.vocab, d.d);
  }
  {
    int hps = 1;
    while ((hps * d.hd) % 64 != 0) ++hps;
    m->o_slices = d.hq % hps == 0 ? d.hq / hps : 1;
  }
  m->g_final = fvec("final_norm", d.d);
  {
    const float* g = reinterpret_cast<const float*>(bytes(rec.need("final_norm", 1)));
    m->gmax_final = 0.f;
    for (int k = 0; k < d.d; ++k) m->gmax_final = std::max(m->gmax_final, std::fabs(g[k]));
  }
  m->layers_host.resize(d.n_layers);
  m->gemm_host.resize(d.n_layers);
  m->chained_host.resize(d.n_layers);
  auto fptr = [&](const std::string& nm) { return reinterpret_cast<const float*>(bytes(rec.need(nm, 1))); };
  for (int i = 0; i < d.n_layers; ++i) {
    std::string p = "L" + std::to_string(i) + ".";
    LayerWeights& L = m->layers_host[i];
    LayerGemmWeights& Gm = m->gemm_host[i];
    memset(&L, 0, sizeof L);
    memset(&Gm, 0, sizeof Gm);
    const TensorEntry& eqkv = qmat(p + "wqkv", d.nqkv(), d.d);
    const TensorEntry& eo = qmat(p + "wo", d.d, d.nq());
    const TensorEntry& eg = qmat(p + "wgate", d.ffn, d.d);
    const TensorEntry& eu = qmat(p + "wup", d.ffn, d.d);
    const TensorEntry& ed = qmat(p + "wdown", d.d, d.ffn);
    const float* sqkv = reinterpret_cast<const float*>(bytes(rec.need(p + "wqkv.scale", 1)));
    const float* so = reinterpret_cast<const float*>(bytes(rec.need(p + "wo.scale", 1)));
    const float* sg = reinterpret_cast<const float*>(bytes(rec.need(p + "wgate.scale", 1)));
    const float* su = reinterpret_cast<const float*>(bytes(rec.need(p + "wup.scale", 1)));
    const float* sd = reinterpret_cast<const float*>(bytes(rec.need(p + "wdown.scale", 1)));
    ChainedLayer& Cl = m->chained_host[i];
    memset(&Cl, 0, sizeof Cl);
    auto ident = [](int64_t r) { return r; };
    {
      auto t = w4t_host(bytes(eqkv), d.nqkv(), d.d, ident);
      L.wqkv = reinterpret_cast<const uint4*>(upload(*m, t.data(), t.size()));
      Cl.wqkv_s = upload_w4ts(*m, t, sqkv, d.nqkv(), d.d);
    }
    L.sqkv = upload(*m, sqkv, d.nqkv());
    {
      auto t = w4t_host(bytes(eo), d.d, d.nq(), ident);
      L.wo = reinterpret_cast<const uint4*>(upload(*m, t.data(), t.size()));
      Cl.wo_s = upload_w4t_sliced(*m, t, d.d, d.nq(), m->o_slices);
    }
    L.so = upload(*m, so, d.d);
    {
      auto t = w4t_host(bytes(ed), d.d, d.ffn, ident);
      L.wdown = reinterpret_cast<const uint4*>(upload(*m, t.data(), t.size()));
      Cl.wdown_k = upload_w4t_kmajor(*m, t, d.d, d.ffn);
    }
    L.sdown = upload(*m, sd, d.d);
    Cl.gA = upload_pair(*m, fptr(p + "pre_attn"), i > 0 ? fptr("L" + std::to_string(i - 1) + ".post_ffn") : nullptr, d.d);
    Cl.gD = upload_pair(*m, fptr(p + "pre_ffn"), fptr(p + "post_attn"), d.d);
    Cl.qk = upload_pair(*m, fptr(p + "q_norm"), fptr(p + "k_norm"), d.hd);
    // gate and up share one matrix: canonical rows [gate ; up]
    std::vector<uint8_t> gu((size_t)2 * d.ffn * d.d / 2);
    memcpy(gu.data(), bytes(eg), (size_t)eg.nbytes);
    memcpy(gu.data() + eg.nbytes, bytes(eu), (size_t)eu.nbytes);
    const int64_t ffn = d.ffn;
    {   // decode layout: 16-row tiles alternate gate, up
      std::vector<uint32_t> buf((size_t)2 * ffn * d.d / 8);
      auto map = [ffn](int64_t r) {
        int64_t tile = r / 16, pair = tile / 2;
        return (tile & 1 ? ffn : (int64_t)0) + pair * 16 + (r % 16);
      };
      repack_w4t(gu.data(), 2 * ffn, d.d, map, buf.data());
      L.wgu = reinterpret_cast<const uint4*>(upload(*m, buf.data(), buf.size()));
      std::vector<float> sc((size_t)2 * ffn);
      for (int64_t r = 0; r < 2 * ffn; ++r) {
        int64_t src = map(r);
        sc[r] = src < ffn ? sg[src] : su[src - ffn];
      }
      L.sgu = upload(*m, sc.data(), sc.size());
      Cl.wgu_s = upload_w4ts(*m, buf, sc.data(), 2 * ffn, d.d);
    }
    auto gmax = [&](const std::string& nm) {
      const float* g = reinterpret_cast<const float*>(bytes(rec.need(nm, 1)));
      float m = 0.f;
      for (int k = 0; k < d.d; ++k) m = std::max(m, std::fabs(g[k]));
      return m;
    };
    L.gmax_pre_attn = gmax(p + "pre_attn");
    L.gmax_pre_ffn = gmax(p + "pre_ffn");
    L.g_pre_attn = fvec(p + "pre_attn", d.d);
    L.g_post_attn = fvec(p + "post_attn", d.d);
    L.g_pre_ffn = fvec(p + "pre_ffn", d.d);
    L.g_post_ffn = fvec(p + "post_ffn", d.d);
    {
      const float* gq = reinterpret_cast<const float*>(bytes(rec.need(p + "q_norm", 1)));
      const float* gk = reinterpret_cast<const float*>(bytes(rec.need(p + "k_norm", 1)));
      float mq = 0.f, mk = 0.f;
      for (int k = 0; k < d.hd; ++k) { mq = std::max(mq, std::fabs(gq[k])); mk = std::max(mk, std::fabs(gk[k])); }
      m->attn_bound.push_back(std::sqrt((float)d.hd) * mq * mk * 1.01f);
      L.attn_bound = m->attn_bound.back();
    }
    L.g_q = fvec(p + "q_norm", d.hd);
    L.g_k = fvec(p + "k_norm", d.hd);
    L.is_global = d.is_global(i) ? 1 : 0;
    if (want_tc) {
      upload_w4g(*m, bytes(eqkv), sqkv, d.nqkv(), d.d, &Gm.wqkv, &Gm.sqkv);
      upload_w4g(*m, bytes(eo), so, d.d, d.nq(), &Gm.wo, &Gm.so);
      upload_w4g(*m, bytes(ed), sd, d.d, d.ffn, &Gm.wdown, &Gm.sdown);
      // 128-row tiles of 64 ffn features: gate row of a feature, then its up row
      int64_t tiles = ffn / 64;
      std::vector<uint32_t> buf((size_t)tiles * 128 * d.d / 8);
      auto map = [ffn](int64_t r) {
        int64_t j = r / 128, c = r % 128;
        return (c & 1 ? ffn : (int64_t)0) + j * 64 + (c >> 1);
      };
      repack_w4g(gu.data(), tiles, d.d, map, buf.data());
      Gm.wgu = reinterpret_cast<const uint8_t*>(upload(*m, buf.data(), buf.size()));
      std::vector<float> sc((size_t)tiles * 128);
      for (int64_t r = 0; r < tiles * 128; ++r) {
        int64_t src = map(r);
        sc[r] = src < ffn ? sg[src] : su[src - ffn];
      }
      Gm.sgu = upload(*m, sc.data(), sc.size());
    }
  }
  m->has_tc = want_tc;
  m->layers_dev = upload(*m, m->layers_host.data(), m->layers_host.size());
  m->chained_dev = upload(*m, m->chained_host.data(), m->chained_host.size());
  m->gH = upload_pair(*m, fptr("final_norm"), fptr("L" + std::to_string(d.n_layers - 1) + ".post_ffn"), d.d);
  for (int t = 0; t < 2; ++t) {
    std::vector<float> c, s;
    build_rope_table(t ? d.rope_global : d.rope_local, d.hd, d.max_ctx, c, s);
    m->rope_cos[t] = upload(*m, c.data(), c.size());
    m->rope_sin[t] = upload(*m, s.data(), s.size());
    const int half = d.hd / 2;
    std::vector<float> cs((size_t)d.max_ctx * d.hd);
    for (int pz = 0; pz < d.max_ctx; ++pz) {
      memcpy(cs.data() + (size_t)pz * d.hd, c.data() + (size_t)pz * half, (size_t)half * 4);
      memcpy(cs.data() + (size_t)pz * d.hd + half, s.data() + (size_t)pz * half, (size_t)half * 4);
    }
    m->rope_cs[t] = upload(*m, cs.data(), cs.size());
  }
  return m;
}

// --------------------------------------------------------------- tensor maps

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    B2_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    B2_CHECK(p != nullptr && q == cudaDriverEntryPointSuccess, kInternal, "cuTensorMapEncodeTiled unavailable");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// bf16 row-major [rows][cols]; box = 64 columns x 128 rows, 128-byte swizzle.
ActMap make_activation_map(const __nv_bfloat16* base, int rows, int cols) {
  ActMap m;
  m.box128 = make_activation_map_box(base, rows, cols, kGemmBM);
  m.box64 = make_activation_map_box(base, rows, cols, 64);
  return m;
}

CUtensorMap make_activation_map_box(const __nv_bfloat16* base, int rows, int cols, int box_rows) {
  CUtensorMap tm;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)kGemmBK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = encode_tiled_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(base), dims,
                                 strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B2_CHECK(r == CUDA_SUCCESS, kInternal, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
  return tm;
}

// bf16 tensor of rank 2 or 3 (innermost dimension first), 128-byte swizzle.
static CUtensorMap make_bf16_map(const void* base, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes,
                                 const cuuint32_t* box) {
  CUtensorMap tm;
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = encode_tiled_fn()(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims,
                                 strides_bytes, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  B2_CHECK(r == CUDA_SUCCESS, kInternal, "cuTensorMapEncodeTiled failed: " + std::to_string((int)r));
  return tm;
}

// Launch with programmatic stream serialisation: the kernel may be scheduled
// while its predecessor in the stream is still running and does its set-up
// (barrier init, TMEM allocation) there; it calls pdl_wait() before it touches
// the predecessor's data.
template <typename... KArgs, typename... Args>
static void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  B2_CUDA(cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...));
}

// Split-K factor for a GEMM of `n_tiles` weight-row tiles over T tokens with KB
// 64-wide k blocks: the smallest divisor of KB (at least 4 k blocks per split,
// at most 8 splits) whose work units fill 90 % of the last round over the SMs,
// else the divisor that fills it best.
int pick_ksplit(int T, int n_tiles, int KB, int sms) {
  const int ntok = ts_tile_tokens(T);
  const int tiles = n_tiles * ((T + ntok - 1) / ntok);
  int best = 1;
  double best_eff = 0.0;
  for (int s = 1; s <= 8; ++s) {
    if (KB % s) continue;
    if (s > 1 && KB / s < 4) break;
    const int units = tiles * s;
    const double eff = (double)units / ((double)((units + sms - 1) / sms) * sms);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = s; }
    if (eff >= 0.9) break;
  }
  return best;
}

// Launches one int4 GEMM.  a_map must describe `A` ([rows >= T][K] bf16); a GEMM of at most 64 token rows
// uses a_map64, the same tensor with a 64-row box.
void launch_gemm(cudaStream_t st, int mode, const ActMap& a_map, const __nv_bfloat16* A,
                 const uint4* w4t, const float* s4t, const uint8_t* w4g, const float* s4g, int T, int N, int K,
                 int ksplit, bool geglu, float* outF, __nv_bfloat16* outB, int* err, int64_t* launches) {
  if (mode == B200LM_GEMM_TCGEN05) {
    GemmArgs g{w4g, s4g, T, N, K, ksplit, outF, outB, err};
    static int sms_of[64] = {0};              // per device: SM count, set once together with the kernel attributes
    int dev = 0;
    B2_CUDA(cudaGetDevice(&dev));
    B2_CHECK(dev >= 0 && dev < 64, kInternal, "device ordinal out of range");
    if (!sms_of[dev]) {
      raise_dyn_smem(gemm_w4_ts_kernel<0, 256>, (size_t)ts_smem(256));
      raise_dyn_smem(gemm_w4_ts_kernel<1, 256>, (size_t)ts_smem(256));
      raise_dyn_smem(gemm_w4_ts_kernel<0, 128>, (size_t)ts_smem(128));
      raise_dyn_smem(gemm_w4_ts_kernel<1, 128>, (size_t)ts_smem(128));
      raise_dyn_smem(gemm_w4_ts_kernel<0, 64>, (size_t)ts_smem(64));
      raise_dyn_smem(gemm_w4_ts_kernel<1, 64>, (size_t)ts_smem(64));
      B2_CUDA(cudaDeviceGetAttribute(&sms_of[dev], cudaDevAttrMultiProcessorCount, dev));
    }
    const int sms = sms_of[dev];
    const int ntok = ts_tile_tokens(T);
    const int total = ((N + kTsRows - 1) / kTsRows) * ((T + ntok - 1) / ntok) * ksplit;
    const int grid = total < sms ? total : sms;
#define B2_TS(EPI_, NTOK_, MAP_) launch_pdl(gemm_w4_ts_kernel<EPI_, NTOK_>, dim3(grid), dim3(ts_threads(NTOK_)), ts_smem(NTOK_), st, MAP_, g)
    if (ntok == 64) { if (geglu) B2_TS(1, 64, a_map.box64); else B2_TS(0, 64, a_map.box64); }
    else if (ntok == 128) { if (geglu) B2_TS(1, 128, a_map.box128); else B2_TS(0, 128, a_map.box128); }
    else { if (geglu) B2_TS(1, 256, a_map.box128); else B2_TS(0, 256, a_map.box128); }
#undef B2_TS
  } else {
    B2_CHECK(ksplit == 1, kInternal, "the check GEMM does not split K");
    dim3 grid(geglu ? N / 32 : N / 16, (T + 7) / 8);
    gemm_w4_simple_kernel<<<grid, 128, 0, st>>>(A, w4t, s4t, T, N, K, geglu ? 1 : 0, outF, outB);
  }
  B2_CUDA(cudaGetLastError());
  if (launches) ++*launches;
}

// --------------------------------------------------------------- the executor

static int round_up(int v, int a) { return (v + a - 1) / a * a; }

Executor::~Executor() {
  cudaSetDevice(device);
  if (stream) cudaStreamSynchronize(stream);
  if (graph_exec) cudaGraphExecDestroy(graph_exec);
  for (auto& g : wide_graphs) cudaGraphExecDestroy(g.second);
  if (tp_comm) {
    try { NcclApi::get().CommDestroy(tp_comm); } catch (...) {}
  }
  for (void* p : allocations) cudaFree(p);
  for (int i = 0; i < kTokRing; ++i)
    if (tok_ring_done[i]) cudaEventDestroy(tok_ring_done[i]);
  if (pinned) cudaFreeHost(pinned);
  if (own_stream && stream) cudaStreamDestroy(stream);
}

void* Executor::alloc(size_t bytes, bool zero) {
  void* p = nullptr;
  B2_CUDA(cudaMalloc(&p, std::max<size_t>(bytes, 256)));
  allocations.push_back(p);
  if (zero) B2_CUDA(cudaMemset(p, 0, std::max<size_t>(bytes, 256)));
  return p;
}

std::unique_ptr<Executor> Executor::create(std::shared_ptr<Model> model, const B200LmConfig& cfg) {
  auto e = std::unique_ptr<Executor>(new Executor());
  e->model = model;
  e->device = model->device;
  const ModelDims& d = model->dims;
  B2_CUDA(cudaSetDevice(e->device));
  cudaDeviceProp prop;
  B2_CUDA(cudaGetDeviceProperties(&prop, e->device));
  B2_CHECK(prop.major == 10, kFailedPrecondition,
           "this library is built for sm_100a (B200); device reports sm_" + std::to_string(prop.major) +
               std::to_string(prop.minor));
  e->n_sms = prop.multiProcessorCount;
  e->smem_optin = (size_t)prop.sharedMemPerBlockOptin;
  if (cfg.stream) {
    e->stream = reinterpret_cast<cudaStream_t>(cfg.stream);
  } else {
    B2_CUDA(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking));
    e->own_stream = true;
  }
  if (cfg.tp_world > 1) {
    B2_CHECK(cfg.tp_rank >= 0 && cfg.tp_rank < cfg.tp_world && cfg.tp_unique_id != nullptr, kInvalidArgument,
             "tensor parallelism needs 0 <= tp_rank < tp_world and the group's unique id");
    const NcclApi& nccl = NcclApi::get();
    NcclApi::UniqueId id;
    memcpy(&id, cfg.tp_unique_id, sizeof id);
    nccl.check(nccl.CommInitRank(&e->tp_comm, cfg.tp_world, id, cfg.tp_rank), "ncclCommInitRank");
    e->tp_rank = cfg.tp_rank;
    e->tp_world = cfg.tp_world;
  }
  e->max_num_tokens = cfg.max_num_tokens > 0 ? std::min(cfg.max_num_tokens, d.max_ctx) : d.max_ctx;
  B2_CHECK(cfg.prefill_gemm >= B200LM_GEMM_AUTO && cfg.prefill_gemm <= B200LM_GEMM_TCGEN05, kInvalidArgument,
           "prefill_gemm must be B200LM_GEMM_AUTO, _CHECK or _TCGEN05");
  e->prefill_gemm = cfg.prefill_gemm == B200LM_GEMM_AUTO ? (model->has_tc ? B200LM_GEMM_TCGEN05 : B200LM_GEMM_CHECK)
                                                          : cfg.prefill_gemm;
  B2_CHECK(e->prefill_gemm != B200LM_GEMM_TCGEN05 || model->has_tc, kFailedPrecondition,
           "tensor-core GEMM weights were not loaded for this model");
  B2_CHECK(cfg.page_order == 0 || cfg.page_order == 1, kInvalidArgument, "page_order must be 0 or 1");
  B2_CHECK(cfg.decode_mode >= B200LM_DECODE_AUTO && cfg.decode_mode <= B200LM_DECODE_WIDE, kInvalidArgument,
           "decode_mode must be one of B200LM_DECODE_*");
  e->decode_mode = cfg.decode_mode == B200LM_DECODE_AUTO ? B200LM_DECODE_CHAINED : cfg.decode_mode;
  // more sessions than the GEMV kernels carry per step: the projections run on the tensor-core GEMM
  if (cfg.n_sessions > kMaxCols && cfg.decode_mode == B200LM_DECODE_AUTO) e->decode_mode = B200LM_DECODE_WIDE;
  if (e->decode_mode == B200LM_DECODE_WIDE)
    B2_CHECK(e->prefill_gemm == B200LM_GEMM_TCGEN05 && cfg.tp_world <= 1, kFailedPrecondition,
             "the wide decode mode needs the tensor-core GEMM weights and no tensor parallelism");
  // a collective cannot run inside a persistent kernel: tensor-parallel decode is one kernel per phase
  if (cfg.tp_world > 1) e->decode_mode = B200LM_DECODE_PHASE_KERNELS;
  const int esz = d.kv_dtype == 0 ? 4 : 2;
  // ---- paged KV cache
  e->pages_per_seq = (e->max_num_tokens + kPage - 1) / kPage;     // the cache holds max_num_tokens positions per session
  e->n_sessions = cfg.n_sessions > 0 ? cfg.n_sessions : 1;
  {
    const int cap = e->decode_mode == B200LM_DECODE_WIDE ? kWideMax : kMaxCols;
    B2_CHECK(e->n_sessions <= cap, kInvalidArgument,
             "n_sessions exceeds the " + std::to_string(cap) + " sessions one decode step of this mode can carry");
  }
  const int max_cols = std::max(kMaxCols, e->n_sessions);
  e->parked.resize(e->n_sessions);
  const int total_pages = e->pages_per_seq * e->n_sessions;
  size_t pool = (size_t)total_pages * d.hkv * kPage * d.hd;
  e->kv_host.resize(d.n_layers);
  // tensor-core prefill attention: head_dim 128 / 256, and every layer's score bound small enough
  e->attn_tc = e->prefill_gemm == B200LM_GEMM_TCGEN05 && (d.hd == 128 || d.hd == 256);
  for (float b : model->attn_bound) e->attn_tc = e->attn_tc && b <= kFaMaxBound;
  for (int i = 0; i < d.n_layers; ++i) {
    e->kv_host[i].k = e->alloc(pool * esz, true);
    e->kv_host[i].v = e->alloc(pool * esz, true);
    e->kv_host[i].k16 = nullptr;
    e->kv_host[i].v16 = nullptr;
    if (e->attn_tc) {
      if (d.kv_dtype == 0) e->kv_host[i].k16 = reinterpret_cast<__nv_bfloat16*>(e->alloc(pool * 2, true));
      e->kv_host[i].v16 = reinterpret_cast<__nv_bfloat16*>(e->alloc(pool * 2, true));
    }
  }
  LayerKv* kvd = reinterpret_cast<LayerKv*>(e->alloc(sizeof(LayerKv) * d.n_layers, false));
  B2_CUDA(cudaMemcpy(kvd, e->kv_host.data(), sizeof(LayerKv) * d.n_layers, cudaMemcpyHostToDevice));
  e->kv_dev = kvd;
  // one page-table row per session, each over its own block of physical pages
  e->page_table_host.resize(total_pages);
  for (int sn = 0; sn < e->n_sessions; ++sn)
    for (int i = 0; i < e->pages_per_seq; ++i)
      e->page_table_host[(size_t)sn * e->pages_per_seq + i] =
          sn * e->pages_per_seq + (cfg.page_order == 1 ? e->pages_per_seq - 1 - i : i);
  int* ptd = reinterpret_cast<int*>(e->alloc(sizeof(int) * total_pages, false));
  B2_CUDA(cudaMemcpy(ptd, e->page_table_host.data(), sizeof(int) * total_pages, cudaMemcpyHostToDevice));
  e->page_table_dev = ptd;
  // ---- decode buffers
  DecodeArgs& a = e->dargs;
  memset(&a, 0, sizeof a);
  a.dims = d;
  a.ncols = 1;
  a.nterms = 3;
  // a split of 32 (local) / 64 (global, at full context) keys fits one staged chunk
  a.n_attn_splits_local = std::max(1, std::min(kMaxSplits, d.window / 32));
  a.n_attn_splits_global = std::max(1, std::min(kMaxSplits, d.max_ctx / 64));
  int hps = 1;
  while ((hps * d.hd) % 64 != 0) ++hps;
  B2_CHECK(d.hq % hps == 0, kUnimplemented, "q heads cannot be grouped into 64-wide slices");
  a.o_slices = d.hq / hps;
  while (a.o_slices > e->n_sms) a.o_slices /= 2;
  {   // the combine of split partials stages (m, l) of one head slice in 512 floats
    int heads_per_slice = d.hq / a.o_slices;
    int cap = std::max(1, 256 / heads_per_slice);
    a.n_attn_splits_local = std::min(a.n_attn_splits_local, cap);
    a.n_attn_splits_global = std::min(a.n_attn_splits_global, cap);
  }
  int KTd = d.ffn / 64;
  a.down_slices = 1;
  for (int s = 4; s >= 2; --s)
    if (KTd % s == 0 && (d.d / 16) * s <= e->n_sms) { a.down_slices = s; break; }
  a.layers = model->layers_dev;
  a.kv = e->kv_dev;
  a.page_table = e->page_table_dev;
  a.pages_per_seq = e->pages_per_seq;
  a.embed_rows = model->embed_rows;
  a.embed_scale = model->embed_scale;
  a.head_w = model->head_w;
  a.g_final = model->g_final;
  a.gmax_final = model->gmax_final;
  for (int t = 0; t < 2; ++t) { a.rope_cos[t] = model->rope_cos[t]; a.rope_sin[t] = model->rope_sin[t]; }
  a.chained = model->chained_dev;
  a.head_ws = model->head_ws;
  a.gH = model->gH;
  for (int t = 0; t < 2; ++t) a.rope_cs[t] = model->rope_cs[t];
  a.progress = reinterpret_cast<int*>(e->alloc(sizeof(int) * 2 * e->n_sms, true));   // live words, then a snapshot
  a.st = reinterpret_cast<DecodeState*>(e->alloc(sizeof(DecodeState), true));
  const int G = d.group();
  const int max_splits = std::max(a.n_attn_splits_local, a.n_attn_splits_global);
  a.xres[0] = reinterpret_cast<float*>(e->alloc(sizeof(float) * kMaxCols * d.d, true));
  a.xres[1] = reinterpret_cast<float*>(e->alloc(sizeof(float) * kMaxCols * d.d, true));
  a.qkv = reinterpret_cast<float*>(e->alloc(sizeof(float) * kMaxCols * d.nqkv(), true));
  a.part_o = reinterpret_cast<float*>(e->alloc(sizeof(float) * kMaxCols * d.hkv * max_splits * G * d.hd, true));
  a.part_ml = reinterpret_cast<float*>(e->alloc(sizeof(float) * kMaxCols * d.hkv * max_splits * G * 2, true));
  a.opart = reinterpret_cast<float*>(e->alloc(sizeof(float) * a.o_slices * kMaxCols * d.d, true));
  a.act = reinterpret_cast<float*>(e->alloc(sizeof(float) * kMaxCols * d.ffn, true));
  a.fpart = reinterpret_cast<float*>(e->alloc(sizeof(float) * a.down_slices * kMaxCols * d.d, true));
  a.logits = reinterpret_cast<float*>(e->alloc(sizeof(float) * max_cols * d.vocab, true));
  a.amax_val = reinterpret_cast<float*>(e->alloc(sizeof(float) * e->n_sms * kMaxCols, true));
  a.amax_idx = reinterpret_cast<int*>(e->alloc(sizeof(int) * e->n_sms * kMaxCols, true));
  a.step_capacity = d.max_ctx;
  a.step_tokens = reinterpret_cast<int*>(e->alloc(sizeof(int) * a.step_capacity * max_cols, true));
  if (e->decode_mode == B200LM_DECODE_WIDE) {
    int* ws = reinterpret_cast<int*>(e->alloc(sizeof(int) * 3 * kWideMax, true));
    e->wide = WideState{ws, ws + kWideMax, ws + 2 * kWideMax};
    {
      WideAttnArgs prep{};
      prep.ctas_per_sm = 2;
      launch_wide_attn(e->stream, d, 0, e->smem_optin, prep);
    }
    e->wide_part = reinterpret_cast<float*>(
        e->alloc(sizeof(float) * (size_t)e->n_sessions * d.hkv * kWideMaxSplits * d.group() * (d.hd + 2), true));
  }
  a.advance = 1;
  // the one-kernel-per-phase fallback drives one session; the persistent kernels carry all of them
  e->dec_smem = dec_smem_bytes(d, e->decode_mode == B200LM_DECODE_PHASE_KERNELS || e->decode_mode == B200LM_DECODE_PERSISTENT_BASIC
                                      ? e->n_sessions : 1);
  B2_CHECK(e->dec_smem <= (size_t)prop.sharedMemPerBlockOptin, kUnimplemented,
           "decode kernels need more shared memory than the device offers");
  raise_dyn_smem(decode_phase_kernel, (size_t)(e->dec_smem));
  raise_dyn_smem(decode_persistent_kernel, (size_t)(e->dec_smem));
  if (e->decode_mode == B200LM_DECODE_CHAINED) {
    // the chained kernel needs its ring to fit and the softmax shift of its attention to be usable;
    // otherwise the barrier-per-phase streaming kernel takes over
    FusedPlan pl;
    size_t smem = 0;
    const int nc = e->n_sessions, nt = nc * 3 <= kQCols ? 3 : kQCols / nc;
    const int cap = std::max(1, e->n_sms / (nc * d.hkv));
    bool ok = prop.cooperativeLaunch &&
              fused_make_plan(d, nc, nt, e->n_sms, a.o_slices, std::min(a.n_attn_splits_local, cap),
                              std::min(a.n_attn_splits_global, cap), (size_t)prop.sharedMemPerBlockOptin, &pl, &smem);
    for (float b : model->attn_bound) ok = ok && b <= kFaMaxBound;
    ok = ok && a.o_slices == model->o_slices;      // the sliced W_o copy was laid out for this split
    if (ok) {
      e->chained_ok = true;
      e->ll_bytes = (size_t)2 * pl.ll_words * sizeof(fu_u64);
      e->ll_dev = reinterpret_cast<fu_u64*>(e->alloc(e->ll_bytes, true));
    } else {
      e->decode_mode = B200LM_DECODE_PERSISTENT;
    }
  }
  if (e->decode_mode == B200LM_DECODE_PERSISTENT) {
    // staging halves take what shared memory the activation staging leaves, up to 96 KiB each
    size_t fixed = stream_fixed_bytes(d, e->n_sessions);
    long room = ((long)prop.sharedMemPerBlockOptin - (long)fixed - 2048) / 2;   // margin: static shared memory
    int half = (int)std::min<long>(room, 96 * 1024) / 1024 * 1024;
    bool ok = half > 0 && stream_model_fits(d, a.o_slices, a.down_slices, half) && prop.cooperativeLaunch;
    for (float b : model->attn_bound) ok = ok && b <= kFaMaxBound;   // its attention shifts the softmax by the bound
    if (ok) {
      e->stream_half = half;
      e->stream_smem = fixed + 2 * (size_t)half;
      const void* kfn = decode_stream_kernel_for(d);
      raise_dyn_smem(kfn, (size_t)(e->stream_smem));
      cudaFuncAttributes fa;
      B2_CUDA(cudaFuncGetAttributes(&fa, kfn));
      int occ = (size_t)fa.maxThreadsPerBlock >= (size_t)kStreamThreads ? 1 : 0;
      ok = occ >= 1;
    }
    if (!ok) e->decode_mode = B200LM_DECODE_PHASE_KERNELS;
  }
  B2_CHECK(e->n_sessions == 1 || e->decode_mode != B200LM_DECODE_PHASE_KERNELS, kUnimplemented,
           "several sessions per executor need a persistent decode kernel, which this model / device does not fit");
  if (e->decode_mode == B200LM_DECODE_PERSISTENT_BASIC) {
    int occ = 0;
    B2_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, decode_persistent_kernel, kDecThreads, e->dec_smem));
    if (occ < 1 || !prop.cooperativeLaunch) e->decode_mode = B200LM_DECODE_PHASE_KERNELS;
  }
  // ---- prefill buffers (rows padded to whole 128-token tiles, zero-filled)
  e->t_max = d.buckets[0];
  e->t_pad = round_up(e->t_max, kGemmBM);
  const size_t tp = e->t_pad;
  e->pf_tokens = reinterpret_cast<int*>(e->alloc(sizeof(int) * tp, true));
  e->pf_xres = reinterpret_cast<float*>(e->alloc(sizeof(float) * tp * d.d, true));
  e->pf_h = reinterpret_cast<__nv_bfloat16*>(e->alloc(2 * tp * d.d, true));
  e->pf_qkv = reinterpret_cast<float*>(e->alloc(sizeof(float) * tp * d.nqkv(), true));
  e->pf_attn = reinterpret_cast<__nv_bfloat16*>(e->alloc(2 * tp * d.nq(), true));
  e->pf_act = reinterpret_cast<__nv_bfloat16*>(e->alloc(2 * tp * d.ffn, true));
  e->pf_parts = reinterpret_cast<float*>(e->alloc(sizeof(float) * 8 * tp * d.d, true));
  if (e->attn_tc) {
    const int G = d.group();
    e->pf_q = reinterpret_cast<__nv_bfloat16*>(e->alloc(2 * tp * d.nq(), true));
    {
      cuuint64_t dims[3] = {(cuuint64_t)d.hd, (cuuint64_t)d.hq, (cuuint64_t)tp};
      cuuint64_t str[2] = {(cuuint64_t)d.hd * 2, (cuuint64_t)d.nq() * 2};
      cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(128 / G)};
      e->tm_q = make_bf16_map(e->pf_q, 3, dims, str, box);
    }
    const cuuint64_t rows = (cuuint64_t)total_pages * d.hkv * kPage;
    for (int i = 0; i < d.n_layers; ++i) {
      const void* kbase = d.kv_dtype == 0 ? (const void*)e->kv_host[i].k16 : (const void*)e->kv_host[i].k;
      cuuint64_t kd[2] = {(cuuint64_t)d.hd, rows};
      cuuint64_t ks[1] = {(cuuint64_t)d.hd * 2};
      cuuint32_t kb[2] = {64, (cuuint32_t)kFaBN};
      e->tm_k.push_back(make_bf16_map(kbase, 2, kd, ks, kb));
      cuuint64_t vd[2] = {(cuuint64_t)kPage, (cuuint64_t)total_pages * d.hkv * d.hd};
      cuuint64_t vs[1] = {(cuuint64_t)kPage * 2};
      cuuint32_t vb[2] = {(cuuint32_t)kFaBN, (cuuint32_t)d.hd};
      e->tm_vt.push_back(make_bf16_map(e->kv_host[i].v16, 2, vd, vs, vb));
    }
    if (d.hd == 256)
      raise_dyn_smem(flash_prefill_tc_kernel<256>, (size_t)(FaSmem<256>::kTotal));
    else
      raise_dyn_smem(flash_prefill_tc_kernel<128>, (size_t)(FaSmem<128>::kTotal));
  }
  raise_dyn_smem(pf_attn_kernel, sizeof(float) * ((size_t)(d.group() + 2) * d.hd + (size_t)8 * d.group() * (d.hd + 2)));
  if (e->prefill_gemm == B200LM_GEMM_TCGEN05) {
    e->tm_h = make_activation_map(e->pf_h, (int)tp, d.d);
    e->tm_attn = make_activation_map(e->pf_attn, (int)tp, d.nq());
    e->tm_act = make_activation_map(e->pf_act, (int)tp, d.ffn);
  }
  // page-locked staging: logits | kTokRing slices of prompt ids | sampled ids of a decode call | state words
  size_t pin = sizeof(float) * (size_t)d.vocab + sizeof(int) * (kTokRing * tp + (size_t)d.max_ctx * max_cols + 3 * kWideMax) + 4096;
  B2_CUDA(cudaMallocHost(&e->pinned, pin));
  e->pin_logits = reinterpret_cast<float*>(e->pinned);
  e->pin_ints = reinterpret_cast<int*>(e->pin_logits + d.vocab);
  e->pin_steps = e->pin_ints + (size_t)kTokRing * tp;
  e->pin_wide = e->pin_steps + (size_t)d.max_ctx * max_cols;
  e->pin_state = reinterpret_cast<DecodeState*>(e->pin_wide + 3 * kWideMax);
  for (int i = 0; i < kTokRing; ++i) B2_CUDA(cudaEventCreateWithFlags(&e->tok_ring_done[i], cudaEventDisableTiming));
  B2_CUDA(cudaDeviceSynchronize());
  return e;
}

void Executor::tp_allreduce(float* buf, size_t count) {
  const NcclApi& nccl = NcclApi::get();
  nccl.check(nccl.AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, tp_comm, stream), "ncclAllReduce");
}

void Executor::check_device_error(const char* where) {
  int err = 0;
  // err, barrier, steps_done and gave_up[4] are adjacent
  const size_t tail = sizeof(DecodeState) - offsetof(DecodeState, err);
  B2_CUDA(cudaMemcpyAsync(&pin_state->err, &dargs.st->err, tail, cudaMemcpyDeviceToHost, stream));
  B2_CUDA(cudaStreamSynchronize(stream));
  err = pin_state->err;
  if (err == kDevOk) return;
  // clear the words and the barrier count so the handle stays usable
  B2_CUDA(cudaMemsetAsync(&dargs.st->err, 0, tail, stream));
  B2_CUDA(cudaStreamSynchronize(stream));
  barrier_epoch = 0;
  std::string w(where);
  if (err == kDevBarrierTimeout) {
    std::string detail;
    const int* g = pin_state->gave_up;
    if (g[3] != 0)
      detail = " (first: " + std::string(g[3] == 1 ? "poll" : g[3] == 2 ? "ring slot" : "copy producer") + ", phase code " +
               std::to_string(g[0]) + ", layer / fill " + std::to_string(g[1]) + ", CTA " + std::to_string(g[2]) +
               (g[7] ? ", thread " + std::to_string(g[7] - 1) + " saw tag " + std::to_string((unsigned)g[4]) + " for " +
                           std::to_string((unsigned)g[5]) + " at word " + std::to_string(g[6]) + " (tag0 " +
                           std::to_string(last_plan_ll.tag0) + ", words per copy " + std::to_string(last_plan_ll.ll_words) +
                           ", ffn out at " + std::to_string(last_plan_ll.ll_f) + ")"
                     : std::string()) + ")";
    if (decode_mode == B200LM_DECODE_CHAINED) {
      std::vector<int> prog(n_sms);      // the snapshot taken by the first wait that gave up
      B2_CUDA(cudaMemcpy(prog.data(), dargs.progress + n_sms, sizeof(int) * n_sms, cudaMemcpyDeviceToHost));
      // a word is step * 10000 + phase code * 1000 + layer; order in time: step, layer, phase (the head phases 6, 7 last)
      auto when = [&](int w) {
        const int code = w / 1000 % 10, layer = code >= 6 ? model->dims.n_layers : w % 1000;
        return (long)(w / 10000) * 1000000L + (long)layer * 10 + code;
      };
      int lo = 0;
      for (int i = 1; i < n_sms; ++i)
        if (when(prog[i]) < when(prog[lo])) lo = i;
      // which words of the exchange area of that layer never received their tag
      if (ll_dev && last_plan_ll.ll_words > 0) {
        const FusedPlan& fp = last_plan_ll;
        const int layer = prog[lo] % 1000, step = prog[lo] / 10000, code = prog[lo] / 1000 % 10;
        const int L = model->dims.n_layers;
        const int src_layer = code == 1 ? layer - 1 : layer;       // phase A waits for the previous layer's reduce
        if (src_layer >= 0 && src_layer < L) {
          const unsigned want = fp.tag0 + (unsigned)step * (unsigned)(L + 1) + (unsigned)src_layer + 1u;
          std::vector<fu_u64> words((size_t)fp.ll_words);
          B2_CUDA(cudaMemcpy(words.data(), ll_dev + (size_t)(src_layer & 1) * fp.ll_words, sizeof(fu_u64) * fp.ll_words,
                             cudaMemcpyDeviceToHost));
          auto count = [&](int off, int n) {
            int bad = 0, first = -1;
            for (int i = 0; i < n; ++i)
              if ((unsigned)(words[off + i] >> 32) != want) { if (first < 0) first = i; ++bad; }
            return std::to_string(bad) + "/" + std::to_string(n) + (bad ? " (first " + std::to_string(first) + ")" : "");
          };
          const int d = model->dims.d;
          detail += "; untagged words of layer " + std::to_string(src_layer) + ": qkv " + count(fp.ll_qkv, last_ncols * model->dims.nqkv()) +
                    ", o " + count(fp.ll_o, dargs.o_slices * last_ncols * d) + ", ffn partials " +
                    count(fp.ll_fpart, fp.nprod * last_ncols * d) + ", ffn out " + count(fp.ll_f, last_ncols * d);
        }
      }
      detail += "; least advanced CTA " + std::to_string(lo) + " at phase code " + std::to_string(prog[lo] / 1000 % 10) + ", layer " +
                std::to_string(prog[lo] % 1000) + ", step " + std::to_string(prog[lo] / 10000);
    }
    throw Error{kDeadlineExceeded, w + ": a bounded device-side wait gave up" + detail};
  }
  if (err == kDevBadToken) throw Error{kInvalidArgument, w + ": token id outside the vocabulary"};
  if (err == kDevBadPosition) throw Error{kInvalidArgument, w + ": position outside the KV capacity"};
  throw Error{kInternal, w + ": device error word " + std::to_string(err)};
}

// ------------------------------------------------------------------- prefill

// x += rmsnorm(sum of split-K partials) * g_post ; h = bf16(rmsnorm(x) * g_pre)
static void launch_resid_norm(cudaStream_t st, const float* parts, int nparts, int T, const ModelDims& d,
                              const float* g_post, const float* g_pre, float* xres, __nv_bfloat16* h) {
  const int d4 = d.d / 4;
  const size_t stride = (size_t)T * d.d;
  const bool few = T <= 128;       // too few CTAs to hide the partial loads behind one another: fetch four partials per round
  if (d4 <= 128 * 3 && few)
    launch_pdl(pf_resid_norm_reg_kernel<128, 3, 4>, dim3(T), dim3(128), 0, st, parts, nparts, stride, d.d, d.eps, g_post, g_pre, xres, h);
  else if (d4 <= 128 * 3)
    launch_pdl(pf_resid_norm_reg_kernel<128, 3>, dim3(T), dim3(128), 0, st, parts, nparts, stride, d.d, d.eps, g_post, g_pre, xres, h);
  else if (d4 <= 256 * 3 && few)
    launch_pdl(pf_resid_norm_reg_kernel<256, 3, 4>, dim3(T), dim3(256), 0, st, parts, nparts, stride, d.d, d.eps, g_post, g_pre, xres, h);
  else if (d4 <= 256 * 6 && few)
    launch_pdl(pf_resid_norm_reg_kernel<256, 6, 4>, dim3(T), dim3(256), 0, st, parts, nparts, stride, d.d, d.eps, g_post, g_pre, xres, h);
  else if (d4 <= 256 * 6)
    launch_pdl(pf_resid_norm_reg_kernel<256, 6>, dim3(T), dim3(256), 0, st, parts, nparts, stride, d.d, d.eps, g_post, g_pre, xres, h);
  else
    pf_resid_norm_kernel<<<T, kPfThreads, sizeof(float) * d.d, st>>>(parts, nparts, stride, d.d, d.eps, g_post, g_pre,
                                                                    xres, h);
}

template <typename T>
static void launch_kv_append(cudaStream_t st, const ModelDims& d, int T_, const float* qkv, int nparts, int pos0, const int* pt,
                             const LayerWeights& L, const float* c, const float* s, const LayerKv& kv,
                             __nv_bfloat16* qout) {
  const int jobs = T_ * (d.hkv + (qout ? d.hq : 0));
  const int per = kKvaThreads / 32;
  const int grid = (jobs + per - 1) / per;
  const size_t stride = (size_t)T_ * d.nqkv();
#define B2_KVA(HD_) launch_pdl(pf_kv_append_kernel<T, HD_>, dim3(grid), dim3(kKvaThreads), 0, st, d, qkv, nparts, stride, T_, pos0, pt, L.g_k, c, s, kv, L.g_q, qout)
  switch (d.hd) {
    case 32: B2_KVA(32); break;
    case 64: B2_KVA(64); break;
    case 128: B2_KVA(128); break;
    default: B2_KVA(256); break;
  }
#undef B2_KVA
}

void Executor::run_prefill_chunk(const int* tokens, int T, int start) {
  const ModelDims& d = model->dims;
  B2_CHECK(T <= t_max, kInternal, "prefill chunk larger than the largest bucket");
  B2_CHECK(start + T <= max_num_tokens, kInvalidArgument,
           "Input token ids are too long. Exceeding the maximum number of tokens allowed: " +
               std::to_string(start + T) + " > " + std::to_string(max_num_tokens));
  // Token ids go through a ring of page-locked slices, one per queued chunk: a slice is rewritten only
  // after the host-to-device copy that reads it has completed (its event), so chunks queued back to
  // back without a wait (several work groups, wait_for_completion = false) never share staging memory.
  {
    const int slot = tok_ring_next;
    tok_ring_next = (tok_ring_next + 1) % kTokRing;
    if (tok_ring_used[slot]) B2_CUDA(cudaEventSynchronize(tok_ring_done[slot]));
    int* stage = pin_ints + (size_t)slot * t_pad;
    memcpy(stage, tokens, sizeof(int) * T);
    // the device-side id buffer is read by the first kernel of the chunk only; chunks are stream-ordered
    B2_CUDA(cudaMemcpyAsync(pf_tokens, stage, sizeof(int) * T, cudaMemcpyHostToDevice, stream));
    B2_CUDA(cudaEventRecord(tok_ring_done[slot], stream));
    tok_ring_used[slot] = true;
  }
  h2d_bytes += sizeof(int) * (size_t)T;
  int* err = &dargs.st->err;
  const int* ptab = page_table_dev + (size_t)active * pages_per_seq;     // the active session's pages
  const size_t sm_d = sizeof(float) * d.d;
  pf_embed_norm_kernel<<<T, kPfThreads, sm_d, stream>>>(pf_tokens, model->embed_rows, model->embed_scale,
                                                        model->layers_host[0].g_pre_attn, d.d, d.vocab, d.eps,
                                                        pf_xres, pf_h, err);
  ++launches;
  const int mode = prefill_gemm;
  const size_t attn_smem = sizeof(float) * ((size_t)(d.group() + 2) * d.hd + (size_t)8 * d.group() * (d.hd + 2));
  for (int li = 0; li < d.n_layers; ++li) {
    const LayerWeights& L = model->layers_host[li];
    const LayerGemmWeights& Gm = model->gemm_host[li];
    const float* cosT = model->rope_cos[L.is_global];
    const float* sinT = model->rope_sin[L.is_global];
    // split-K partials of the QKV rows go to the partials buffer (8 x d floats per token) and are summed by
    // the append kernel; the CUDA-core attention reads whole rows, so it keeps one split
    int ks_q = 1;
    if (mode == B200LM_GEMM_TCGEN05 && attn_tc) {
      ks_q = pick_ksplit(T, (d.nqkv() + kTsRows - 1) / kTsRows, d.d / 64, n_sms);
      if ((size_t)ks_q * d.nqkv() > (size_t)8 * d.d) ks_q = 1;
    }
    float* qkv_buf = ks_q > 1 ? pf_parts : pf_qkv;
    launch_gemm(stream, mode, tm_h, pf_h, L.wqkv, L.sqkv, Gm.wqkv, Gm.sqkv, T, d.nqkv(), d.d, ks_q, false, qkv_buf,
                nullptr, err, &launches);
    __nv_bfloat16* qout = attn_tc ? pf_q : nullptr;
    if (d.kv_dtype == 0) launch_kv_append<float>(stream, d, T, qkv_buf, ks_q, start, ptab, L, cosT, sinT, kv_host[li], qout);
    else launch_kv_append<__nv_bfloat16>(stream, d, T, qkv_buf, ks_q, start, ptab, L, cosT, sinT, kv_host[li], qout);
    ++launches;
    if (attn_tc) {
      FaArgs fa{T, start, d.hq, d.hkv, d.window, L.is_global, ptab, pf_attn, model->attn_bound[li], err};
      const int TT = 128 / d.group();
      dim3 grid((T + TT - 1) / TT, d.hkv);
      if (d.hd == 256) launch_pdl(flash_prefill_tc_kernel<256>, grid, dim3(kFaThreads), FaSmem<256>::kTotal, stream, tm_q, tm_k[li], tm_vt[li], fa);
      else launch_pdl(flash_prefill_tc_kernel<128>, grid, dim3(kFaThreads), FaSmem<128>::kTotal, stream, tm_q, tm_k[li], tm_vt[li], fa);
      ++launches;
    } else {
    AttnJob j;
    memset(&j, 0, sizeof j);
    j.qkv = pf_qkv;
    j.pos = nullptr;
    j.pos0 = start;
    j.page_table = ptab;
    j.pages_per_seq = pages_per_seq;
    j.seq_stride = 0;
    j.is_global = L.is_global;
    j.nsplit = 1;
    j.appended = 1;
    j.g_q = L.g_q;
    j.g_k = L.g_k;
    j.cosT = cosT;
    j.sinT = sinT;
    j.kv = kv_host[li];
    j.out_bf16 = pf_attn;
    j.err = err;
    pf_attn_kernel<<<T * d.hkv, 256, attn_smem, stream>>>(d, j);
    ++launches;
    }
    int ks_o = mode == B200LM_GEMM_TCGEN05 ? pick_ksplit(T, (d.d + kTsRows - 1) / kTsRows, d.nq() / 64, n_sms) : 1;
    launch_gemm(stream, mode, tm_attn, pf_attn, L.wo, L.so, Gm.wo, Gm.so, T, d.d, d.nq(), ks_o, false, pf_parts,
                nullptr, err, &launches);
    if (tp_world > 1) tp_allreduce(pf_parts, (size_t)ks_o * T * d.d);
    launch_resid_norm(stream, pf_parts, ks_o, T, d, L.g_post_attn, L.g_pre_ffn, pf_xres, pf_h);
    ++launches;
    launch_gemm(stream, mode, tm_h, pf_h, L.wgu, L.sgu, Gm.wgu, Gm.sgu, T, 2 * d.ffn, d.d, 1, true, nullptr, pf_act,
                err, &launches);
    int ks_d = mode == B200LM_GEMM_TCGEN05 ? pick_ksplit(T, (d.d + kTsRows - 1) / kTsRows, d.ffn / 64, n_sms) : 1;
    launch_gemm(stream, mode, tm_act, pf_act, L.wdown, L.sdown, Gm.wdown, Gm.sdown, T, d.d, d.ffn, ks_d, false,
                pf_parts, nullptr, err, &launches);
    if (tp_world > 1) tp_allreduce(pf_parts, (size_t)ks_d * T * d.d);
    const float* g_next = li + 1 < d.n_layers ? model->layers_host[li + 1].g_pre_attn : nullptr;
    launch_resid_norm(stream, pf_parts, ks_d, T, d, L.g_post_ffn, g_next, pf_xres, pf_h);
    ++launches;
  }
  B2_CUDA(cudaGetLastError());
}

// llm_litert_compiled_model_executor.cc:157-276: a group of `len` ids runs the
// pending id (if any) followed by ids[0..len-2]; ids[len-1] becomes pending.
void Executor::prefill_group(const int* ids, int len) {
  std::vector<int> run;
  run.reserve(len);
  int start = current_step;
  for (int i = 0; i < len - 1;) {
    if (next_input_token != -1) {
      run.push_back(next_input_token);
      next_input_token = -1;
    } else {
      run.push_back(ids[i++]);
    }
    ++current_step;
  }
  next_input_token = ids[len - 1];
  if (!run.empty()) run_prefill_chunk(run.data(), (int)run.size(), start);
}

void Executor::prefill(const int* ids, int n, bool wait, const volatile int* cancel) {
  B2_CHECK(ids != nullptr, kInvalidArgument, "ids is null");
  B2_CHECK(n > 0, kInternal, "Prefill token ids must be non-empty.");
  B2_CUDA(cudaSetDevice(device));
  const ModelDims& d = model->dims;
  // Same bound the caller loop enforces before it reaches the executor
  // (runtime/core/pipeline.cc:249-255), checked before any work is queued.
  const int would_run = n - 1 + (next_input_token != -1 ? 1 : 0);
  B2_CHECK(current_step + would_run <= max_num_tokens, kInvalidArgument,
           "Input token ids are too long. Exceeding the maximum number of tokens allowed: " +
               std::to_string(current_step + would_run) + " > " + std::to_string(max_num_tokens));
  auto groups = plan_work_groups(d.buckets, d.n_buckets, n);
  last_plan = groups;
  int used = 0;
  for (auto& g : groups) {
    if (cancel && *cancel) throw Error{kCancelled, "Prefill cancelled."};
    prefill_group(ids + used, g.second);
    used += g.second;
  }
  B2_CHECK(used == n, kInternal, "Work groups not covering the entire prefill input.");
  if (wait) check_device_error("Prefill");
}

// -------------------------------------------------------------------- decode

// ncols sessions advance together, starting at `first_session` (default: the active one alone).
void Executor::launch_decode_steps(int nsteps, int ncols, int first_session) {
  const ModelDims& d = model->dims;
  const int ncta = n_sms;
  if (first_session < 0) first_session = active;
  if (decode_mode == B200LM_DECODE_WIDE) {
    launch_wide_steps(nsteps, ncols, first_session);
    return;
  }
  if (decode_mode == B200LM_DECODE_CHAINED) {
    DecodeArgs a = dargs;
    a.ncols = ncols;
    a.nterms = ncols * 3 <= kQCols ? 3 : kQCols / ncols;
    a.page_table = page_table_dev + (size_t)first_session * pages_per_seq;
    const int cap = std::max(1, ncta / (ncols * d.hkv));
    a.n_attn_splits_local = std::min(a.n_attn_splits_local, cap);
    a.n_attn_splits_global = std::min(a.n_attn_splits_global, cap);
    FusedPlan pl;
    size_t smem = 0;
    B2_CHECK(fused_make_plan(d, a.ncols, a.nterms, ncta, a.o_slices, a.n_attn_splits_local, a.n_attn_splits_global,
                             smem_optin, &pl, &smem),
             kInternal, "the chained decode kernel does not fit this launch");
    B2_CHECK((size_t)2 * pl.ll_words * sizeof(fu_u64) <= ll_bytes, kInternal, "exchange area too small");
    // tags grow by one per (step, layer) and once more per step; start over (area cleared) long before they wrap
    const unsigned need = (unsigned)nsteps * (unsigned)(d.n_layers + 1) + 2u;
    if (ll_tag > 0xF0000000u - need) {
      B2_CUDA(cudaMemsetAsync(ll_dev, 0, ll_bytes, stream));
      ll_tag = 0;
    }
    pl.tag0 = ll_tag;
    ll_tag += need;
    last_plan_ll = pl;
    last_ncols = a.ncols;
    const void* kfn = decode_fused_kernel_for(d);
    raise_dyn_smem(kfn, smem);
    fu_u64* ll = ll_dev;
    void* params[] = {&a, &pl, &ll, &nsteps};
    cudaError_t le = cudaLaunchCooperativeKernel(kfn, dim3(ncta), dim3(kFuThreads), params, smem, stream);
    if (le != cudaSuccess) {
      cudaGetLastError();
      cudaFuncAttributes fa{};
      cudaFuncGetAttributes(&fa, kfn);
      int occ = -1;
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kfn, kFuThreads, smem);
      throw Error{kInternal, std::string("chained decode kernel launch: ") + cudaGetErrorString(le) + " (registers " +
                                 std::to_string(fa.numRegs) + ", static shared " + std::to_string(fa.sharedSizeBytes) +
                                 ", dynamic shared " + std::to_string(smem) + ", max threads " +
                                 std::to_string(fa.maxThreadsPerBlock) + ", blocks per SM " + std::to_string(occ) + ")"};
    }
    launches += 1;
    return;
  }
  if (decode_mode == B200LM_DECODE_PERSISTENT || decode_mode == B200LM_DECODE_PERSISTENT_BASIC) {
    DecodeArgs a = dargs;
    a.ncols = ncols;
    a.nterms = ncols * 3 <= kQCols ? 3 : kQCols / ncols;      // int8 terms per activation: 3, or 2 with 3-4 sessions
    a.page_table = page_table_dev + (size_t)first_session * pages_per_seq;
    // one CTA per (session, kv head, split)
    const int cap = std::max(1, ncta / (ncols * d.hkv));
    a.n_attn_splits_local = std::min(a.n_attn_splits_local, cap);
    a.n_attn_splits_global = std::min(a.n_attn_splits_global, cap);
    unsigned epoch0 = barrier_epoch;
    if (decode_mode == B200LM_DECODE_PERSISTENT) {
      int half = stream_half;
      void* params[] = {&a, &nsteps, &epoch0, &half};
      B2_CUDA(cudaLaunchCooperativeKernel(decode_stream_kernel_for(d), dim3(ncta), dim3(kStreamThreads), params,
                                          stream_smem, stream));
    } else {
      void* params[] = {&a, &nsteps, &epoch0};
      B2_CUDA(cudaLaunchCooperativeKernel((void*)decode_persistent_kernel, dim3(ncta), dim3(kDecThreads), params,
                                          dec_smem, stream));
    }
    barrier_epoch += (unsigned)nsteps * (unsigned)(5 * d.n_layers + 2) * (unsigned)ncta;
    launches += 1;
    return;
  }
  B2_CHECK(ncols == 1, kFailedPrecondition, "batched decode needs a persistent decode mode");
  B2_CHECK(n_sessions == 1, kFailedPrecondition, "several sessions per executor need a persistent decode mode");
  if (tp_world > 1) {
    // the same phases, launched one by one, with the ranks' partial O and down outputs summed in between
    for (int s = 0; s < nsteps; ++s) {
      for (int li = 0; li < d.n_layers; ++li)
        for (int ph = kPhQkv; ph <= kPhDown; ++ph) {
          decode_phase_kernel<<<ncta, kDecThreads, dec_smem, stream>>>(dargs, ph, li);
          if (ph == kPhOproj) tp_allreduce(dargs.opart, (size_t)dargs.o_slices * dargs.ncols * d.d);
          if (ph == kPhDown) tp_allreduce(dargs.fpart, (size_t)dargs.down_slices * dargs.ncols * d.d);
        }
      decode_phase_kernel<<<ncta, kDecThreads, dec_smem, stream>>>(dargs, kPhHead, 0);
      decode_phase_kernel<<<1, kDecThreads, dec_smem, stream>>>(dargs, kPhArgmax, ncta);
    }
    B2_CUDA(cudaGetLastError());
    launches += (int64_t)nsteps * (5 * d.n_layers + 2);
    return;
  }
  if (!graph_exec) {
    cudaGraph_t graph;
    B2_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    for (int li = 0; li < d.n_layers; ++li)
      for (int ph = kPhQkv; ph <= kPhDown; ++ph)
        decode_phase_kernel<<<ncta, kDecThreads, dec_smem, stream>>>(dargs, ph, li);
    decode_phase_kernel<<<ncta, kDecThreads, dec_smem, stream>>>(dargs, kPhHead, 0);
    decode_phase_kernel<<<1, kDecThreads, dec_smem, stream>>>(dargs, kPhArgmax, ncta);
    B2_CUDA(cudaStreamEndCapture(stream, &graph));
    B2_CUDA(cudaGraphInstantiate(&graph_exec, graph, 0));
    cudaGraphDestroy(graph);
  }
  for (int s = 0; s < nsteps; ++s) B2_CUDA(cudaGraphLaunch(graph_exec, stream));
  launches += (int64_t)nsteps * (5 * d.n_layers + 2);
}

// One wide step for sessions [first, first + nb): the token rows of the GEMMs are the sessions.
void Executor::wide_step(int nb, int first) {
  const ModelDims& d = model->dims;
  int* err = &dargs.st->err;
  const int mode = B200LM_GEMM_TCGEN05;
  // key splits so that few sessions still fill the SMs: one CTA per (session, kv head, split)
  const int nsplit = std::max(1, std::min(kWideMaxSplits, 2 * n_sms / std::max(1, nb * d.hkv)));   // two CTAs per SM
  // The streaming kernel runs two CTAs per SM over key splits; with well over one (session, kv head) pair per SM
  // the plain-load kernel, several CTAs resident per SM and no splits, was measured faster (64 sessions of the 4B shape).
  const bool stream_attn = nb * d.hkv * 2 <= n_sms * 3;
  const size_t attn_smem = sizeof(float) * ((size_t)(d.group() + 2) * d.hd + (size_t)8 * d.group() * (d.hd + 2));
  pf_embed_norm_kernel<<<nb, kPfThreads, sizeof(float) * d.d, stream>>>(wide.tok, model->embed_rows, model->embed_scale,
                                                                        model->layers_host[0].g_pre_attn, d.d, d.vocab, d.eps,
                                                                        pf_xres, pf_h, err);
  int64_t* nl = &launches;
  ++*nl;
  for (int li = 0; li < d.n_layers; ++li) {
    const LayerWeights& L = model->layers_host[li];
    const LayerGemmWeights& Gm = model->gemm_host[li];
    // split K so that the few token rows still spread the weight tiles over the SMs; the attention reads whole rows
    int ks_q = pick_ksplit(nb, (d.nqkv() + kTsRows - 1) / kTsRows, d.d / 64, n_sms);
    if ((size_t)ks_q * d.nqkv() > (size_t)8 * d.d) ks_q = 1;
    launch_gemm(stream, mode, tm_h, pf_h, L.wqkv, L.sqkv, Gm.wqkv, Gm.sqkv, nb, d.nqkv(), d.d, ks_q, false,
                ks_q > 1 ? pf_parts : pf_qkv, nullptr, err, nl);
    const bool fold_parts = ks_q > 1 && stream_attn;       // the streaming attention sums the partials as it reads them
    if (ks_q > 1 && !fold_parts) {
      const size_t count = (size_t)nb * d.nqkv();
      wide_sum_parts_kernel<<<(unsigned)((count / 4 + 255) / 256), 256, 0, stream>>>(pf_parts, ks_q, count, count, pf_qkv);
      ++*nl;
    }
    if (stream_attn) {
    WideAttnArgs wa{fold_parts ? pf_parts : pf_qkv, wide.pos, page_table_dev + (size_t)first * pages_per_seq, pages_per_seq, L.is_global, nsplit, 0,
                    L.g_q, L.g_k, model->rope_cos[L.is_global], model->rope_sin[L.is_global], kv_host[li], wide_part, pf_attn, err,
                    1, 0, nullptr, 2, fold_parts ? ks_q : 1, (size_t)nb * d.nqkv()};
    launch_wide_attn(stream, d, nb, smem_optin, wa);
    ++*nl;
    if (nsplit > 1) {
      wide_attn_combine_kernel<<<nb * d.hq, 128, 0, stream>>>(wide_part, nsplit, d.hq, d.hkv, d.hd, pf_attn, nullptr);
      ++*nl;
    }
    } else {
      AttnJob j;
      memset(&j, 0, sizeof j);
      j.qkv = pf_qkv;
      j.pos = wide.pos;
      j.page_table = page_table_dev + (size_t)first * pages_per_seq;
      j.pages_per_seq = pages_per_seq;
      j.seq_stride = 1;
      j.is_global = L.is_global;
      j.nsplit = 1;
      j.appended = 0;                               // the kernel norms, rotates and appends this step's K / V rows
      j.g_q = L.g_q;
      j.g_k = L.g_k;
      j.cosT = model->rope_cos[L.is_global];
      j.sinT = model->rope_sin[L.is_global];
      j.kv = kv_host[li];
      j.out_bf16 = pf_attn;
      j.err = err;
      pf_attn_kernel<<<nb * d.hkv, 256, attn_smem, stream>>>(d, j);
      ++*nl;
    }
    const int ks_o = pick_ksplit(nb, (d.d + kTsRows - 1) / kTsRows, d.nq() / 64, n_sms);
    launch_gemm(stream, mode, tm_attn, pf_attn, L.wo, L.so, Gm.wo, Gm.so, nb, d.d, d.nq(), ks_o, false, pf_parts, nullptr, err, nl);
    launch_resid_norm(stream, pf_parts, ks_o, nb, d, L.g_post_attn, L.g_pre_ffn, pf_xres, pf_h);
    ++*nl;
    launch_gemm(stream, mode, tm_h, pf_h, L.wgu, L.sgu, Gm.wgu, Gm.sgu, nb, 2 * d.ffn, d.d, 1, true, nullptr, pf_act, err, nl);
    const int ks_d = pick_ksplit(nb, (d.d + kTsRows - 1) / kTsRows, d.ffn / 64, n_sms);
    launch_gemm(stream, mode, tm_act, pf_act, L.wdown, L.sdown, Gm.wdown, Gm.sdown, nb, d.d, d.ffn, ks_d, false, pf_parts, nullptr,
                err, nl);
    const float* g_next = li + 1 < d.n_layers ? model->layers_host[li + 1].g_pre_attn : model->g_final;
    launch_resid_norm(stream, pf_parts, ks_d, nb, d, L.g_post_ffn, g_next, pf_xres, pf_h);
    ++*nl;
  }
  launch_gemm(stream, mode, tm_h, pf_h, nullptr, nullptr, model->head_g, model->head_gs, nb, d.vocab, d.d, 1, false, dargs.logits,
              nullptr, err, nl);
  wide_argmax_kernel<<<nb, kWideArgThreads, 0, stream>>>(dargs.logits, d.vocab, nb, wide, dargs.step_tokens);
  ++*nl;
  B2_CUDA(cudaGetLastError());
}

void Executor::launch_wide_steps(int nsteps, int nb, int first) {
  B2_CHECK(nb >= 1 && nb <= kWideMax && first >= 0 && first + nb <= n_sessions, kInternal, "wide step outside the sessions");
  B2_CHECK(model->head_g != nullptr, kFailedPrecondition, "the wide decode mode needs the tensor-core GEMM weights");
  if (nsteps == 1) {                                 // a single step is not worth a capture
    wide_step(nb, first);
    return;
  }
  auto key = std::make_pair(nb, first);
  auto it = wide_graphs.find(key);
  if (it == wide_graphs.end()) {
    const int64_t before = launches;
    cudaGraph_t graph;
    B2_CUDA(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
    try {
      wide_step(nb, first);
    } catch (...) {
      cudaGraph_t dead = nullptr;
      cudaStreamEndCapture(stream, &dead);
      if (dead) cudaGraphDestroy(dead);
      throw;
    }
    B2_CUDA(cudaStreamEndCapture(stream, &graph));
    cudaGraphExec_t exec = nullptr;
    B2_CUDA(cudaGraphInstantiate(&exec, graph, 0));
    cudaGraphDestroy(graph);
    wide_per_step = launches - before;
    launches = before;
    it = wide_graphs.emplace(key, exec).first;
  }
  for (int s = 0; s < nsteps; ++s) B2_CUDA(cudaGraphLaunch(it->second, stream));
  launches += (int64_t)nsteps * wide_per_step;
}

void Executor::push_decode_state(const int* tokens, const int* pos, int ncols) {
  if (decode_mode == B200LM_DECODE_WIDE) {
    B2_CUDA(cudaStreamSynchronize(stream));        // the staging words of the previous call have been read
    for (int c = 0; c < ncols; ++c) {
      pin_wide[c] = tokens[c];
      pin_wide[kWideMax + c] = pos[c];
      pin_wide[2 * kWideMax + c] = pos[c];
    }
    B2_CUDA(cudaMemcpyAsync(wide.tok, pin_wide, sizeof(int) * 3 * kWideMax, cudaMemcpyHostToDevice, stream));
    h2d_bytes += 2 * sizeof(int) * (size_t)ncols;
    return;
  }
  DecodeState* ps = pin_state;
  memset(ps, 0, sizeof(DecodeState));
  for (int c = 0; c < ncols; ++c) {
    ps->token[c] = tokens[c];
    ps->pos[c] = pos[c];
  }
  // token, pos, out_token: the first three arrays; err / barrier / steps_done handled separately
  B2_CUDA(cudaMemcpyAsync(dargs.st, ps, offsetof(DecodeState, err), cudaMemcpyHostToDevice, stream));
  B2_CUDA(cudaMemsetAsync(&dargs.st->steps_done, 0, sizeof(int), stream));
  h2d_bytes += 2 * sizeof(int) * (size_t)ncols;
}

int Executor::take_decode_id(const int* id_or_null) {
  int id = next_input_token;
  if (id_or_null) id = *id_or_null;
  B2_CHECK(id != -1, kInvalidArgument, "No id available to be decoded.");
  next_input_token = -1;
  B2_CHECK(current_step < max_num_tokens, kInvalidArgument, "Maximum kv-cache size reached.");
  return id;
}

void Executor::decode_logits(const int* id_or_null, float* host_logits) {
  B2_CHECK(host_logits != nullptr, kInvalidArgument, "logits destination is null");
  B2_CUDA(cudaSetDevice(device));
  int id = take_decode_id(id_or_null);
  push_decode_state(&id, &current_step, 1);
  launch_decode_steps(1);
  const size_t nb = sizeof(float) * (size_t)model->dims.vocab;
  // a page-locked destination takes the copy directly; pageable memory goes through the pinned staging
  cudaPointerAttributes pa{};
  const bool direct = cudaPointerGetAttributes(&pa, host_logits) == cudaSuccess && pa.type == cudaMemoryTypeHost;
  if (!direct) cudaGetLastError();
  B2_CUDA(cudaMemcpyAsync(direct ? host_logits : pin_logits, dargs.logits, nb, cudaMemcpyDeviceToHost, stream));
  d2h_bytes += nb;
  check_device_error("DecodeLogits");
  if (!direct) memcpy(host_logits, pin_logits, nb);
  ++current_step;
}

void Executor::decode_tokens(int nsteps, int* out_ids) {
  B2_CHECK(nsteps > 0, kInvalidArgument, "n_steps must be positive");
  B2_CUDA(cudaSetDevice(device));
  B2_CHECK(current_step + nsteps <= max_num_tokens, kInvalidArgument, "Maximum kv-cache size reached.");
  int id = take_decode_id(nullptr);
  push_decode_state(&id, &current_step, 1);
  launch_decode_steps(nsteps);
  int* dst = pin_steps;
  B2_CUDA(cudaMemcpyAsync(dst, dargs.step_tokens, sizeof(int) * (size_t)nsteps, cudaMemcpyDeviceToHost, stream));
  d2h_bytes += sizeof(int) * (size_t)nsteps;
  check_device_error("Decode");
  for (int s = 0; s < nsteps; ++s) {
    int t = dst[s];
    if (t < 0) t = 0;   // "The sampled token is casted to 0 to avoid crash."
    if (out_ids) out_ids[s] = t;
    next_input_token = t;
  }
  current_step += nsteps;
}

// All sessions take `nsteps` greedy steps together: one pass over the weights per step.
void Executor::decode_tokens_batch(int nsteps, int* out_ids) {
  B2_CHECK(nsteps > 0, kInvalidArgument, "n_steps must be positive");
  B2_CUDA(cudaSetDevice(device));
  const int keep = active;
  std::vector<int> tok(n_sessions), pos(n_sessions);
  for (int sn = 0; sn < n_sessions; ++sn) {        // validate every session before any state changes
    const int pending = sn == active ? next_input_token : parked[sn].next_input_token;
    const int step = sn == active ? current_step : parked[sn].current_step;
    B2_CHECK(pending != -1, kInvalidArgument, "No id available to be decoded (session " + std::to_string(sn) + ").");
    B2_CHECK(step + nsteps <= max_num_tokens, kInvalidArgument, "Maximum kv-cache size reached.");
  }
  for (int sn = 0; sn < n_sessions; ++sn) {
    select_session(sn);
    tok[sn] = take_decode_id(nullptr);
    pos[sn] = current_step;
  }
  push_decode_state(tok.data(), pos.data(), n_sessions);
  launch_decode_steps(nsteps, n_sessions, 0);
  int* dst = pin_steps;
  B2_CUDA(cudaMemcpyAsync(dst, dargs.step_tokens, sizeof(int) * (size_t)nsteps * n_sessions, cudaMemcpyDeviceToHost,
                          stream));
  d2h_bytes += sizeof(int) * (size_t)nsteps * n_sessions;
  check_device_error("Decode");
  for (int sn = 0; sn < n_sessions; ++sn) {
    select_session(sn);
    for (int s = 0; s < nsteps; ++s) {
      int t = dst[(size_t)s * n_sessions + sn];
      if (t < 0) t = 0;
      if (out_ids) out_ids[(size_t)s * n_sessions + sn] = t;
      next_input_token = t;
    }
    current_step += nsteps;
  }
  select_session(keep);
}

void Executor::trace_decode_step(int* out_id, long long* stamps, long long capacity, int* n_barriers, int* n_cta,
                                 int* khz) {
  const ModelDims& d = model->dims;
  B2_CHECK(decode_mode == B200LM_DECODE_PERSISTENT || decode_mode == B200LM_DECODE_PERSISTENT_BASIC ||
               decode_mode == B200LM_DECODE_CHAINED,
           kFailedPrecondition, "the decode timeline needs a persistent decode mode");
  B2_CUDA(cudaSetDevice(device));
  const int nb = 5 * d.n_layers + 2;
  const long long need = (long long)nb * n_sms * 10;     // 2 barrier stamps + 8 in-phase stamps
  B2_CHECK(stamps != nullptr && capacity >= need, kInvalidArgument,
           "stamps must hold " + std::to_string(need) + " int64 values");
  if (!trace_dev) trace_dev = reinterpret_cast<long long*>(alloc(sizeof(long long) * need, true));
  B2_CUDA(cudaMemsetAsync(trace_dev, 0, sizeof(long long) * need, stream));
  dargs.trace = trace_dev;
  dargs.trace_pts = trace_dev + (size_t)nb * n_sms * 2;
  try {
    decode_tokens(1, out_id);
  } catch (...) {
    dargs.trace = nullptr;
    dargs.trace_pts = nullptr;
    throw;
  }
  dargs.trace = nullptr;
  dargs.trace_pts = nullptr;
  B2_CUDA(cudaMemcpy(stamps, trace_dev, sizeof(long long) * need, cudaMemcpyDeviceToHost));
  *n_barriers = nb;
  *n_cta = n_sms;
  int rate = 0;
  B2_CUDA(cudaDeviceGetAttribute(&rate, cudaDevAttrClockRate, device));
  *khz = rate;
}

void Executor::reset() {
  current_step = 0;
  next_input_token = -1;
}

void Executor::select_session(int session) {
  B2_CHECK(session >= 0 && session < n_sessions, kInvalidArgument,
           "session " + std::to_string(session) + " out of range (the executor has " + std::to_string(n_sessions) + ")");
  if (session == active) return;
  parked[active] = SessionState{current_step, next_input_token, last_plan};
  current_step = parked[session].current_step;
  next_input_token = parked[session].next_input_token;
  last_plan = parked[session].last_plan;
  active = session;
}

void Executor::read_kv_row(int layer, int is_v, int kv_head, int pos, float* out, int* page, int* slot) {
  const ModelDims& d = model->dims;
  B2_CHECK(layer >= 0 && layer < d.n_layers && kv_head >= 0 && kv_head < d.hkv && pos >= 0 && pos < d.max_ctx,
           kInvalidArgument, "KV row index out of range");
  B2_CUDA(cudaSetDevice(device));
  B2_CUDA(cudaStreamSynchronize(stream));
  int pg = page_table_host[(size_t)active * pages_per_seq + pos / kPage], sl = pos % kPage;
  size_t off = (((size_t)pg * d.hkv + kv_head) * kPage + sl) * d.hd;
  const void* base = is_v ? kv_host[layer].v : kv_host[layer].k;
  if (d.kv_dtype == 0) {
    B2_CUDA(cudaMemcpy(out, reinterpret_cast<const float*>(base) + off, sizeof(float) * d.hd, cudaMemcpyDeviceToHost));
  } else {
    std::vector<__nv_bfloat16> tmp(d.hd);
    B2_CUDA(cudaMemcpy(tmp.data(), reinterpret_cast<const __nv_bfloat16*>(base) + off, 2 * d.hd, cudaMemcpyDeviceToHost));
    for (int i = 0; i < d.hd; ++i) out[i] = __bfloat162float(tmp[i]);
  }
  if (page) *page = pg;
  if (slot) *slot = sl;
}

}  // namespace b200lm

// ===================================================================== C ABI

using namespace b200lm;

struct B200LmExecutor {
  std::unique_ptr<Executor> impl;
};

static int fail(char** err, int code, const std::string& msg) {
  if (err) {
    *err = reinterpret_cast<char*>(malloc(msg.size() + 1));
    if (*err) memcpy(*err, msg.c_str(), msg.size() + 1);
  }
  return code;
}

#define B2_API_BEGIN \
  if (err) *err = nullptr; \
  try {
#define B2_API_END                                                     \
  }                                                                    \
  catch (const Error& e_) { return fail(err, e_.code, e_.msg); }       \
  catch (const std::exception& e_) { return fail(err, kInternal, e_.what()); } \
  catch (...) { return fail(err, kInternal, "unknown failure"); }      \
  return kOk;

static void require_gpu(int device) {
  int n = 0;
  cudaError_t r = cudaGetDeviceCount(&n);
  if (r != cudaSuccess || n <= 0) {
    cudaGetLastError();
    throw Error{kFailedPrecondition, "no CUDA device: this backend has no CPU fallback"};
  }
  B2_CHECK(device >= 0 && device < n, kInvalidArgument, "device ordinal out of range");
}

static B200LmConfig effective_config(const B200LmConfig* c) {
  B200LmConfig cfg;
  memset(&cfg, 0, sizeof cfg);
  if (c) memcpy(&cfg, c, std::min<size_t>(sizeof cfg, c->struct_size > 0 ? (size_t)c->struct_size : sizeof cfg));
  return cfg;
}

extern "C" {

int B200Lm_Create(const B200LmConfig* config, const void* bytes, uint64_t n_bytes, const char* path,
                  B200LmExecutor** out, char** err) {
  B2_API_BEGIN
  B2_CHECK(out != nullptr, kInvalidArgument, "out is null");
  *out = nullptr;
  B200LmConfig cfg = effective_config(config);
  std::vector<uint8_t> file;
  const uint8_t* p = reinterpret_cast<const uint8_t*>(bytes);
  if (!p) {
    B2_CHECK(path != nullptr, kInvalidArgument, "neither bytes nor a path were given");
    std::ifstream f(path, std::ios::binary | std::ios::ate);
    B2_CHECK(f.good(), kNotFound, std::string("cannot open ") + path);
    std::streamsize sz = f.tellg();
    f.seekg(0);
    file.resize((size_t)sz);
    f.read(reinterpret_cast<char*>(file.data()), sz);
    B2_CHECK(f.good(), kInternal, std::string("cannot read ") + path);
    p = file.data();
    n_bytes = (uint64_t)sz;
  }
  // Parse first: malformed input is reported as such even without a GPU.
  (void)locate_weights(p, (size_t)n_bytes);
  require_gpu(cfg.device);
  auto model = Model::load(p, (size_t)n_bytes, cfg.device, cfg.prefill_gemm != B200LM_GEMM_CHECK);
  auto h = new B200LmExecutor();
  try {
    h->impl = Executor::create(model, cfg);
  } catch (...) {
    delete h;
    throw;
  }
  *out = h;
  B2_API_END
}

int B200Lm_CreateShared(B200LmExecutor* owner, const B200LmConfig* config, B200LmExecutor** out, char** err) {
  B2_API_BEGIN
  B2_CHECK(owner && owner->impl && out, kInvalidArgument, "null handle");
  B200LmConfig cfg = effective_config(config);
  cfg.device = owner->impl->device;
  auto h = new B200LmExecutor();
  try {
    h->impl = Executor::create(owner->impl->model, cfg);
  } catch (...) {
    delete h;
    throw;
  }
  *out = h;
  B2_API_END
}

void B200Lm_Destroy(B200LmExecutor* e) { delete e; }

int B200Lm_Prefill(B200LmExecutor* e, const int32_t* ids, int32_t n, int32_t wait, const volatile int32_t* cancel,
                   char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->prefill(ids, n, wait != 0, cancel);
  B2_API_END
}

int B200Lm_DecodeLogits(B200LmExecutor* e, const int32_t* id, float* logits, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->decode_logits(id, logits);
  B2_API_END
}

int B200Lm_DecodeToken(B200LmExecutor* e, int32_t* out_id, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out_id, kInvalidArgument, "null argument");
  e->impl->decode_tokens(1, out_id);
  B2_API_END
}

int B200Lm_DecodeTokens(B200LmExecutor* e, int32_t n_steps, int32_t* out_ids, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->decode_tokens(n_steps, out_ids);
  B2_API_END
}

int B200Lm_PrefillSession(B200LmExecutor* e, int32_t session, const int32_t* ids, int32_t n, int32_t wait_for_completion,
                          const volatile int32_t* cancel_or_null, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->select_session(session);
  e->impl->prefill(ids, n, wait_for_completion != 0, reinterpret_cast<const volatile int*>(cancel_or_null));
  B2_API_END
}

int B200Lm_DecodeTokensBatch(B200LmExecutor* e, int32_t n_steps, int32_t* out_ids, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->decode_tokens_batch(n_steps, out_ids);
  B2_API_END
}

int B200Lm_SelectSession(B200LmExecutor* e, int32_t session, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->select_session(session);
  B2_API_END
}

int B200Lm_GetNumSessions(B200LmExecutor* e, int32_t* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out, kInvalidArgument, "null argument");
  *out = e->impl->n_sessions;
  B2_API_END
}

int B200Lm_Reset(B200LmExecutor* e, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  e->impl->reset();
  B2_API_END
}

int B200Lm_GetVocabSize(B200LmExecutor* e, int32_t* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out, kInvalidArgument, "null argument");
  *out = e->impl->model->dims.vocab;
  B2_API_END
}

int B200Lm_GetCurrentStep(B200LmExecutor* e, int32_t* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out, kInvalidArgument, "null argument");
  *out = e->impl->current_step + (e->impl->next_input_token == -1 ? 0 : 1);
  B2_API_END
}

int B200Lm_GetMaxNumTokens(B200LmExecutor* e, int32_t* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out, kInvalidArgument, "null argument");
  *out = e->impl->max_num_tokens;
  B2_API_END
}

int B200Lm_TpUniqueId(void* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(out != nullptr, kInvalidArgument, "out is null");
  const NcclApi& nccl = NcclApi::get();
  NcclApi::UniqueId id;
  nccl.check(nccl.GetUniqueId(&id), "ncclGetUniqueId");
  memcpy(out, &id, sizeof id);
  B2_API_END
}

int B200Lm_TpAllReduceProbe(B200LmExecutor* e, int64_t count, int32_t iters, float* ms_out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && ms_out && count > 0 && iters > 0, kInvalidArgument, "bad argument");
  Executor& x = *e->impl;
  B2_CHECK(x.tp_world > 1, kFailedPrecondition, "this executor is not tensor-parallel");
  B2_CUDA(cudaSetDevice(x.device));
  float* buf = nullptr;
  B2_CUDA(cudaMalloc(&buf, sizeof(float) * (size_t)count));
  B2_CUDA(cudaMemsetAsync(buf, 0, sizeof(float) * (size_t)count, x.stream));
  cudaEvent_t e0, e1;
  B2_CUDA(cudaEventCreate(&e0));
  B2_CUDA(cudaEventCreate(&e1));
  for (int i = 0; i < 3; ++i) x.tp_allreduce(buf, (size_t)count);
  B2_CUDA(cudaEventRecord(e0, x.stream));
  for (int i = 0; i < iters; ++i) x.tp_allreduce(buf, (size_t)count);
  B2_CUDA(cudaEventRecord(e1, x.stream));
  B2_CUDA(cudaEventSynchronize(e1));
  float ms = 0.f;
  B2_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  *ms_out = ms / (float)iters;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(buf);
  B2_API_END
}

int B200Lm_GetDecodeMode(B200LmExecutor* e, int32_t* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out, kInvalidArgument, "null argument");
  *out = e->impl->decode_mode;
  B2_API_END
}

const char* B200Lm_BackendName(void) { return "B200 CUDA (sm_100a)"; }

int B200Lm_Synchronize(B200LmExecutor* e, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl, kInvalidArgument, "null handle");
  B2_CUDA(cudaSetDevice(e->impl->device));
  e->impl->check_device_error("Synchronize");
  B2_API_END
}

int B200Lm_GetLastPrefillPlan(B200LmExecutor* e, int32_t* buckets, int32_t* lengths, int32_t capacity,
                              int32_t* n_groups, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && n_groups, kInvalidArgument, "null argument");
  const auto& plan = e->impl->last_plan;
  *n_groups = (int32_t)plan.size();
  for (int i = 0; i < (int)plan.size() && i < capacity; ++i) {
    if (buckets) buckets[i] = plan[i].first;
    if (lengths) lengths[i] = plan[i].second;
  }
  B2_API_END
}

int B200Lm_ReadKvRow(B200LmExecutor* e, int32_t layer, int32_t is_v, int32_t kv_head, int32_t pos, float* out_row,
                     int32_t* out_page, int32_t* out_slot, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out_row, kInvalidArgument, "null argument");
  e->impl->read_kv_row(layer, is_v, kv_head, pos, out_row, out_page, out_slot);
  B2_API_END
}

int B200Lm_TraceDecodeStep(B200LmExecutor* e, int32_t* out_id, int64_t* stamps, int64_t capacity,
                           int32_t* n_barriers, int32_t* n_cta, int32_t* sm_clock_khz, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out_id && n_barriers && n_cta && sm_clock_khz, kInvalidArgument, "null argument");
  e->impl->trace_decode_step(out_id, reinterpret_cast<long long*>(stamps), capacity, n_barriers, n_cta, sm_clock_khz);
  B2_API_END
}

int B200Lm_GetLaunchCount(B200LmExecutor* e, int64_t* out, char** err) {
  B2_API_BEGIN
  B2_CHECK(e && e->impl && out, kInvalidArgument, "null argument");
  *out = e->impl->launches;
  B2_API_END
}

}  // extern "C"

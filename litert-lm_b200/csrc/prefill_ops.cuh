// Prefill-side device code: T prompt tokens at consecutive positions.
//
// Per layer:  RMSNorm -> int4 GEMM (QKV) -> QK-RMSNorm + RoPE + KV append ->
// attention -> int4 GEMM (O) -> norm + residual + norm -> int4 GEMM (gate/up,
// GeGLU fused in the epilogue) -> int4 GEMM (down) -> norm + residual.
//
// The projections run on the 5th-generation tensor cores: activation tiles are
// fetched by TMA (128-byte swizzle), int4 weight tiles by 1-D bulk copies, a
// group of warps expands the int4 tile to bf16 in shared memory in the same
// swizzled layout, and one thread issues tcgen05.mma with the fp32 accumulator
// in tensor memory.  The per-output-channel scale is applied in the epilogue.
// Every mbarrier wait is bounded; a wait that gives up sets the error word and
// the kernel still runs to its end and frees its tensor memory.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "decode_ops.cuh"

namespace b200lm {

constexpr int kPfThreads = 128;

// ----------------------------------------------------- token-parallel kernels

__device__ __forceinline__ float pf_block_sum(float v, float* scratch) {
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += scratch[i];
  return t;
}

// xres[t] = dequant(E[token]) * sqrt(d) ; h[t] = bf16(rmsnorm(x) * g)
__global__ void __launch_bounds__(kPfThreads)
pf_embed_norm_kernel(const int* __restrict__ tokens, const uint8_t* __restrict__ embed_rows,
                     const float* __restrict__ embed_scale, const float* __restrict__ g, int d,
                     int vocab, float eps, float* __restrict__ xres, __nv_bfloat16* __restrict__ h,
                     int* err) {
  extern __shared__ float pf_sm[];
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  int tok = tokens[t];
  if (tok < 0 || tok >= vocab) {
    if (threadIdx.x == 0) atomicExch(err, (int)kDevBadToken);
    tok = 0;
  }
  const uint8_t* row = embed_rows + (size_t)tok * (d / 2);
  const float sc = embed_scale[tok] * sqrtf((float)d);
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    int b = row[i >> 1];
    int nib = (i & 1) ? (b >> 4) : (b & 0xF);
    float v = (float)(nib >= 8 ? nib - 16 : nib) * sc;
    pf_sm[i] = v;
    xres[(size_t)t * d + i] = v;
    ss += v * v;
  }
  ss = pf_block_sum(ss, scratch);
  float r = rsqrtf(ss / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    h[(size_t)t * d + i] = __float2bfloat16(pf_sm[i] * r * g[i]);
}

// x[t] += rmsnorm(sum_p parts[p][t]) * g_post ; h[t] = bf16(rmsnorm(x[t]) * g_pre) (if g_pre)
__global__ void __launch_bounds__(kPfThreads)
pf_resid_norm_kernel(const float* __restrict__ parts, int nparts, size_t part_stride, int d,
                     float eps, const float* __restrict__ g_post, const float* __restrict__ g_pre,
                     float* __restrict__ xres, __nv_bfloat16* __restrict__ h) {
  extern __shared__ float pf_sm[];
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float f = 0.f;
    for (int p = 0; p < nparts; ++p) f += parts[(size_t)p * part_stride + (size_t)t * d + i];
    pf_sm[i] = f;
    ss += f * f;
  }
  ss = pf_block_sum(ss, scratch);
  float r = rsqrtf(ss / (float)d + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = xres[(size_t)t * d + i] + pf_sm[i] * r * g_post[i];
    pf_sm[i] = v;
    xres[(size_t)t * d + i] = v;
    ss2 += v * v;
  }
  if (g_pre == nullptr) return;
  ss2 = pf_block_sum(ss2, scratch);
  float r2 = rsqrtf(ss2 / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x)
    h[(size_t)t * d + i] = __float2bfloat16(pf_sm[i] * r2 * g_pre[i]);
}

// K-RMSNorm + RoPE on the new keys, then K and V rows into the paged cache (and
// the bf16 operands of the tensor-core attention); with qout, also Q-RMSNorm +
// RoPE + 1/sqrt(hd) on the query heads into a bf16 [T][hq][hd] buffer.  One CTA
// per token; one warp per head (looped).
template <typename T>
__global__ void __launch_bounds__(256)
pf_kv_append_kernel(ModelDims dm, const float* __restrict__ qkv, int pos0,
                    const int* __restrict__ page_table, const float* __restrict__ g_k,
                    const float* __restrict__ cosT, const float* __restrict__ sinT, LayerKv kv,
                    const float* __restrict__ g_q, __nv_bfloat16* __restrict__ qout) {
  const int t = blockIdx.x, pos = pos0 + t;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const int hd = dm.hd, half = hd / 2;
  const float* row = qkv + (size_t)t * dm.nqkv();
  const int page = page_table[pos / kPage], slot = pos % kPage;
  T* kbase = reinterpret_cast<T*>(kv.k);
  T* vbase = reinterpret_cast<T*>(kv.v);
  const int nheads = dm.hkv + (qout ? dm.hq : 0);
  for (int h = warp; h < nheads; h += nwarps) {
    if (h >= dm.hkv) {           // a query head
      const int qh = h - dm.hkv;
      const float* qs = row + (size_t)qh * hd;
      float ss = 0.f;
      for (int e = lane; e < hd; e += 32) ss += qs[e] * qs[e];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)hd + dm.eps) * rsqrtf((float)hd);
      __nv_bfloat16* dst = qout + ((size_t)t * dm.hq + qh) * hd;
      for (int e = lane; e < half; e += 32) {
        float a0 = qs[e] * r * g_q[e], b0 = qs[e + half] * r * g_q[e + half];
        float cs = cosT[(size_t)pos * half + e], sn = sinT[(size_t)pos * half + e];
        dst[e] = __float2bfloat16(a0 * cs - b0 * sn);
        dst[e + half] = __float2bfloat16(b0 * cs + a0 * sn);
      }
      continue;
    }
    const int kh = h;
    const float* ks = row + dm.nq() + (size_t)kh * hd;
    const float* vs = row + dm.nq() + dm.nkv() + (size_t)kh * hd;
    size_t off = (((size_t)page * dm.hkv + kh) * kPage + slot) * hd;
    float ss = 0.f;
    for (int e = lane; e < hd; e += 32) ss += ks[e] * ks[e];
    ss = warp_sum(ss);
    float r = rsqrtf(ss / (float)hd + dm.eps);
    for (int e = lane; e < half; e += 32) {
      float a0 = ks[e] * r * g_k[e], b0 = ks[e + half] * r * g_k[e + half];
      float cs = cosT[(size_t)pos * half + e], sn = sinT[(size_t)pos * half + e];
      float k0 = a0 * cs - b0 * sn, k1 = b0 * cs + a0 * sn;
      float v0 = vs[e], v1 = vs[e + half];
      if constexpr (sizeof(T) == 4) {
        kbase[off + e] = k0; kbase[off + e + half] = k1;
        vbase[off + e] = v0; vbase[off + e + half] = v1;
        if (kv.k16) { kv.k16[off + e] = __float2bfloat16(k0); kv.k16[off + e + half] = __float2bfloat16(k1); }
      } else {
        kbase[off + e] = __float2bfloat16(k0); kbase[off + e + half] = __float2bfloat16(k1);
        vbase[off + e] = __float2bfloat16(v0); vbase[off + e + half] = __float2bfloat16(v1);
      }
      if (kv.v16) {
        size_t vt = (((size_t)page * dm.hkv + kh) * hd + e) * kPage + slot;
        kv.v16[vt] = __float2bfloat16(v0);
        kv.v16[vt + (size_t)half * kPage] = __float2bfloat16(v1);
      }
    }
  }
}

// Attention for T queries against the cache (keys already appended): one CTA
// per (query, kv head), all G query heads of the group together.
__global__ void __launch_bounds__(256)
pf_attn_kernel(ModelDims dm, AttnJob job) {
  extern __shared__ __align__(16) float attn_sm[];
  int it = blockIdx.x;
  int kvh = it % dm.hkv, qi = it / dm.hkv;
  attn_dispatch(dm, job, attn_sm, qi, kvh, 0);
}

// ------------------------------------------------------------ check GEMM
// C[t][n] = scale[n] * sum_k W[n][k] * A[t][k] straight from the mma-tiled
// weights, one thread per (row of a 16-row tile, token).  Slow; used for shapes
// the tensor-core kernel does not take and as its on-device cross-check.
__global__ void __launch_bounds__(128)
gemm_w4_simple_kernel(const __nv_bfloat16* __restrict__ A, const uint4* __restrict__ w,
                      const float* __restrict__ wscale, int T, int N, int K, int geglu,
                      float* __restrict__ outF, __nv_bfloat16* __restrict__ outB) {
  const int r = threadIdx.x & 15, tt = threadIdx.x >> 4;
  const int t = blockIdx.y * 8 + tt;
  const int KT = K / 64;
  if (t >= T) return;
  const __nv_bfloat16* a = A + (size_t)t * K;
  if (!geglu) {
    const int rt = blockIdx.x;
    float acc = 0.f;
    for (int kt = 0; kt < KT; ++kt) {
      const uint4* tile = w + ((size_t)rt * KT + kt) * 32;
      for (int k = 0; k < 64; ++k) acc += (float)w4t_element(tile, r, k) * __bfloat162float(a[kt * 64 + k]);
    }
    outF[(size_t)t * N + rt * 16 + r] = acc * wscale[rt * 16 + r];
  } else {
    const int p = blockIdx.x;   // tile pair: gate tile 2p, up tile 2p+1
    float ag = 0.f, au = 0.f;
    for (int kt = 0; kt < KT; ++kt) {
      const uint4* tg = w + ((size_t)(2 * p) * KT + kt) * 32;
      const uint4* tu = w + ((size_t)(2 * p + 1) * KT + kt) * 32;
      for (int k = 0; k < 64; ++k) {
        float x = __bfloat162float(a[kt * 64 + k]);
        ag += (float)w4t_element(tg, r, k) * x;
        au += (float)w4t_element(tu, r, k) * x;
      }
    }
    float gate = ag * wscale[(2 * p) * 16 + r], up = au * wscale[(2 * p + 1) * 16 + r];
    outB[(size_t)t * (N / 2) + p * 16 + r] = __float2bfloat16(gelu_tanh(gate) * up);
  }
}

// ------------------------------------------------- tcgen05 / TMA primitives

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: false (and the error word set) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* err) {
  const uint32_t addr = smem_u32(bar);
  for (int tries = 0; tries < (1 << 22); ++tries) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((tries & 1023) == 1023 && *reinterpret_cast<volatile int*>(err) == (int)kDevBarrierTimeout) return false;
  }
  atomicExch(err, (int)kDevBarrierTimeout);
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand tile, rows of 128 bytes (64 bf16), 128-byte swizzle: 8-row
// groups are 1024 bytes apart (SBO), LBO is not used by swizzled K-major tiles.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;                 // leading byte offset (unused) = 16 B
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
  d |= (uint64_t)1 << 46;                 // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}
// kind::f16, bf16 x bf16 -> fp32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------ int4 tensor-core GEMM

constexpr int kGemmBM = 128, kGemmBN = 128, kGemmBK = 64, kGemmStages = 3;
constexpr int kGemmDeqWarps = 8;
constexpr int kGemmThreads = 64 + 32 * kGemmDeqWarps;   // warp 0 loads, warp 1 issues MMA
constexpr int kGemmStageA = kGemmBM * kGemmBK * 2;      // 16384
constexpr int kGemmStageB = kGemmBN * kGemmBK * 2;      // 16384
constexpr int kGemmStageQ = kGemmBN * kGemmBK / 2;      // 4096
constexpr int kGemmSmem = kGemmStages * (kGemmStageA + kGemmStageB + kGemmStageQ) + 1024 + 256;

// Weight tiles ("W4G"): [n_tile][k_block] blocks of 128 rows x 32 bytes; a
// 32-bit word holds 8 consecutive k of one row as nibbles ordered
// k0,k2,k4,k6,k1,k3,k5,k7 (low to high), each stored as q + 8.
struct GemmArgs {
  const uint8_t* w;        // W4G tiles
  const float* wscale;     // per weight row, in tile order, padded to the tile grid
  int T, N, K;             // N = logical output columns (unpadded)
  int ksplit;              // grid.z; partial outputs [ksplit][T][N]
  float* outF;             // epilogue 0
  __nv_bfloat16* outB;     // epilogue 1 (GeGLU): [T][N/2]
  int* err;
};

template <int EPI>
__global__ void __launch_bounds__(kGemmThreads, 2)
gemm_w4_tc_kernel(const __grid_constant__ CUtensorMap tmA, GemmArgs g) {
  extern __shared__ unsigned char gsm_raw[];
  unsigned char* gsm = reinterpret_cast<unsigned char*>(((uintptr_t)gsm_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sA = gsm;
  unsigned char* sB = gsm + kGemmStages * kGemmStageA;
  unsigned char* sQ = sB + kGemmStages * kGemmStageB;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sQ + kGemmStages * kGemmStageQ);
  uint64_t* full_bar = bars;                       // [stages] TMA bytes landed
  uint64_t* deq_bar = bars + kGemmStages;          // [stages] bf16 weight tile written
  uint64_t* empty_bar = bars + 2 * kGemmStages;    // [stages] MMA finished with the stage
  uint64_t* acc_bar = bars + 3 * kGemmStages;      // accumulator complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * kGemmStages + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_tile = blockIdx.x, m_tile = blockIdx.y, ks = blockIdx.z;
  const int KB = g.K / kGemmBK;
  const int kb_per = KB / g.ksplit;
  const int kb0 = ks * kb_per;
  const int nkb = kb_per;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kGemmStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&deq_bar[s], kGemmDeqWarps);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kGemmBN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const uint8_t* wtile = g.w + ((size_t)n_tile * KB + kb0) * kGemmStageQ;
      for (int kb = 0; kb < nkb; ++kb) {
        int s = kb % kGemmStages, n = kb / kGemmStages;
        if (n > 0 && !mbar_wait(&empty_bar[s], (n - 1) & 1, g.err)) break;
        mbar_arrive_expect_tx(&full_bar[s], kGemmStageA + kGemmStageQ);
        tma_load_2d(sA + s * kGemmStageA, &tmA, (kb0 + kb) * kGemmBK, m_tile * kGemmBM, &full_bar[s]);
        bulk_load_1d(sQ + s * kGemmStageQ, wtile + (size_t)kb * kGemmStageQ, kGemmStageQ, &full_bar[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(kGemmBM, kGemmBN);
      bool ok = true;
      for (int kb = 0; kb < nkb && ok; ++kb) {
        int s = kb % kGemmStages, n = kb / kGemmStages;
        ok = mbar_wait(&full_bar[s], n & 1, g.err) && mbar_wait(&deq_bar[s], n & 1, g.err);
        if (!ok) break;
        tc_fence_after();
        uint64_t ad = umma_desc_sw128(smem_u32(sA + s * kGemmStageA));
        uint64_t bd = umma_desc_sw128(smem_u32(sB + s * kGemmStageB));
#pragma unroll
        for (int k = 0; k < kGemmBK / 16; ++k)   // 16 bf16 = 32 bytes along K per MMA
          umma_bf16(tmem_acc, ad + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
        umma_commit(&empty_bar[s]);
      }
      umma_commit(acc_bar);
    }
  } else {
    // ---- int4 -> bf16 expansion into the swizzled B tile
    const int dt = threadIdx.x - 64;            // 0..255
    const int row = dt >> 1, hrow = dt & 1;     // half a row (32 k) per thread
    bool ok = true;
    for (int kb = 0; kb < nkb && ok; ++kb) {
      int s = kb % kGemmStages, n = kb / kGemmStages;
      ok = mbar_wait(&full_bar[s], n & 1, g.err);
      if (ok && n > 0) ok = mbar_wait(&empty_bar[s], (n - 1) & 1, g.err);
      if (!ok) break;
      const uint4 q = *reinterpret_cast<const uint4*>(sQ + s * kGemmStageQ + row * 32 + hrow * 16);
      const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
      unsigned char* brow = sB + s * kGemmStageB + row * 128;
      const __nv_bfloat162 bias = __float2bfloat162_rn(136.0f);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t w = qw[j];
        uint32_t r[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t v = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;   // bf16(128 + nibble) pairs
          __nv_bfloat162 h = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias);
          r[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        int chunk = (hrow * 4 + j) ^ (row & 7);
        *reinterpret_cast<uint4*>(brow + chunk * 16) = make_uint4(r[0], r[1], r[2], r[3]);
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&deq_bar[s]);
    }
    // ---- epilogue: TMEM -> registers -> global
    if (mbar_wait(acc_bar, 0, g.err)) {
      tc_fence_after();
      const int quarter = warp & 3;               // TMEM lanes this warp may read
      const int second = (warp - 2) >> 2;         // 0 for warps 2..5, 1 for warps 6..9
      const int t = m_tile * kGemmBM + quarter * 32 + lane;
      const uint32_t lane_addr = tmem_acc + ((uint32_t)(quarter * 32) << 16);
      uint32_t v[32];
      if constexpr (EPI == 0) {
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
          int c0 = second * 64 + cb * 32;
          tmem_ld32(lane_addr + c0, v);
          int nbase = n_tile * kGemmBN + c0;
          if (t < g.T) {
            float* dst = g.outF + ((size_t)ks * g.T + t) * g.N + nbase;
            const float* sc = g.wscale + nbase;
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
              if (nbase + c + 3 < g.N) {
                float4 o = make_float4(__uint_as_float(v[c]) * sc[c], __uint_as_float(v[c + 1]) * sc[c + 1],
                                       __uint_as_float(v[c + 2]) * sc[c + 2], __uint_as_float(v[c + 3]) * sc[c + 3]);
                *reinterpret_cast<float4*>(dst + c) = o;
              } else {
                for (int e = 0; e < 4; ++e)
                  if (nbase + c + e < g.N) dst[c + e] = __uint_as_float(v[c + e]) * sc[c + e];
              }
            }
          }
        }
      } else {
        // tile columns 0..63 are gate rows, 64..127 the matching up rows
        uint32_t u[32];
        int c0 = second * 32;
        tmem_ld32(lane_addr + c0, v);
        tmem_ld32(lane_addr + 64 + c0, u);
        int fbase = n_tile * 64 + c0;            // index into the ffn dimension
        const int F = g.N / 2;
        if (t < g.T) {
          const float* scg = g.wscale + n_tile * kGemmBN + c0;
          const float* scu = scg + 64;
          __nv_bfloat16* dst = g.outB + (size_t)t * F + fbase;
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            float a0 = gelu_tanh(__uint_as_float(v[c]) * scg[c]) * (__uint_as_float(u[c]) * scu[c]);
            float a1 = gelu_tanh(__uint_as_float(v[c + 1]) * scg[c + 1]) * (__uint_as_float(u[c + 1]) * scu[c + 1]);
            if (fbase + c + 1 < F) {
              *reinterpret_cast<__nv_bfloat162*>(dst + c) = __floats2bfloat162_rn(a0, a1);
            } else if (fbase + c < F) {
              dst[c] = __float2bfloat16(a0);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(g.err) == (int)kDevBarrierTimeout) {
    // a wait gave up: let any bulk copy still in flight land before the CTA retires
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_acc, kGemmBN);
  }
}

}  // namespace b200lm

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
  pdl_wait();
  pdl_launch_dependents();
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

// Same as pf_resid_norm_kernel with the token's row in registers: one CTA of
// THREADS threads per token, MAXV float4 per thread, 16-byte loads, two block
// reductions.  Small CTAs keep many tokens in flight per SM, which is what
// hides the latency of the partial-sum loads.  With few tokens (the wide decode step) there are too few CTAs
// for that, so PU > 1 fetches PU partials per round of loads; the sums are taken in the same order.
template <int THREADS, int MAXV, int PU = 1>
__global__ void __launch_bounds__(THREADS)
pf_resid_norm_reg_kernel(const float* __restrict__ parts, int nparts, size_t part_stride, int d, float eps,
                         const float* __restrict__ g_post, const float* __restrict__ g_pre,
                         float* __restrict__ xres, __nv_bfloat16* __restrict__ h) {
  pdl_wait();
  pdl_launch_dependents();
  __shared__ float red[2][THREADS / 32];
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int d4 = d / 4;
  float4 f[MAXV], x[MAXV];
  float4* xr = reinterpret_cast<float4*>(xres + (size_t)t * d);
#pragma unroll
  for (int u = 0; u < MAXV; ++u) {
    const int i = threadIdx.x + THREADS * u;
    f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    x[u] = i < d4 ? xr[i] : f[u];
  }
  for (int p = 0; p < nparts; p += PU) {
    float4 v[PU][MAXV];
#pragma unroll
    for (int q = 0; q < PU; ++q) {
      const float4* src = reinterpret_cast<const float4*>(parts + (size_t)(p + q) * part_stride + (size_t)t * d);
#pragma unroll
      for (int u = 0; u < MAXV; ++u) {
        const int i = threadIdx.x + THREADS * u;
        v[q][u] = (p + q < nparts && i < d4) ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
    }
#pragma unroll
    for (int q = 0; q < PU; ++q) {
#pragma unroll
      for (int u = 0; u < MAXV; ++u) { f[u].x += v[q][u].x; f[u].y += v[q][u].y; f[u].z += v[q][u].z; f[u].w += v[q][u].w; }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < MAXV; ++u) ss += f[u].x * f[u].x + f[u].y * f[u].y + f[u].z * f[u].z + f[u].w * f[u].w;
  ss = warp_sum(ss);
  if (lane == 0) red[0][warp] = ss;
  __syncthreads();
  ss = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) ss += red[0][w];
  const float r = rsqrtf(ss / (float)d + eps);
  float ss2 = 0.f;
#pragma unroll
  for (int u = 0; u < MAXV; ++u) {
    const int i = threadIdx.x + THREADS * u;
    if (i < d4) {
      float4 gp = reinterpret_cast<const float4*>(g_post)[i];
      x[u].x += f[u].x * r * gp.x; x[u].y += f[u].y * r * gp.y; x[u].z += f[u].z * r * gp.z; x[u].w += f[u].w * r * gp.w;
      xr[i] = x[u];
      ss2 += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
    }
  }
  if (g_pre == nullptr) return;
  ss2 = warp_sum(ss2);
  if (lane == 0) red[1][warp] = ss2;
  __syncthreads();
  ss2 = 0.f;
#pragma unroll
  for (int w = 0; w < THREADS / 32; ++w) ss2 += red[1][w];
  const float r2 = rsqrtf(ss2 / (float)d + eps);
#pragma unroll
  for (int u = 0; u < MAXV; ++u) {
    const int i = threadIdx.x + THREADS * u;
    if (i < d4) {
      float4 gq = reinterpret_cast<const float4*>(g_pre)[i];
      __nv_bfloat162 a = __floats2bfloat162_rn(x[u].x * r2 * gq.x, x[u].y * r2 * gq.y);
      __nv_bfloat162 b = __floats2bfloat162_rn(x[u].z * r2 * gq.z, x[u].w * r2 * gq.w);
      uint2 w;
      w.x = *reinterpret_cast<uint32_t*>(&a);
      w.y = *reinterpret_cast<uint32_t*>(&b);
      reinterpret_cast<uint2*>(h + (size_t)t * d)[i] = w;
    }
  }
}

// V consecutive floats (V = 1, 2 or 4) with one load / store; p is V*4-byte aligned
template <int V>
__device__ __forceinline__ void ld_vec(const float* p, float (&o)[V]) {
  if constexpr (V == 4) { float4 v = *reinterpret_cast<const float4*>(p); o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w; }
  else if constexpr (V == 2) { float2 v = *reinterpret_cast<const float2*>(p); o[0] = v.x; o[1] = v.y; }
  else o[0] = *p;
}
template <int V>
__device__ __forceinline__ void st_vec(float* p, const float (&o)[V]) {
  if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  else if constexpr (V == 2) *reinterpret_cast<float2*>(p) = make_float2(o[0], o[1]);
  else *p = o[0];
}
template <int V>
__device__ __forceinline__ void st_vec(__nv_bfloat16* p, const float (&o)[V]) {
  if constexpr (V == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&a);
    w.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = w;
  } else if constexpr (V == 2) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(o[0], o[1]);
  } else {
    *p = __float2bfloat16(o[0]);
  }
}

// K-RMSNorm + RoPE on the new keys, then K and V rows into the paged cache (and
// the bf16 operands of the tensor-core attention); with qout, also Q-RMSNorm +
// RoPE + 1/sqrt(hd) on the query heads into a bf16 [T][hq][hd] buffer.  One
// warp per (token, head): job = token * nheads + head, kv heads first.  Lane l
// holds V consecutive elements of each half of the head (V = HD / 64, or one
// element on the low lanes for HD 32).  The QKV row may arrive as `nparts`
// split-K partial sums `part_stride` floats apart; they are added on load.
constexpr int kKvaThreads = 128;
template <typename T, int HD>
__global__ void __launch_bounds__(kKvaThreads, HD == 256 ? 8 : 10)
pf_kv_append_kernel(ModelDims dm, const float* __restrict__ qkv, int nparts, size_t part_stride, int ntok, int pos0,
                    const int* __restrict__ page_table, const float* __restrict__ g_k,
                    const float* __restrict__ cosT, const float* __restrict__ sinT, LayerKv kv,
                    const float* __restrict__ g_q, __nv_bfloat16* __restrict__ qout) {
  pdl_wait();
  pdl_launch_dependents();
  constexpr int V = HD >= 64 ? HD / 64 : 1;
  constexpr int half = HD / 2;
  const int lane = threadIdx.x & 31;
  const int nheads = dm.hkv + (qout ? dm.hq : 0);
  const int job = blockIdx.x * (kKvaThreads / 32) + (threadIdx.x >> 5);
  if (job >= ntok * nheads) return;
  const int t = job / nheads, h = job - t * nheads, pos = pos0 + t;
  const bool is_q = h >= dm.hkv;
  const int e0 = lane * V;
  const bool act = e0 < half;                                   // HD 32: lanes 16..31 idle
  // head offset within the QKV row: [q heads | k heads | v heads]
  const int col = is_q ? (h - dm.hkv) * HD : dm.nq() + h * HD;
  const float* row = qkv + (size_t)t * dm.nqkv() + col;
  float a[V], b[V], va[V], vb[V];
#pragma unroll
  for (int i = 0; i < V; ++i) a[i] = b[i] = va[i] = vb[i] = 0.f;
  if (act) {
    for (int p = 0; p < nparts; ++p) {
      const float* src = row + (size_t)p * part_stride;
      float x[V], y[V];
      ld_vec<V>(src + e0, x);
      ld_vec<V>(src + e0 + half, y);
#pragma unroll
      for (int i = 0; i < V; ++i) { a[i] += x[i]; b[i] += y[i]; }
      if (!is_q) {
        ld_vec<V>(src + dm.nkv() + e0, x);
        ld_vec<V>(src + dm.nkv() + e0 + half, y);
#pragma unroll
        for (int i = 0; i < V; ++i) { va[i] += x[i]; vb[i] += y[i]; }
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) ss += a[i] * a[i] + b[i] * b[i];
  ss = warp_sum(ss);
  float r = rsqrtf(ss / (float)HD + dm.eps);
  if (is_q) r *= rsqrtf((float)HD);
  if (!act) return;
  const float* gain = is_q ? g_q : g_k;
  float k0[V], k1[V];
  {
    float ga[V], gb[V], cs[V], sn[V];
    ld_vec<V>(gain + e0, ga);
    ld_vec<V>(gain + e0 + half, gb);
    ld_vec<V>(cosT + (size_t)pos * half + e0, cs);
    ld_vec<V>(sinT + (size_t)pos * half + e0, sn);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float a0 = a[i] * r * ga[i], b0 = b[i] * r * gb[i];
      k0[i] = a0 * cs[i] - b0 * sn[i];
      k1[i] = b0 * cs[i] + a0 * sn[i];
    }
  }
  if (is_q) {
    __nv_bfloat16* dst = qout + ((size_t)t * dm.hq + (h - dm.hkv)) * HD;
    st_vec<V>(dst + e0, k0);
    st_vec<V>(dst + e0 + half, k1);
    return;
  }
  const int page = page_table[pos / kPage], slot = pos % kPage;
  const size_t off = (((size_t)page * dm.hkv + h) * kPage + slot) * HD;
  T* kbase = reinterpret_cast<T*>(kv.k);
  T* vbase = reinterpret_cast<T*>(kv.v);
  st_vec<V>(kbase + off + e0, k0);
  st_vec<V>(kbase + off + e0 + half, k1);
  st_vec<V>(vbase + off + e0, va);
  st_vec<V>(vbase + off + e0 + half, vb);
  if constexpr (sizeof(T) == 4) {
    if (kv.k16) {
      st_vec<V>(kv.k16 + off + e0, k0);
      st_vec<V>(kv.k16 + off + e0 + half, k1);
    }
  }
  if (kv.v16) {
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const size_t vt = (((size_t)page * dm.hkv + h) * HD + e0 + i) * kPage + slot;
      kv.v16[vt] = __float2bfloat16(va[i]);
      kv.v16[vt + (size_t)half * kPage] = __float2bfloat16(vb[i]);
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

constexpr int kGemmBM = 128;                      // activation rows are padded to this
constexpr int kGemmBK = 64;                       // k block: one 128-byte swizzled row of bf16
constexpr int kGemmStageQ = 128 * kGemmBK / 2;    // one int4 weight block: 128 rows x 32 bytes

// Weight tiles ("W4G"): [n_tile][k_block] blocks of 128 rows x 32 bytes; a
// 32-bit word holds 8 consecutive k of one row as nibbles ordered
// k0,k2,k4,k6,k1,k3,k5,k7 (low to high), each stored as q + 8.
struct GemmArgs {
  const uint8_t* w;        // W4G tiles
  const float* wscale;     // per weight row, in tile order, padded to the tile grid
  int T, N, K;             // N = logical output columns (unpadded)
  int ksplit;              // K splits; partial outputs [ksplit][T][N]
  float* outF;             // epilogue 0
  __nv_bfloat16* outB;     // epilogue 1 (GeGLU): [T][N/2]
  int* err;
};

}  // namespace b200lm

// Wide lockstep decode: one greedy step for MANY sessions at once, with the projections on the
// tensor-core int4 GEMM of the prefill path (the sessions' current tokens are the GEMM's token rows)
// and one attention CTA per (session, kv head) over that session's own pages.  The weights stream
// once per step for the whole group, which is what a group of more sessions than the GEMV kernels
// carry (kMaxCols) needs.  Activations are bf16 as in prefill.
//
// This file holds the two small kernels the step adds to the prefill kernels; the step itself is
// Executor::launch_wide_steps.
#pragma once
#include <algorithm>
#include "decode_ops.cuh"
#include "prefill_ops.cuh"

namespace b200lm {

constexpr int kWideMax = 128;          // sessions of one wide step (half a token tile of the GEMM)
constexpr int kWideArgThreads = 1024;
constexpr int kWideMaxSplits = 8;     // key splits of one (session, kv head) in the wide attention

// Per-session state of a wide run, device resident: [0, n) token of the next step, [kWideMax, +n)
// its position, [2 kWideMax, +n) the position of the run's first step.
struct WideState {
  int* tok;
  int* pos;
  int* pos0;
};

// One CTA per session: arg-max of its logits row (lowest index among equal maxima, the rule of
// runtime/components/sampling_cpu_util.cc:32-41), recorded as the step's id and as the next input.
__global__ void __launch_bounds__(kWideArgThreads)
wide_argmax_kernel(const float* __restrict__ logits, int vocab, int n, WideState st, int* __restrict__ step_tokens) {
  __shared__ float sv[kWideArgThreads / 32];
  __shared__ int si[kWideArgThreads / 32];
  const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float4* src = reinterpret_cast<const float4*>(logits + (size_t)row * vocab);
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab / 4; i += kWideArgThreads) {     // ascending per thread: > keeps the first
    const float4 v = __ldcs(src + i);
    if (v.x > bv) { bv = v.x; bi = 4 * i; }
    if (v.y > bv) { bv = v.y; bi = 4 * i + 1; }
    if (v.z > bv) { bv = v.z; bi = 4 * i + 2; }
    if (v.w > bv) { bv = v.w; bi = 4 * i + 3; }
  }
  for (int i = (vocab / 4) * 4 + threadIdx.x; i < vocab; i += kWideArgThreads) {
    const float v = logits[(size_t)row * vocab + i];
    if (v > bv) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    bv = lane < kWideArgThreads / 32 ? sv[lane] : -INFINITY;
    bi = lane < kWideArgThreads / 32 ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      if (bi == 0x7fffffff) bi = 0;                 // a row of NaNs: id 0, as the host path casts
      const int p = st.pos[row];
      step_tokens[(size_t)(p - st.pos0[row]) * n + row] = bi;
      st.tok[row] = bi;
      st.pos[row] = p + 1;
    }
  }
}

// ------------------------------------------------------------------ attention of a wide step
// One CTA per (session, kv head, key split).  The session's K / V rows of this head are contiguous inside
// a page ([page][kv head][slot][hd]), so the CTA streams them in blocks of kWaChunk consecutive positions
// with one bulk async copy each for K and V into a ring of shared-memory stages, several blocks in flight;
// the eight warps take two keys of a block each (online softmax per warp, all G query heads of the group
// together) and the per-warp states are merged at the end.  Split 0 also norms, rotates and appends this
// step's own K / V row; the current position's row is taken from shared memory, not from the cache.
constexpr int kWaThreads = 256, kWaWarps = 8, kWaChunk = 2 * kWaWarps, kWaMaxStages = 6;

struct WideAttnArgs {
  const float* qkv;          // [sessions][nqkv] raw projections of this step
  const int* pos;            // [sessions] position of this step's token
  const int* page_table;     // first session's row; rows of pages_per_seq entries
  int pages_per_seq;
  int is_global;
  int nsplit;
  int stages;                // ring depth (2 .. kWaMaxStages), sized by the host to the shared memory
  const float *g_q, *g_k, *cosT, *sinT;
  LayerKv kv;
  float* part;               // nsplit > 1: [session][kv head][split][G][hd + 2] (o, then m and l)
  __nv_bfloat16* out;        // nsplit == 1: [session][hq * hd]
  int* err;
  int seq_stride;            // 1: session i has row i of the page table; 0: every query reads sequence 0
  int appended;              // 1: q rows are final (no norm, no rotation) and every K / V row is already in the cache
  float* out_f32;            // nsplit == 1: the same output in fp32 (operator-level callers), optional
  int ctas_per_sm;           // host-side hint: size the ring so that this many CTAs fit one SM (0 = 1)
  int qkv_parts;             // > 1: qkv is that many split-K partials, qkv_part_stride floats apart, summed on load
  size_t qkv_part_stride;
};

template <typename T, int HD>
__host__ __device__ constexpr int wa_stage_bytes() { return 2 * kWaChunk * HD * (int)sizeof(T); }
__host__ __device__ inline size_t wa_fixed_bytes(int hd, int G) {
  return sizeof(float) * ((size_t)(G + 2) * hd + (size_t)kWaWarps * G * (hd + 2)) + 16 * kWaMaxStages + 128;
}

template <typename T, int HD, int G>
__global__ void __launch_bounds__(kWaThreads, 2)
wide_attn_kernel(ModelDims dm, WideAttnArgs a) {
  constexpr int VEC = HD / 32, half = HD / 2;
  constexpr int kStage = wa_stage_bytes<T, HD>();
  extern __shared__ __align__(128) unsigned char wa_sm[];
  const int S = a.stages;
  unsigned char* ring = wa_sm;
  float* q_s = reinterpret_cast<float*>(wa_sm + (size_t)S * kStage);   // [G][HD]
  float* k_s = q_s + G * HD;                                           // [HD]
  float* v_s = k_s + HD;                                               // [HD]
  float* wm = v_s + HD;                                                // [warps][G]
  float* wl = wm + kWaWarps * G;
  float* wo = wl + kWaWarps * G;                                       // [warps][G][HD]
  uint64_t* full = reinterpret_cast<uint64_t*>(wo + kWaWarps * G * HD);
  uint64_t* empty = full + kWaMaxStages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x % a.nsplit;
  const int kvh = (blockIdx.x / a.nsplit) % dm.hkv;
  const int qi = blockIdx.x / (a.nsplit * dm.hkv);
  int pos = a.pos[qi];
  if (pos < 0 || pos >= dm.max_ctx) {
    if (threadIdx.x == 0) atomicExch(a.err, (int)kDevBadPosition);
    pos = 0;
  }
  const int* ptab = a.page_table + (size_t)(a.seq_stride ? qi : 0) * a.pages_per_seq;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], kWaWarps); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const T* kbase = reinterpret_cast<const T*>(a.kv.k);
  const T* vbase = reinterpret_cast<const T*>(a.kv.v);
  // ---- key range of this split; the current position is served from shared memory.  The first blocks are
  // requested before the prologue below (they depend on the position only), so their latency hides behind it.
  int k0, k1;
  attn_split_range(dm, pos, a.is_global, a.nsplit, split, &k0, &k1);
  const bool has_cur = !a.appended && k1 == pos + 1 && k1 > k0;
  const int k1s = has_cur ? pos : k1;                  // streamed keys: [k0, k1s)
  const int cb0 = k0 / kWaChunk;
  const int nchunks = k1s > k0 ? (k1s + kWaChunk - 1) / kWaChunk - cb0 : 0;
  auto issue = [&](int c) {                            // thread 0: block c of this split into its stage
    const int s = c % S, key = (cb0 + c) * kWaChunk;
    const size_t off = (((size_t)ptab[key / kPage] * dm.hkv + kvh) * kPage + (key % kPage)) * HD;
    unsigned char* dst = ring + (size_t)s * kStage;
    mbar_arrive_expect_tx(&full[s], (uint32_t)kStage);
    bulk_load_1d(dst, kbase + off, kStage / 2, &full[s]);
    bulk_load_1d(dst + kStage / 2, vbase + off, kStage / 2, &full[s]);
  };
  if (threadIdx.x == 0)
    for (int c = 0; c < nchunks && c < S - 1; ++c) issue(c);
  // ---- this step's q heads (normed, rotated, scaled), k head and v head
  const float* row = a.qkv + (size_t)qi * dm.nqkv();
  const float att_scale = rsqrtf((float)HD);
  const int nparts = a.qkv_parts > 1 ? a.qkv_parts : 1;
  const size_t pstride = a.qkv_part_stride;
  auto ld = [&](const float* p) {                      // one projection value: the sum of its split-K partials, in order
    float v = p[0];
    for (int q = 1; q < nparts; ++q) v += p[(size_t)q * pstride];
    return v;
  };
  for (int h = warp; h < (a.appended ? G : G + 2); h += kWaWarps) {
    if (a.appended) {                                  // final q rows: only the attention scale
      const float* src = row + (size_t)(kvh * G + h) * HD;
      for (int e = lane; e < HD; e += 32) q_s[h * HD + e] = ld(src + e) * att_scale;
    } else if (h <= G) {
      const float* src = h < G ? row + (size_t)(kvh * G + h) * HD : row + dm.nq() + (size_t)kvh * HD;
      const float* gain = h < G ? a.g_q : a.g_k;
      float* dst = h < G ? q_s + h * HD : k_s;
      float ss = 0.f;
      for (int e = lane; e < HD; e += 32) { const float v = ld(src + e); ss += v * v; }
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)HD + dm.eps);
      const float post = h < G ? att_scale : 1.0f;
      for (int e = lane; e < half; e += 32) {
        const float a0 = ld(src + e) * r * gain[e], b0 = ld(src + e + half) * r * gain[e + half];
        const float cs = a.cosT[(size_t)pos * half + e], sn = a.sinT[(size_t)pos * half + e];
        dst[e] = (a0 * cs - b0 * sn) * post;
        dst[e + half] = (b0 * cs + a0 * sn) * post;
      }
    } else {
      const float* src = row + dm.nq() + dm.nkv() + (size_t)kvh * HD;
      for (int e = lane; e < HD; e += 32) v_s[e] = ld(src + e);
    }
  }
  __syncthreads();
  if (split == 0 && !a.appended) {          // append: exactly one CTA per (session, kv head)
    const int page = ptab[pos / kPage], slot = pos % kPage;
    const size_t off = (((size_t)page * dm.hkv + kvh) * kPage + slot) * HD;
    T* kw = reinterpret_cast<T*>(a.kv.k);
    T* vw = reinterpret_cast<T*>(a.kv.v);
    for (int e = threadIdx.x; e < HD; e += kWaThreads) {
      if constexpr (sizeof(T) == 4) {
        kw[off + e] = k_s[e];
        vw[off + e] = v_s[e];
        if (a.kv.k16) a.kv.k16[off + e] = __float2bfloat16(k_s[e]);
      } else {
        kw[off + e] = __float2bfloat16(k_s[e]);
        vw[off + e] = __float2bfloat16(v_s[e]);
      }
      if (a.kv.v16) a.kv.v16[(((size_t)page * dm.hkv + kvh) * HD + e) * kPage + slot] = __float2bfloat16(v_s[e]);
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");     // later steps fetch these rows with bulk copies
  }
  float q[G][VEC], o[G][VEC], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      q[g][c] = q_s[g * HD + head_elem<HD>(lane, c)];
      o[g][c] = 0.f;
    }
  }
  bool ok = true;
  for (int c = 0; c < nchunks && ok; ++c) {
    const int s = c % S;
    if (threadIdx.x == 0 && c + S - 1 < nchunks) {     // refill the stage that block c - 1 used
      const int cn = c + S - 1;
      if (cn >= S) ok = mbar_wait(&empty[cn % S], (uint32_t)((cn / S - 1) & 1), a.err);
      if (ok) issue(cn);
    }
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;    // warp 0 follows its producer lane; the others see the error word
    if (!ok) break;
    ok = mbar_wait(&full[s], (uint32_t)((c / S) & 1), a.err);
    if (!ok) break;
    const T* ks = reinterpret_cast<const T*>(ring + (size_t)s * kStage);
    const T* vs = ks + kWaChunk * HD;
    const int ka = (cb0 + c) * kWaChunk + warp, kb = ka + kWaWarps;
    const bool hasa = ka >= k0 && ka < k1s, hasb = kb >= k0 && kb < k1s;
    float kA[VEC], kB[VEC], vA[VEC], vB[VEC];
    load_head_row_smem<T, HD>(ks + (size_t)warp * HD, lane, kA);
    load_head_row_smem<T, HD>(ks + (size_t)(warp + kWaWarps) * HD, lane, kB);
    load_head_row_smem<T, HD>(vs + (size_t)warp * HD, lane, vA);
    load_head_row_smem<T, HD>(vs + (size_t)(warp + kWaWarps) * HD, lane, vB);
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);             // rows are in registers
    if (hasa || hasb) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int cc = 0; cc < VEC; ++cc) { sa += q[g][cc] * kA[cc]; sb += q[g][cc] * kB[cc]; }
        sa = hasa ? warp_sum(sa) : -INFINITY;
        sb = hasb ? warp_sum(sb) : -INFINITY;
        const float mn = fmaxf(m[g], fmaxf(sa, sb));
        const float corr = __expf(m[g] - mn);
        const float pa = hasa ? __expf(sa - mn) : 0.f, pb = hasb ? __expf(sb - mn) : 0.f;
        l[g] = l[g] * corr + pa + pb;
        m[g] = mn;
#pragma unroll
        for (int cc = 0; cc < VEC; ++cc) o[g][cc] = o[g][cc] * corr + (hasa ? pa * vA[cc] : 0.f) + (hasb ? pb * vB[cc] : 0.f);
      }
    }
  }
  if (has_cur && warp == 0) {                          // this step's own key
    float kA[VEC], vA[VEC];
#pragma unroll
    for (int cc = 0; cc < VEC; ++cc) {
      kA[cc] = k_s[head_elem<HD>(lane, cc)];
      vA[cc] = v_s[head_elem<HD>(lane, cc)];
      if constexpr (sizeof(T) == 2) {                  // what a bf16 cache hands back
        kA[cc] = __bfloat162float(__float2bfloat16(kA[cc]));
        vA[cc] = __bfloat162float(__float2bfloat16(vA[cc]));
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sa = 0.f;
#pragma unroll
      for (int cc = 0; cc < VEC; ++cc) sa += q[g][cc] * kA[cc];
      sa = warp_sum(sa);
      const float mn = fmaxf(m[g], sa);
      const float corr = __expf(m[g] - mn), pa = __expf(sa - mn);
      l[g] = l[g] * corr + pa;
      m[g] = mn;
#pragma unroll
      for (int cc = 0; cc < VEC; ++cc) o[g][cc] = o[g][cc] * corr + pa * vA[cc];
    }
  }
  // ---- merge the warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { wm[warp * G + g] = m[g]; wl[warp * G + g] = l[g]; }
#pragma unroll
    for (int cc = 0; cc < VEC; ++cc) wo[((size_t)warp * G + g) * HD + head_elem<HD>(lane, cc)] = o[g][cc];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += kWaThreads) {
    const int g = i / HD, e = i - g * HD;
    float M = -INFINITY;
    for (int w = 0; w < kWaWarps; ++w) M = fmaxf(M, wm[w * G + g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
      for (int w = 0; w < kWaWarps; ++w) {
        const float f = __expf(wm[w * G + g] - M);
        L += wl[w * G + g] * f;
        O += wo[((size_t)w * G + g) * HD + e] * f;
      }
    }
    if (a.nsplit > 1) {
      float* dst = a.part + ((((size_t)qi * dm.hkv + kvh) * a.nsplit + split) * G + g) * (HD + 2);
      dst[e] = O;
      if (e == 0) { dst[HD] = M; dst[HD + 1] = L; }
    } else {
      const float val = L > 0.f ? O / L : 0.f;
      const size_t oi = ((size_t)qi * dm.hq + kvh * G + g) * HD + e;
      if (a.out) a.out[oi] = __float2bfloat16(val);
      if (a.out_f32) a.out_f32[oi] = val;
    }
  }
  if (*reinterpret_cast<volatile int*>(a.err) == (int)kDevBarrierTimeout) {
    // a wait gave up: let the bulk copies still in flight land before the CTA retires
    for (int i = 0; i < 2000; ++i) __nanosleep(100);
    __syncthreads();
  }
}

// Sum of the key splits' partial states: one CTA per (session, query head).  The splits' (m, l) pairs are fetched
// by one thread each and their weights exp(m_s - M) / L shared, so the element loop is independent loads only.
__global__ void __launch_bounds__(128)
wide_attn_combine_kernel(const float* __restrict__ part, int nsplit, int hq, int hkv, int hd, __nv_bfloat16* __restrict__ out,
                         float* __restrict__ out_f32) {
  __shared__ float w_s[kMaxSplits];
  const int G = hq / hkv;
  const int qi = blockIdx.x / hq, h = blockIdx.x % hq, kvh = h / G, g = h % G;
  const float* base = part + (((size_t)qi * hkv + kvh) * nsplit * G + g) * (hd + 2);
  const size_t stride = (size_t)G * (hd + 2);
  if (threadIdx.x < 32) {
    float M = -INFINITY, L = 0.f;
    float ms[(kMaxSplits + 31) / 32], ls[(kMaxSplits + 31) / 32];
#pragma unroll
    for (int r = 0; r < (kMaxSplits + 31) / 32; ++r) {
      const int sp = threadIdx.x + 32 * r;
      ms[r] = sp < nsplit ? base[sp * stride + hd] : -INFINITY;
      ls[r] = sp < nsplit ? base[sp * stride + hd + 1] : 0.f;
      M = fmaxf(M, ms[r]);
    }
    M = warp_max(M);
#pragma unroll
    for (int r = 0; r < (kMaxSplits + 31) / 32; ++r) {
      ms[r] = M > -INFINITY ? __expf(ms[r] - M) : 0.f;
      L += ls[r] * ms[r];
    }
    L = warp_sum(L);
    const float inv = L > 0.f ? 1.0f / L : 0.f;
#pragma unroll
    for (int r = 0; r < (kMaxSplits + 31) / 32; ++r) {
      const int sp = threadIdx.x + 32 * r;
      if (sp < nsplit) w_s[sp] = ms[r] * inv;
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < hd; e += 128) {
    float O = 0.f;
    for (int s = 0; s < nsplit; ++s) O += base[s * stride + e] * w_s[s];
    if (out) out[((size_t)qi * hq + h) * hd + e] = __float2bfloat16(O);
    if (out_f32) out_f32[((size_t)qi * hq + h) * hd + e] = O;
  }
}

// Host side: the kernel instantiated for the cache type, head size and group size.  nb <= 0 only sets the
// kernel's shared-memory attribute (executor creation, outside any stream capture).
template <typename T, int HD, int G>
inline void launch_wide_attn_t(cudaStream_t st, const ModelDims& d, int nb, size_t smem_optin, WideAttnArgs a) {
  const size_t fixed = wa_fixed_bytes(HD, G);
  const int stage = wa_stage_bytes<T, HD>();
  // The loop is a chain of dependent shuffles and exponentials on eight warps, so one CTA alone leaves the SM
  // mostly idle (about 2 us per block of 16 keys, whatever its bytes): with two CTAs per SM the ring is shallower
  // but twice as many chains run.
  int per_sm = std::max(1, a.ctas_per_sm);
  int stages = 0;
  for (; per_sm >= 1; --per_sm) {
    const size_t budget = smem_optin / per_sm - 1024;
    stages = budget > fixed ? (int)std::min<size_t>(kWaMaxStages, (budget - fixed) / stage) : 0;
    if (stages >= 2) break;
  }
  B2_CHECK(stages >= 2, kUnimplemented, "the streaming decode attention does not fit the device's shared memory");
  a.stages = stages;
  const size_t smem = fixed + (size_t)stages * stage;
  raise_dyn_smem(wide_attn_kernel<T, HD, G>, smem);
  if (nb <= 0) return;
  wide_attn_kernel<T, HD, G><<<nb * d.hkv * a.nsplit, kWaThreads, smem, st>>>(d, a);
}
template <typename T, int HD>
inline void launch_wide_attn_g(cudaStream_t st, const ModelDims& d, int nb, size_t smem_optin, const WideAttnArgs& a) {
  switch (d.group()) {
    case 1: launch_wide_attn_t<T, HD, 1>(st, d, nb, smem_optin, a); break;
    case 2: launch_wide_attn_t<T, HD, 2>(st, d, nb, smem_optin, a); break;
    case 4: launch_wide_attn_t<T, HD, 4>(st, d, nb, smem_optin, a); break;
    default: throw Error{kUnimplemented, "query heads per kv head must be 1, 2 or 4"};
  }
}
template <typename T>
inline void launch_wide_attn_h(cudaStream_t st, const ModelDims& d, int nb, size_t smem_optin, const WideAttnArgs& a) {
  switch (d.hd) {
    case 32: launch_wide_attn_g<T, 32>(st, d, nb, smem_optin, a); break;
    case 64: launch_wide_attn_g<T, 64>(st, d, nb, smem_optin, a); break;
    case 128: launch_wide_attn_g<T, 128>(st, d, nb, smem_optin, a); break;
    case 256: launch_wide_attn_g<T, 256>(st, d, nb, smem_optin, a); break;
    default: throw Error{kUnimplemented, "head size must be 32, 64, 128 or 256"};
  }
}
inline void launch_wide_attn(cudaStream_t st, const ModelDims& d, int nb, size_t smem_optin, const WideAttnArgs& a) {
  if (d.kv_dtype == 0) launch_wide_attn_h<float>(st, d, nb, smem_optin, a);
  else launch_wide_attn_h<__nv_bfloat16>(st, d, nb, smem_optin, a);
}

// out[t][:] = sum of the split-K partials parts[p][t][:], rows of `cols` floats.
__global__ void __launch_bounds__(256)
wide_sum_parts_kernel(const float* __restrict__ parts, int nparts, size_t part_stride, size_t count, float* __restrict__ out) {
  const size_t i = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (i * 4 >= count) return;
  float4 a = reinterpret_cast<const float4*>(parts)[i];
  for (int p = 1; p < nparts; ++p) {
    const float4 b = reinterpret_cast<const float4*>(parts + (size_t)p * part_stride)[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  reinterpret_cast<float4*>(out)[i] = a;
}

}  // namespace b200lm

// Decode-step device code (one new token per session).
//
// A decode step is five dependent phases per layer plus the LM head:
//   A  residual update + pre-attention RMSNorm  -> int4 QKV GEMV
//   B  QK-RMSNorm + RoPE + KV append            -> split-KV attention partials
//   C  log-sum-exp combine (per head slice)     -> int4 O GEMV (K split by head)
//   D  post-attn norm + residual + pre-FFN norm -> int4 gate/up GEMV + GeGLU
//   E  activation slice                         -> int4 down GEMV (K split)
//   H  final residual + final norm              -> int4 LM-head GEMV + arg-max
// Every phase is a __device__ function of (cta, n_cta), so the same code runs
// either as one kernel per phase or inside one persistent cooperative kernel
// with a grid barrier between phases.
//
// int4 GEMV: weights are stored pre-tiled for mma.sync.m16n8k32 (s8 x s8 ->
// s32).  Activations are quantised per column to up to three int8 terms
// (x ~ s*(t0 + t1/128 + t2/16384)), one MMA column per term, so accumulation is
// exact integer arithmetic (order-independent, hence deterministic) and the
// result carries ~fp32 accuracy.  Nibbles are two's complement; masking a
// nibble into the high half of a byte yields the int8 value 16*q, so the
// unpack is two logic ops per eight weights and the factor 16 leaves in the
// epilogue.
#pragma once
#include "common.cuh"

namespace b200lm {

constexpr int kDecThreads = 512;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kMaxRoundUnits = 16;   // row tiles reduced per round in shared memory
constexpr int kMaxCols = 4;          // sessions per decode launch
constexpr int kQCols = 8;            // quantised columns (= one MMA n-tile)
constexpr int kLoadDepth = 4;        // 16-byte weight loads in flight per lane
constexpr int kMaxSplits = 64;

struct LayerWeights {
  const uint4 *wqkv, *wo, *wgu, *wdown;      // mma-tiled int4 (see repack_w4t)
  const float *sqkv, *so, *sgu, *sdown;      // per-output-row scales (sgu in tile order)
  const float *g_pre_attn, *g_post_attn, *g_pre_ffn, *g_post_ffn, *g_q, *g_k;
  int is_global;
  float gmax_pre_attn, gmax_pre_ffn;   // max |gain| of the two pre-norm gain vectors
  float attn_bound;                    // |q.k| / sqrt(hd) <= attn_bound after QK-RMSNorm: sqrt(hd) max|g_q| max|g_k|
};

// Copies of a layer's decode weights in the layouts the chained kernel streams with ONE bulk copy per
// ring slot (the barrier-per-phase kernels use the plain tile order of LayerWeights).
struct ChainedLayer {
  const unsigned char* wqkv_s;   // per 16-row tile: its KT 512-byte tiles, then its 16 scales (64 bytes)
  const unsigned char* wgu_s;    // same for the gate / up tiles (alternating)
  const uint4* wdown_k;          // tiles ordered [k_tile][row_tile]: a 64-feature K slice is contiguous
  const uint4* wo_s;             // tiles ordered [head slice][row_tile][k_tile of the slice]
  const float* gA;               // [g_pre_attn | g_post_ffn of the previous layer]
  const float* gD;               // [g_pre_ffn | g_post_attn]
  const float* qk;               // [g_q | g_k]
};

struct LayerKv {
  void* k;               // [pages][hkv][kPage][hd], fp32 or bf16
  void* v;
  // operands of the tensor-core prefill attention, or null when it is not used:
  __nv_bfloat16* k16;    // bf16 copy of K rows, same layout (null when the cache itself is bf16)
  __nv_bfloat16* v16;    // bf16 V TRANSPOSED per page: [page][kv_head][hd][kPage]
};

struct DecodeState {          // lives in device memory, one per executor
  int token[kMaxCols];        // input token of the next step
  int pos[kMaxCols];          // its position
  int out_token[kMaxCols];    // arg-max of the last step
  int err;                    // DeviceError
  unsigned int barrier;       // grid barrier counter (persistent kernel)
  int steps_done;
  int gave_up[8];             // first bounded wait that gave up (chained kernel): phase code, layer, CTA, kind of wait,
                              // then for a poll: tag seen, tag wanted, word offset in the exchange area, thread
};

struct DecodeArgs {
  ModelDims dims;
  int ncols, nterms;
  int n_attn_splits_local, n_attn_splits_global;
  int o_slices, down_slices;          // K-splits of the O and down GEMVs
  const LayerWeights* layers;         // device array [n_layers]
  const LayerKv* kv;                  // device array [n_layers]
  const int* page_table;              // [ncols][pages_per_seq]
  int pages_per_seq;
  const uint8_t* embed_rows;          // canonical [vocab][d/2] for the row gather
  const float* embed_scale;           // [vocab]
  const uint4* head_w;                // mma-tiled tied embedding
  const float* g_final;
  float gmax_final;
  const float *rope_cos[2], *rope_sin[2];   // [max_ctx][hd/2]; 0 local, 1 global
  DecodeState* st;
  // activations (all fp32, device)
  float* xres[2];       // [ncols][d] residual stream, ping-pong
  float* qkv;           // [ncols][nqkv]
  float* part_o;        // [ncols][hkv][splits][G][hd]
  float* part_ml;       // [ncols][hkv][splits][G][2]
  float* opart;         // [o_slices][ncols][d]
  float* act;           // [ncols][ffn]
  float* fpart;         // [down_slices][ncols][d]
  float* logits;        // [ncols][vocab]
  float* amax_val;      // [n_cta][ncols]
  int* amax_idx;        // [n_cta][ncols]
  int* step_tokens;     // [capacity][ncols] arg-max of every step since steps_done was reset
  int step_capacity;
  int advance;          // 1: feed arg-max back as next token and bump pos (device loop)
  // chained kernel only
  const ChainedLayer* chained;        // device array [n_layers]
  const unsigned char* head_ws;       // tied embedding as row-tile records (tiles + scales)
  const float* gH;                    // [g_final | g_post_ffn of the last layer]
  const float* rope_cs[2];            // [max_ctx][cos(hd/2) | sin(hd/2)]; 0 local, 1 global
  int* progress;                      // [n_cta] phase code * 1000 + layer each CTA has reached (diagnostics)
  long long* trace;     // optional [n_barriers][n_cta][2] SM-clock stamps (arrive, release), or null
  long long* trace_pts; // optional [n_barriers][n_cta][8] stamps inside the phase that ends at that barrier
};

// Barrier of the 512 compute threads of a decode CTA (named barrier 1), so a
// kernel may carry extra warps (a copy producer) that do not take part.
__device__ __forceinline__ void dec_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }

// ----------------------------------------------------------------- reductions

// The per-warp partials meet in shared memory; every warp then folds the 16 of
// them with shuffles (one load per lane instead of 16 per thread).
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  dec_sync();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  dec_sync();
  float t = scratch[threadIdx.x & (kDecWarps - 1)];
#pragma unroll
  for (int o = kDecWarps / 2; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  v = warp_max(v);
  dec_sync();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  dec_sync();
  float t = scratch[threadIdx.x & (kDecWarps - 1)];
#pragma unroll
  for (int o = kDecWarps / 2; o > 0; o >>= 1) t = fmaxf(t, __shfl_xor_sync(0xffffffffu, t, o));
  return t;
}

// ----------------------------------------------------------------- int4 tiles

// One 16x64 weight tile is 512 bytes: lane l owns bytes [16l, 16l+16) = words
// w0..w3.  With g = l/4, t = l%4, word j covers k = 32*(j/2) + 16*(j%2) + 4t + i
// (i = 0..3): nibble 2i is row g, nibble 2i+1 is row g+8, two's complement.
__device__ __forceinline__ void mma_s8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Integer value of element (row r of 16, k of 64) of a tile; used by the
// bit-exact unpack check and by the embedding gather test.
__device__ __forceinline__ int w4t_element(const uint4* tile, int r, int k) {
  int g = r & 7, hi = r >> 3;
  int m = k >> 5, half = (k >> 4) & 1, t = (k >> 2) & 3, i = k & 3;
  const uint32_t* words = reinterpret_cast<const uint32_t*>(tile + (g * 4 + t));
  uint32_t w = words[m * 2 + half];
  int v = (int)((w >> (8 * i + 4 * hi)) & 0xF);
  return v >= 8 ? v - 16 : v;
}

// Two 16x32 MMAs on one lane's 16 bytes of a tile (words x,y then z,w).
__device__ __forceinline__ void mma_tile_words(int (&acc)[4], const uint4& w, uint32_t b0, uint32_t b1,
                                               uint32_t b2, uint32_t b3) {
  const uint32_t m = 0xF0F0F0F0u;   // high nibble of every byte = 16 * q as int8
  mma_s8s8(acc, (w.x << 4) & m, w.x & m, (w.y << 4) & m, w.y & m, b0, b1);
  mma_s8s8(acc, (w.z << 4) & m, w.z & m, (w.w << 4) & m, w.w & m, b2, b3);
}

struct QuantCols {
  const int8_t* q;   // [nq][stride]
  int stride;
  int nq;
};

__device__ __forceinline__ void flush_tile(int* red, int unit, const int (&c)[4], int lane, int nq) {
  int g = lane >> 2, t = lane & 3;
  int* base = red + unit * 16 * kQCols;
  if (2 * t < nq) {
    atomicAdd(base + g * kQCols + 2 * t, c[0]);
    atomicAdd(base + (g + 8) * kQCols + 2 * t, c[2]);
  }
  if (2 * t + 1 < nq) {
    atomicAdd(base + g * kQCols + 2 * t + 1, c[1]);
    atomicAdd(base + (g + 8) * kQCols + 2 * t + 1, c[3]);
  }
}

// Accumulates nu row tiles (u0..u0+nu-1) over k-tiles [kt0, kt0+ktn) into
// red[nu][16][kQCols].  The nu*ktn tile blocks are dealt to the warps as
// contiguous runs, so every warp streams consecutive memory.
__device__ __forceinline__ void gemv_tiles(const uint4* __restrict__ w, int KT, int kt0, int ktn,
                                           int u0, int nu, QuantCols xc, int* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int total = nu * ktn;
  const int per = (total + kDecWarps - 1) / kDecWarps;
  const int beg = warp * per;
  const int end = min(total, beg + per);
  const bool colok = g < xc.nq;
  const int8_t* xrow = xc.q + (size_t)g * xc.stride + 4 * t;
  int acc[4] = {0, 0, 0, 0};
  int cur = -1;
  for (int b = beg; b < end; b += kLoadDepth) {
    uint4 wv[kLoadDepth];
#pragma unroll
    for (int u = 0; u < kLoadDepth; ++u) {
      int bb = b + u;
      if (bb < end) {
        int un = bb / ktn, kt = bb - un * ktn;
        wv[u] = ldg_nc_v4(w + ((size_t)(u0 + un) * KT + kt0 + kt) * 32 + lane);
      } else {
        wv[u] = make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int u = 0; u < kLoadDepth; ++u) {
      int bb = b + u;
      if (bb < end) {
        int un = bb / ktn, kt = bb - un * ktn;
        if (un != cur) {
          if (cur >= 0) flush_tile(red, cur, acc, lane, xc.nq);
          cur = un;
          acc[0] = acc[1] = acc[2] = acc[3] = 0;
        }
        uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        if (colok) {
          const int8_t* xp = xrow + kt * 64;
          b0 = *reinterpret_cast<const uint32_t*>(xp);
          b1 = *reinterpret_cast<const uint32_t*>(xp + 16);
          b2 = *reinterpret_cast<const uint32_t*>(xp + 32);
          b3 = *reinterpret_cast<const uint32_t*>(xp + 48);
        }
        mma_tile_words(acc, wv[u], b0, b1, b2, b3);
      }
    }
  }
  if (cur >= 0) flush_tile(red, cur, acc, lane, xc.nq);
}

// Shared-memory carve-up of the decode kernels.
struct DecodeSmem {
  float* xf;        // [ncols][kmax] staging vector(s)
  int8_t* xq;       // [kQCols][xstride]
  int xstride;
  int* red;         // [kMaxRoundUnits][16][kQCols]
  float* scratch;   // [64]
  float* colscale;  // [kMaxCols]
  int* colsum;      // [kQCols]
  float* attn;      // attention work area
  float* argbuf;    // [2 * kDecThreads] arg-max reduction
};

__host__ __device__ inline int dec_xstride(int kmax) { return ((kmax + 127) / 128) * 128 + 16; }
__host__ __device__ inline size_t dec_attn_floats(const ModelDims& d) {
  int G = d.hq / d.hkv;
  return (size_t)(G + 2) * d.hd + (size_t)kDecWarps * G * (d.hd + 2);
}
// rows of the quantised staging: three int8 terms per session, at most one MMA n-tile
__host__ __device__ inline int dec_xq_rows(int ncols) { return ncols * 3 < kQCols ? ncols * 3 : kQCols; }
__host__ __device__ inline size_t dec_smem_bytes(const ModelDims& d, int ncols) {
  int kmax = d.ffn > d.d ? d.ffn : d.d;
  if (d.hq * d.hd > kmax) kmax = d.hq * d.hd;
  size_t b = (size_t)ncols * kmax * 4;
  b += (size_t)dec_xq_rows(ncols) * dec_xstride(kmax);
  b += (size_t)kMaxRoundUnits * 16 * kQCols * 4;
  b += 64 * 4 + kMaxCols * 4 + kQCols * 4 + 2 * kDecThreads * 4;
  b += dec_attn_floats(d) * 4;
  return b + 256 + 16;
}
__device__ inline DecodeSmem carve_smem(unsigned char* base, const ModelDims& d, int ncols) {
  int kmax = d.ffn > d.d ? d.ffn : d.d;
  if (d.hq * d.hd > kmax) kmax = d.hq * d.hd;
  DecodeSmem s;
  size_t off = 0;
  s.xf = reinterpret_cast<float*>(base + off);
  off += (size_t)ncols * kmax * 4;
  s.xstride = dec_xstride(kmax);
  s.xq = reinterpret_cast<int8_t*>(base + off);
  off += (size_t)dec_xq_rows(ncols) * s.xstride;
  off = (off + 15) & ~size_t(15);
  s.red = reinterpret_cast<int*>(base + off);
  off += (size_t)kMaxRoundUnits * 16 * kQCols * 4;
  s.scratch = reinterpret_cast<float*>(base + off);
  off += 64 * 4;
  s.colscale = reinterpret_cast<float*>(base + off);
  off += kMaxCols * 4;
  s.colsum = reinterpret_cast<int*>(base + off);
  off += kQCols * 4;
  s.argbuf = reinterpret_cast<float*>(base + off);
  off += 2 * kDecThreads * 4;
  off = (off + 15) & ~size_t(15);
  s.attn = reinterpret_cast<float*>(base + off);
  return s;
}

// Quantises one value with scale inv into up to three int8 terms.
__device__ __forceinline__ void quantize_value(float r, int nterms, int8_t* q0, int stride) {
  float t0 = fminf(fmaxf(rintf(r), -127.f), 127.f);
  q0[0] = (int8_t)(int)t0;
  if (nterms > 1) {
    float r1 = (r - t0) * 128.0f;
    float t1 = fminf(fmaxf(rintf(r1), -127.f), 127.f);
    q0[stride] = (int8_t)(int)t1;
    if (nterms > 2) {
      float r2 = (r1 - t1) * 128.0f;
      q0[2 * stride] = (int8_t)(int)fminf(fmaxf(rintf(r2), -127.f), 127.f);
    }
  }
}

// Quantises xf[ncols][K] (shared) into xq with nterms int8 terms per column.
__device__ __noinline__ void quantize_cols(const DecodeSmem& s, int K, int ncols, int nterms) {
  for (int col = 0; col < ncols; ++col) {
    const float* x = s.xf + (size_t)col * K;
    float m = 0.f;
    for (int i = threadIdx.x; i < K; i += kDecThreads) m = fmaxf(m, fabsf(x[i]));
    m = block_max(m, s.scratch);
    float inv = m > 0.f ? 127.0f / m : 0.f;
    int8_t* q0 = s.xq + (size_t)(col * nterms) * s.xstride;
    for (int i = threadIdx.x; i < K; i += kDecThreads) quantize_value(x[i] * inv, nterms, q0 + i, s.xstride);
    if (threadIdx.x == 0) s.colscale[col] = m > 0.f ? m / 127.0f : 0.f;
  }
  dec_sync();
}

// Value of output (unit, row, col) after a round: sum over terms, bias removed.
__device__ __forceinline__ float finalize_value(const DecodeSmem& s, int unit, int row, int col,
                                                int nterms) {
  const int* r = s.red + (unit * 16 + row) * kQCols + col * nterms;
  float v = (float)r[0];
  if (nterms > 1) v += (float)r[1] * (1.0f / 128.0f);
  if (nterms > 2) v += (float)r[2] * (1.0f / 16384.0f);
  return v * (s.colscale[col] * (1.0f / 16.0f));      // weights entered the MMA as 16 * q
}

enum GemvEpilogue { kEpiPlain = 0, kEpiGeglu = 1, kEpiHead = 2 };

struct GemvJob {
  const uint4* w;
  const float* wscale;
  int N, K;          // full matrix: N rows (multiple of 16), K columns (multiple of 64)
  int slices;        // K split across CTAs; partial outputs when > 1
  float* y;          // plain: [slices][ncols][N]; geglu: [ncols][N/2]; head: [ncols][N]
  int epilogue;
};

// Which (slice, tile range) this CTA owns.  Returns false when it has no work.
__device__ __forceinline__ bool gemv_assignment(const GemvJob& j, int cta, int ncta, int* slice,
                                                int* t0, int* t1) {
  int ntiles = j.N / 16;
  int cps = ncta / j.slices;
  if (cps < 1) cps = 1;
  int sl = cta / cps;
  if (sl >= j.slices) return false;
  int local = cta - sl * cps;
  int per = (ntiles + cps - 1) / cps;
  if (j.epilogue == kEpiGeglu) per = (per + 1) & ~1;   // keep gate/up tile pairs together
  int a = local * per, b = min(ntiles, a + per);
  if (a >= b) return false;
  *slice = sl;
  *t0 = a;
  *t1 = b;
  return true;
}

// Runs the GEMV for this CTA's tiles; xq/colscale/colsum must already describe
// the activation slice.  best_val/best_idx carry the running arg-max (head).
__device__ inline void gemv_run(const GemvJob& j, const DecodeSmem& s, int ncols, int nterms,
                                int slice, int t0, int t1, float* best_val, int* best_idx) {
  const int KT = j.K / 64;
  const int ktn = KT / j.slices;
  const int kt0 = slice * ktn;
  QuantCols xc{s.xq, s.xstride, ncols * nterms};
  for (int r0 = t0; r0 < t1; r0 += kMaxRoundUnits) {
    int nu = min(kMaxRoundUnits, t1 - r0);
    for (int i = threadIdx.x; i < nu * 16 * kQCols; i += kDecThreads) s.red[i] = 0;
    dec_sync();
    gemv_tiles(j.w, KT, kt0, ktn, r0, nu, xc, s.red);
    dec_sync();
    if (j.epilogue == kEpiGeglu) {
      int npair = nu / 2;
      for (int i = threadIdx.x; i < npair * 16 * ncols; i += kDecThreads) {
        int col = i / (npair * 16), rem = i - col * npair * 16;
        int p = rem / 16, row = rem & 15;
        int ng = (r0 + 2 * p) * 16 + row, nu_ = ng + 16;
        float gate = finalize_value(s, 2 * p, row, col, nterms) * j.wscale[ng];
        float up = finalize_value(s, 2 * p + 1, row, col, nterms) * j.wscale[nu_];
        j.y[(size_t)col * (j.N / 2) + (size_t)((r0 / 2) + p) * 16 + row] = gelu_tanh(gate) * up;
      }
    } else {
      for (int i = threadIdx.x; i < nu * 16 * ncols; i += kDecThreads) {
        int col = i / (nu * 16), rem = i - col * nu * 16;
        int un = rem / 16, row = rem & 15;
        int n = (r0 + un) * 16 + row;
        float v = finalize_value(s, un, row, col, nterms) * j.wscale[n];
        j.y[((size_t)slice * ncols + col) * j.N + n] = v;
        if (j.epilogue == kEpiHead && col < kMaxCols) {
          if (v > best_val[col] || (v == best_val[col] && n < best_idx[col])) {
            best_val[col] = v;
            best_idx[col] = n;
          }
        }
      }
    }
    dec_sync();
  }
}

// ------------------------------------------------------------- phase prologues

// x = xin + rmsnorm(sum of parts) * g_post ; xout <- x (cta 0) ; xf <- rmsnorm(x) * g_pre
__device__ inline void prologue_resid_norm(const DecodeArgs& a, const DecodeSmem& s, int cta,
                                           const float* parts, int nparts, const float* xin,
                                           float* xout, const float* g_post, const float* g_pre) {
  const int d = a.dims.d;
  for (int col = 0; col < a.ncols; ++col) {
    float* x = s.xf + (size_t)col * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += kDecThreads) {
      float f = 0.f;
      for (int p = 0; p < nparts; ++p) f += __ldcg(parts + ((size_t)p * a.ncols + col) * d + i);
      x[i] = f;
      ss += f * f;
    }
    ss = block_sum(ss, s.scratch);
    float r = rsqrtf(ss / (float)d + a.dims.eps);
    float ss2 = 0.f;
    for (int i = threadIdx.x; i < d; i += kDecThreads) {
      float v = __ldcg(xin + (size_t)col * d + i) + x[i] * r * g_post[i];
      x[i] = v;
      ss2 += v * v;
      if (cta == 0) xout[(size_t)col * d + i] = v;
    }
    ss2 = block_sum(ss2, s.scratch);
    float r2 = rsqrtf(ss2 / (float)d + a.dims.eps);
    for (int i = threadIdx.x; i < d; i += kDecThreads) x[i] = x[i] * r2 * g_pre[i];
  }
  dec_sync();
}

// x = dequant(E[token]) * sqrt(d) ; xout <- x (cta 0) ; xf <- rmsnorm(x) * g_pre
__device__ inline void prologue_embed_norm(const DecodeArgs& a, const DecodeSmem& s, int cta,
                                           float* xout, const float* g_pre) {
  const int d = a.dims.d;
  const float emb = sqrtf((float)d);
  for (int col = 0; col < a.ncols; ++col) {
    int tok = __ldcg(&a.st->token[col]);
    if (tok < 0 || tok >= a.dims.vocab) {
      if (threadIdx.x == 0) atomicExch(&a.st->err, (int)kDevBadToken);
      tok = 0;
    }
    const uint8_t* row = a.embed_rows + (size_t)tok * (d / 2);
    float sc = a.embed_scale[tok] * emb;
    float* x = s.xf + (size_t)col * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += kDecThreads) {
      int b = row[i >> 1];
      int nib = (i & 1) ? (b >> 4) : (b & 0xF);
      int q = nib >= 8 ? nib - 16 : nib;
      float v = (float)q * sc;
      x[i] = v;
      ss += v * v;
      if (cta == 0) xout[(size_t)col * d + i] = v;
    }
    ss = block_sum(ss, s.scratch);
    float r = rsqrtf(ss / (float)d + a.dims.eps);
    for (int i = threadIdx.x; i < d; i += kDecThreads) x[i] = x[i] * r * g_pre[i];
  }
  dec_sync();
}

// ------------------------------------------------------------------ attention

template <typename T>
__device__ __forceinline__ float kv_to_float(T v);
template <>
__device__ __forceinline__ float kv_to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float kv_to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Lane l of a warp holds VEC = HD/32 elements of a head row: for HD >= 128 the
// elements 128*i + 4*l + c (16-byte loads), below that l*VEC + c.
template <typename T, int HD>
__device__ __forceinline__ void load_head_row(const T* __restrict__ p, int lane, float (&out)[HD / 32]) {
  constexpr int VEC = HD / 32;
  if constexpr (HD >= 128) {
#pragma unroll
    for (int i = 0; i < HD / 128; ++i) {
      if constexpr (sizeof(T) == 4) {
        float4 v = __ldcg(reinterpret_cast<const float4*>(p + i * 128 + lane * 4));
        out[i * 4 + 0] = v.x; out[i * 4 + 1] = v.y; out[i * 4 + 2] = v.z; out[i * 4 + 3] = v.w;
      } else {
        uint2 v = __ldcg(reinterpret_cast<const uint2*>(p + i * 128 + lane * 4));
        __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x);
        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
        out[i * 4 + 0] = __low2float(a); out[i * 4 + 1] = __high2float(a);
        out[i * 4 + 2] = __low2float(b); out[i * 4 + 3] = __high2float(b);
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < VEC; ++c) {
      if constexpr (sizeof(T) == 4) {
        out[c] = __ldcg(reinterpret_cast<const float*>(p) + lane * VEC + c);
      } else {
        unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(p) + lane * VEC + c);
        out[c] = __bfloat162float(__ushort_as_bfloat16(raw));
      }
    }
  }
}
// Same element mapping, source in shared memory (rows staged there by bulk copies).
template <typename T, int HD>
__device__ __forceinline__ void load_head_row_smem(const T* p, int lane, float (&out)[HD / 32]) {
  constexpr int VEC = HD / 32;
  if constexpr (HD >= 128) {
#pragma unroll
    for (int i = 0; i < HD / 128; ++i) {
      if constexpr (sizeof(T) == 4) {
        float4 v = *reinterpret_cast<const float4*>(p + i * 128 + lane * 4);
        out[i * 4 + 0] = v.x; out[i * 4 + 1] = v.y; out[i * 4 + 2] = v.z; out[i * 4 + 3] = v.w;
      } else {
        uint2 v = *reinterpret_cast<const uint2*>(p + i * 128 + lane * 4);
        __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&v.x);
        __nv_bfloat162 b = *reinterpret_cast<__nv_bfloat162*>(&v.y);
        out[i * 4 + 0] = __low2float(a); out[i * 4 + 1] = __high2float(a);
        out[i * 4 + 2] = __low2float(b); out[i * 4 + 3] = __high2float(b);
      }
    }
  } else {
#pragma unroll
    for (int c = 0; c < VEC; ++c) out[c] = kv_to_float<T>(p[lane * VEC + c]);
  }
}
template <int HD>
__device__ __forceinline__ int head_elem(int lane, int c) {
  if constexpr (HD >= 128) return (c >> 2) * 128 + lane * 4 + (c & 3);
  else return lane * (HD / 32) + c;
}

struct AttnJob {
  const float* qkv;          // [nq_tokens][nqkv] raw projections (fp32)
  const int* pos;            // [nq_tokens] position of each query (device) ...
  int pos0;                  // ... or pos0 + index when pos == nullptr
  const int* page_table;     // [seqs][pages_per_seq]
  int pages_per_seq;
  int seq_stride;            // 1: query i belongs to sequence i (decode); 0: all to sequence 0
  int is_global;
  int nsplit;
  int appended;              // 1: K/V rows (normed, roped) are already in the cache
  const float *g_q, *g_k;
  const float *cosT, *sinT;
  LayerKv kv;
  float *part_o, *part_ml;   // split partials (m, l, unnormalised o); null = write normalised output
  float* out_f32;            // [nq_tokens][hq][hd] normalised output (needs nsplit == 1), optional
  __nv_bfloat16* out_bf16;   // same in bf16, optional
  int* err;
  // optional staging (streaming decode kernel): rows of keys k0 .. k0+npre-1 of this
  // split already sit in shared memory, as does the RoPE row of the query position
  const void* k_pre;
  const void* v_pre;
  int npre;
  int rope_is_row;           // cosT / sinT point at the row of `pos`, not at the table
  int max_warps;             // > 0: only this many warps walk keys (smaller merge area)
};

// Key range [k0, k1) of one split.
__device__ __forceinline__ void attn_split_range(const ModelDims& dm, int pos, int is_global, int nsplit,
                                                 int split, int* k0, int* k1) {
  int nkeys = is_global ? pos + 1 : min(pos + 1, dm.window);
  int lo = pos + 1 - nkeys;
  int chunk = (nkeys + nsplit - 1) / nsplit;
  *k0 = lo + split * chunk;
  *k1 = min(*k0 + chunk, pos + 1);
}

// One (query, kv head, split) work item: all G query heads of the group share
// every K/V row that is loaded.
template <typename T, int HD, int G>
__device__ inline void attn_item(const ModelDims& dm, const AttnJob& j, float* sm, int qi, int kvh,
                                 int split) {
  constexpr int VEC = HD / 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps_all = blockDim.x >> 5;
  const int nwarps = (j.max_warps > 0 && j.max_warps < nwarps_all) ? j.max_warps : nwarps_all;
  const int half = HD / 2;
  int pos = j.pos ? __ldcg(j.pos + qi) : j.pos0 + qi;
  if (pos < 0 || pos >= dm.max_ctx) {
    if (threadIdx.x == 0) atomicExch(j.err, (int)kDevBadPosition);
    pos = 0;
  }
  const int* ptab = j.page_table + (size_t)(j.seq_stride ? qi : 0) * j.pages_per_seq;
  float* q_s = sm;                    // [G][HD]
  float* k_s = sm + G * HD;           // [HD]
  float* v_s = k_s + HD;              // [HD]
  float* wm = v_s + HD;               // [nwarps][G]
  float* wl = wm + nwarps * G;        // [nwarps][G]
  float* wo = wl + nwarps * G;        // [nwarps][G][HD]
  const float* row = j.qkv + (size_t)qi * dm.nqkv();
  const float att_scale = rsqrtf((float)HD);
  const int nheads_stage = j.appended ? G : G + 2;
  for (int h = warp; h < nheads_stage; h += nwarps_all) {
    if (h <= G) {   // q heads 0..G-1, k head at G
      const float* src = h < G ? row + (size_t)(kvh * G + h) * HD : row + dm.nq() + (size_t)kvh * HD;
      const float* gain = h < G ? j.g_q : j.g_k;
      float* dst = h < G ? q_s + h * HD : k_s;
      float r = 1.0f;
      if (gain) {   // no gain vector: raw q/k, no normalisation
        float ss = 0.f;
        for (int e = lane; e < HD; e += 32) { float v = __ldcg(src + e); ss += v * v; }
        ss = warp_sum(ss);
        r = rsqrtf(ss / (float)HD + dm.eps);
      }
      float post = h < G ? att_scale : 1.0f;
      for (int e = lane; e < half; e += 32) {
        float a0 = __ldcg(src + e) * r * (gain ? gain[e] : 1.0f);
        float b0 = __ldcg(src + e + half) * r * (gain ? gain[e + half] : 1.0f);
        float cs = 1.0f, sn = 0.0f;
        if (j.cosT) {
          size_t ri = j.rope_is_row ? (size_t)e : (size_t)pos * half + e;
          cs = j.cosT[ri];
          sn = j.sinT[ri];
        }
        dst[e] = (a0 * cs - b0 * sn) * post;
        dst[e + half] = (b0 * cs + a0 * sn) * post;
      }
    } else {        // v head: plain copy
      const float* src = row + dm.nq() + dm.nkv() + (size_t)kvh * HD;
      for (int e = lane; e < HD; e += 32) v_s[e] = __ldcg(src + e);
    }
  }
  __syncthreads();
  T* kbase = reinterpret_cast<T*>(j.kv.k);
  T* vbase = reinterpret_cast<T*>(j.kv.v);
  if (!j.appended && split == 0) {   // KV append: exactly one CTA per (query, kv head)
    int page = ptab[pos / kPage], slot = pos % kPage;
    size_t off = (((size_t)page * dm.hkv + kvh) * kPage + slot) * HD;
    for (int e = threadIdx.x; e < HD; e += blockDim.x) {
      if constexpr (sizeof(T) == 4) {
        kbase[off + e] = k_s[e];
        vbase[off + e] = v_s[e];
        if (j.kv.k16) j.kv.k16[off + e] = __float2bfloat16(k_s[e]);
      } else {
        kbase[off + e] = __float2bfloat16(k_s[e]);
        vbase[off + e] = __float2bfloat16(v_s[e]);
      }
      if (j.kv.v16) j.kv.v16[(((size_t)page * dm.hkv + kvh) * HD + e) * kPage + slot] = __float2bfloat16(v_s[e]);
    }
    // later steps fetch these rows with bulk async copies
    asm volatile("fence.proxy.async.global;" ::: "memory");
  }
  // key range of this split
  int k0, k1;
  attn_split_range(dm, pos, j.is_global, j.nsplit, split, &k0, &k1);
  const T* kpre = reinterpret_cast<const T*>(j.k_pre);
  const T* vpre = reinterpret_cast<const T*>(j.v_pre);
  const int kend = warp < nwarps ? k1 : k0;     // idle warps walk no keys
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
  for (int ka = k0 + warp; ka < kend; ka += 2 * nwarps) {
    int kb = ka + nwarps;
    bool hasb = kb < kend;
    float kA[VEC], kB[VEC], vA[VEC], vB[VEC];
    {
      size_t offa = (((size_t)ptab[ka / kPage] * dm.hkv + kvh) * kPage + (ka % kPage)) * HD;
      if (!j.appended && ka == pos) {
#pragma unroll
        for (int c = 0; c < VEC; ++c) { kA[c] = k_s[head_elem<HD>(lane, c)]; vA[c] = v_s[head_elem<HD>(lane, c)]; }
        if constexpr (sizeof(T) == 2) {
#pragma unroll
          for (int c = 0; c < VEC; ++c) {   // what a bf16 cache would hand back
            kA[c] = __bfloat162float(__float2bfloat16(kA[c]));
            vA[c] = __bfloat162float(__float2bfloat16(vA[c]));
          }
        }
      } else if (ka - k0 < j.npre) {
        load_head_row_smem<T, HD>(kpre + (size_t)(ka - k0) * HD, lane, kA);
        load_head_row_smem<T, HD>(vpre + (size_t)(ka - k0) * HD, lane, vA);
      } else {
        load_head_row<T, HD>(kbase + offa, lane, kA);
        load_head_row<T, HD>(vbase + offa, lane, vA);
      }
      if (hasb) {
        size_t offb = (((size_t)ptab[kb / kPage] * dm.hkv + kvh) * kPage + (kb % kPage)) * HD;
        if (!j.appended && kb == pos) {
#pragma unroll
          for (int c = 0; c < VEC; ++c) { kB[c] = k_s[head_elem<HD>(lane, c)]; vB[c] = v_s[head_elem<HD>(lane, c)]; }
          if constexpr (sizeof(T) == 2) {
#pragma unroll
            for (int c = 0; c < VEC; ++c) {
              kB[c] = __bfloat162float(__float2bfloat16(kB[c]));
              vB[c] = __bfloat162float(__float2bfloat16(vB[c]));
            }
          }
        } else if (kb - k0 < j.npre) {
          load_head_row_smem<T, HD>(kpre + (size_t)(kb - k0) * HD, lane, kB);
          load_head_row_smem<T, HD>(vpre + (size_t)(kb - k0) * HD, lane, vB);
        } else {
          load_head_row<T, HD>(kbase + offb, lane, kB);
          load_head_row<T, HD>(vbase + offb, lane, vB);
        }
      } else {
#pragma unroll
        for (int c = 0; c < VEC; ++c) { kB[c] = 0.f; vB[c] = 0.f; }
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sa = 0.f, sb = 0.f;
#pragma unroll
      for (int c = 0; c < VEC; ++c) { sa += q[g][c] * kA[c]; sb += q[g][c] * kB[c]; }
      sa = warp_sum(sa);
      sb = hasb ? warp_sum(sb) : -INFINITY;
      if (!hasb) sb = -INFINITY;
      float mn = fmaxf(m[g], fmaxf(sa, sb));
      float corr = __expf(m[g] - mn);
      float pa = __expf(sa - mn);
      float pb = hasb ? __expf(sb - mn) : 0.f;
      l[g] = l[g] * corr + pa + pb;
      m[g] = mn;
#pragma unroll
      for (int c = 0; c < VEC; ++c) o[g][c] = o[g][c] * corr + pa * vA[c] + pb * vB[c];
    }
  }
  // merge the warps of this CTA
  if (warp < nwarps) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (lane == 0) { wm[warp * G + g] = m[g]; wl[warp * G + g] = l[g]; }
#pragma unroll
      for (int c = 0; c < VEC; ++c) wo[((size_t)warp * G + g) * HD + head_elem<HD>(lane, c)] = o[g][c];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
    int g = i / HD, e = i - g * HD;
    float M = -INFINITY;
    for (int w = 0; w < nwarps; ++w) M = fmaxf(M, wm[w * G + g]);
    float L = 0.f, O = 0.f;
    if (M > -INFINITY) {
      for (int w = 0; w < nwarps; ++w) {
        float f = __expf(wm[w * G + g] - M);
        L += wl[w * G + g] * f;
        O += wo[((size_t)w * G + g) * HD + e] * f;
      }
    }
    if (j.part_o != nullptr) {
      size_t pi = (((size_t)qi * dm.hkv + kvh) * j.nsplit + split) * G + g;
      j.part_o[pi * HD + e] = O;
      if (e == 0) { j.part_ml[pi * 2] = M; j.part_ml[pi * 2 + 1] = L; }
    } else {
      float val = L > 0.f ? O / L : 0.f;
      size_t oi = ((size_t)qi * dm.hq + kvh * G + g) * HD + e;
      if (j.out_f32) j.out_f32[oi] = val;
      if (j.out_bf16) j.out_bf16[oi] = __float2bfloat16(val);
    }
  }
  __syncthreads();
}

template <typename T, int HD>
__device__ inline void attn_item_g(const ModelDims& dm, const AttnJob& j, float* sm, int qi, int kvh, int split) {
  switch (dm.hq / dm.hkv) {
    case 1: attn_item<T, HD, 1>(dm, j, sm, qi, kvh, split); break;
    case 2: attn_item<T, HD, 2>(dm, j, sm, qi, kvh, split); break;
    case 4: attn_item<T, HD, 4>(dm, j, sm, qi, kvh, split); break;
    default: break;   // rejected on the host
  }
}
__device__ inline void attn_dispatch(const ModelDims& dm, const AttnJob& j, float* sm, int qi, int kvh, int split) {
  if (dm.kv_dtype == 0) {
    switch (dm.hd) {
      case 32: attn_item_g<float, 32>(dm, j, sm, qi, kvh, split); break;
      case 64: attn_item_g<float, 64>(dm, j, sm, qi, kvh, split); break;
      case 128: attn_item_g<float, 128>(dm, j, sm, qi, kvh, split); break;
      case 256: attn_item_g<float, 256>(dm, j, sm, qi, kvh, split); break;
      default: break;
    }
  } else {
    switch (dm.hd) {
      case 32: attn_item_g<__nv_bfloat16, 32>(dm, j, sm, qi, kvh, split); break;
      case 64: attn_item_g<__nv_bfloat16, 64>(dm, j, sm, qi, kvh, split); break;
      case 128: attn_item_g<__nv_bfloat16, 128>(dm, j, sm, qi, kvh, split); break;
      case 256: attn_item_g<__nv_bfloat16, 256>(dm, j, sm, qi, kvh, split); break;
      default: break;
    }
  }
}

// ---------------------------------------------------------------------- phases

__device__ inline AttnJob make_decode_attn_job(const DecodeArgs& a, int layer) {
  const LayerWeights& L = a.layers[layer];
  AttnJob j;
  j.qkv = a.qkv;
  j.pos = a.st->pos;
  j.pos0 = 0;
  j.page_table = a.page_table;
  j.pages_per_seq = a.pages_per_seq;
  j.seq_stride = 1;
  j.is_global = L.is_global;
  j.nsplit = L.is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
  j.appended = 0;
  j.g_q = L.g_q;
  j.g_k = L.g_k;
  j.cosT = a.rope_cos[L.is_global ? 1 : 0];
  j.sinT = a.rope_sin[L.is_global ? 1 : 0];
  j.kv = a.kv[layer];
  j.part_o = a.part_o;
  j.part_ml = a.part_ml;
  j.out_f32 = nullptr;
  j.out_bf16 = nullptr;
  j.err = &a.st->err;
  j.k_pre = nullptr;
  j.v_pre = nullptr;
  j.npre = 0;
  j.rope_is_row = 0;
  j.max_warps = 0;
  return j;
}

__device__ inline void phase_qkv(const DecodeArgs& a, const DecodeSmem& s, int layer, int cta, int ncta) {
  const LayerWeights& L = a.layers[layer];
  GemvJob j{L.wqkv, L.sqkv, a.dims.nqkv(), a.dims.d, 1, a.qkv, kEpiPlain};
  int slice, t0, t1;
  bool work = gemv_assignment(j, cta, ncta, &slice, &t0, &t1);
  if (!work && cta != 0) return;
  if (layer == 0) {
    prologue_embed_norm(a, s, cta, a.xres[1], L.g_pre_attn);
  } else {
    prologue_resid_norm(a, s, cta, a.fpart, a.down_slices, a.xres[0], a.xres[1],
                        a.layers[layer - 1].g_post_ffn, L.g_pre_attn);
  }
  if (!work) return;
  quantize_cols(s, a.dims.d, a.ncols, a.nterms);
  gemv_run(j, s, a.ncols, a.nterms, slice, t0, t1, nullptr, nullptr);
}

__device__ inline void phase_attn(const DecodeArgs& a, const DecodeSmem& s, int layer, int cta, int ncta) {
  AttnJob j = make_decode_attn_job(a, layer);
  int items = a.ncols * a.dims.hkv * j.nsplit;
  for (int it = cta; it < items; it += ncta) {
    int split = it % j.nsplit;
    int rest = it / j.nsplit;
    int kvh = rest % a.dims.hkv, col = rest / a.dims.hkv;
    attn_dispatch(a.dims, j, s.attn, col, kvh, split);
  }
}

// Slice sl of the O projection covers heads [sl*hps, (sl+1)*hps).
__device__ inline void phase_oproj(const DecodeArgs& a, const DecodeSmem& s, int layer, int cta, int ncta) {
  const LayerWeights& L = a.layers[layer];
  const ModelDims& dm = a.dims;
  GemvJob j{L.wo, L.so, dm.d, dm.nq(), a.o_slices, a.opart, kEpiPlain};
  int slice, t0, t1;
  if (!gemv_assignment(j, cta, ncta, &slice, &t0, &t1)) return;
  const int Ks = dm.nq() / a.o_slices;      // whole heads
  const int hps = Ks / dm.hd, G = dm.group();
  const int nsplit = L.is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
  for (int col = 0; col < a.ncols; ++col) {
    for (int i = threadIdx.x; i < Ks; i += kDecThreads) {
      int h = slice * hps + i / dm.hd, e = i % dm.hd;
      int kvh = h / G, g = h % G;
      size_t base = (((size_t)col * dm.hkv + kvh) * nsplit) * G + g;
      float M = -INFINITY;
      for (int sp = 0; sp < nsplit; ++sp) M = fmaxf(M, __ldcg(a.part_ml + (base + (size_t)sp * G) * 2));
      float Ls = 0.f, O = 0.f;
      for (int sp = 0; sp < nsplit; ++sp) {
        size_t pi = base + (size_t)sp * G;
        float f = __expf(__ldcg(a.part_ml + pi * 2) - M);
        Ls += __ldcg(a.part_ml + pi * 2 + 1) * f;
        O += __ldcg(a.part_o + pi * dm.hd + e) * f;
      }
      s.xf[(size_t)col * Ks + i] = Ls > 0.f ? O / Ls : 0.f;
    }
  }
  dec_sync();
  quantize_cols(s, Ks, a.ncols, a.nterms);
  gemv_run(j, s, a.ncols, a.nterms, slice, t0, t1, nullptr, nullptr);
}

__device__ inline void phase_gateup(const DecodeArgs& a, const DecodeSmem& s, int layer, int cta, int ncta) {
  const LayerWeights& L = a.layers[layer];
  GemvJob j{L.wgu, L.sgu, 2 * a.dims.ffn, a.dims.d, 1, a.act, kEpiGeglu};
  int slice, t0, t1;
  bool work = gemv_assignment(j, cta, ncta, &slice, &t0, &t1);
  if (!work && cta != 0) return;
  prologue_resid_norm(a, s, cta, a.opart, a.o_slices, a.xres[1], a.xres[0], L.g_post_attn, L.g_pre_ffn);
  if (!work) return;
  quantize_cols(s, a.dims.d, a.ncols, a.nterms);
  gemv_run(j, s, a.ncols, a.nterms, slice, t0, t1, nullptr, nullptr);
}

__device__ inline void phase_down(const DecodeArgs& a, const DecodeSmem& s, int layer, int cta, int ncta) {
  const LayerWeights& L = a.layers[layer];
  GemvJob j{L.wdown, L.sdown, a.dims.d, a.dims.ffn, a.down_slices, a.fpart, kEpiPlain};
  int slice, t0, t1;
  if (!gemv_assignment(j, cta, ncta, &slice, &t0, &t1)) return;
  const int Ks = a.dims.ffn / a.down_slices;
  for (int col = 0; col < a.ncols; ++col)
    for (int i = threadIdx.x; i < Ks; i += kDecThreads)
      s.xf[(size_t)col * Ks + i] = __ldcg(a.act + (size_t)col * a.dims.ffn + (size_t)slice * Ks + i);
  dec_sync();
  quantize_cols(s, Ks, a.ncols, a.nterms);
  gemv_run(j, s, a.ncols, a.nterms, slice, t0, t1, nullptr, nullptr);
}

__device__ inline void phase_head(const DecodeArgs& a, const DecodeSmem& s, int cta, int ncta) {
  const int last = a.dims.n_layers - 1;
  GemvJob j{a.head_w, a.embed_scale, a.dims.vocab, a.dims.d, 1, a.logits, kEpiHead};
  int slice, t0, t1;
  bool work = gemv_assignment(j, cta, ncta, &slice, &t0, &t1);
  float bv[kMaxCols];
  int bi[kMaxCols];
#pragma unroll
  for (int c = 0; c < kMaxCols; ++c) { bv[c] = -INFINITY; bi[c] = 0x7fffffff; }
  if (work) {
    prologue_resid_norm(a, s, cta, a.fpart, a.down_slices, a.xres[0], a.xres[1],
                        a.layers[last].g_post_ffn, a.g_final);
    quantize_cols(s, a.dims.d, a.ncols, a.nterms);
    gemv_run(j, s, a.ncols, a.nterms, slice, t0, t1, bv, bi);
  }
  // CTA-level arg-max (lowest index wins ties), one slot per CTA.
  float* sv = s.argbuf;
  int* si = reinterpret_cast<int*>(s.argbuf + kDecThreads);
  for (int col = 0; col < a.ncols; ++col) {
    dec_sync();
    sv[threadIdx.x] = bv[col];
    si[threadIdx.x] = bi[col];
    dec_sync();
    for (int st = kDecThreads / 2; st > 0; st >>= 1) {
      if (threadIdx.x < st) {
        float ov = sv[threadIdx.x + st];
        int oi = si[threadIdx.x + st];
        if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
          sv[threadIdx.x] = ov;
          si[threadIdx.x] = oi;
        }
      }
      dec_sync();
    }
    if (threadIdx.x == 0) {
      a.amax_val[(size_t)cta * a.ncols + col] = sv[0];
      a.amax_idx[(size_t)cta * a.ncols + col] = si[0];
    }
  }
}

// Final arg-max over the per-CTA candidates; optionally feeds the token back.
__device__ __noinline__ void phase_argmax(const DecodeArgs& a, int ncta_head) {
  if (threadIdx.x < 32) {
    // the state words are fetched up front, next to the first candidates: one L2 round trip, not a chain
    const int sd = threadIdx.x == 0 ? __ldcg(&a.st->steps_done) : 0;
    for (int col = 0; col < a.ncols; ++col) {
      const int pos_now = threadIdx.x == 0 ? __ldcg(&a.st->pos[col]) : 0;
      constexpr int kPer = 8;                       // candidates a lane loads together (covers 256 CTAs)
      float vv[kPer];
      int ii[kPer];
#pragma unroll
      for (int u = 0; u < kPer; ++u) {
        const int c = threadIdx.x + 32 * u;
        const bool in = c < ncta_head;
        vv[u] = in ? __ldcg(a.amax_val + (size_t)c * a.ncols + col) : -INFINITY;
        ii[u] = in ? __ldcg(a.amax_idx + (size_t)c * a.ncols + col) : 0x7fffffff;
      }
      float bv = -INFINITY;
      int bi = 0x7fffffff;
#pragma unroll
      for (int u = 0; u < kPer; ++u)
        if (vv[u] > bv || (vv[u] == bv && ii[u] < bi)) { bv = vv[u]; bi = ii[u]; }
      for (int c = threadIdx.x + 32 * kPer; c < ncta_head; c += 32) {      // grids beyond 256 CTAs
        float v = __ldcg(a.amax_val + (size_t)c * a.ncols + col);
        int i = __ldcg(a.amax_idx + (size_t)c * a.ncols + col);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
      }
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (threadIdx.x == 0) {
        if (bi == 0x7fffffff) bi = 0;
        a.st->out_token[col] = bi;
        if (a.step_tokens && sd < a.step_capacity) a.step_tokens[(size_t)sd * a.ncols + col] = bi;
        if (a.advance) {
          a.st->token[col] = bi;
          a.st->pos[col] = pos_now + 1;
        }
      }
    }
    if (threadIdx.x == 0) a.st->steps_done = sd + 1;
  }
}

// ------------------------------------------------------- one kernel per phase

enum DecodePhase { kPhQkv = 0, kPhAttn, kPhOproj, kPhGateUp, kPhDown, kPhHead, kPhArgmax };

__global__ void __launch_bounds__(kDecThreads, 1)
decode_phase_kernel(const __grid_constant__ DecodeArgs a, int phase, int layer) {
  extern __shared__ __align__(16) unsigned char dsm[];
  DecodeSmem s = carve_smem(dsm, a.dims, a.ncols);
  const int cta = blockIdx.x, ncta = gridDim.x;
  switch (phase) {
    case kPhQkv: phase_qkv(a, s, layer, cta, ncta); break;
    case kPhAttn: phase_attn(a, s, layer, cta, ncta); break;
    case kPhOproj: phase_oproj(a, s, layer, cta, ncta); break;
    case kPhGateUp: phase_gateup(a, s, layer, cta, ncta); break;
    case kPhDown: phase_down(a, s, layer, cta, ncta); break;
    case kPhHead: phase_head(a, s, cta, ncta); break;
    case kPhArgmax: phase_argmax(a, layer /* = head grid size */); break;
  }
}

// ------------------------------------------ persistent kernel: whole step(s)

// Sense-free counting barrier: every CTA adds one and waits for the count to
// reach the next multiple of the grid size.  The wait is bounded; on give-up
// the error word is set and the kernel runs to completion without waiting again.
__device__ __forceinline__ void grid_barrier(DecodeState* st, unsigned int* epoch, int ncta,
                                             long long* trace = nullptr, int bar_idx = 0) {
  dec_sync();
  if (threadIdx.x == 0) {
    *epoch += (unsigned)ncta;
    if (trace) trace[((size_t)bar_idx * ncta + blockIdx.x) * 2] = clock64();
    __threadfence();
    atomicAdd(&st->barrier, 1u);
    unsigned int target = *epoch;
    long spins = 0;
    while (true) {
      unsigned int v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(&st->barrier));
      if ((int)(v - target) >= 0) break;
      ++spins;
      if ((spins & 255) == 0 && *reinterpret_cast<volatile int*>(&st->err) == (int)kDevBarrierTimeout) break;
      if (spins > 4000000L) {   // ~ a second; never reached in a healthy run
        atomicExch(&st->err, (int)kDevBarrierTimeout);
        break;
      }
    }
    if (trace) trace[((size_t)bar_idx * ncta + blockIdx.x) * 2 + 1] = clock64();
  }
  dec_sync();
}

__global__ void __launch_bounds__(kDecThreads, 1)
decode_persistent_kernel(const __grid_constant__ DecodeArgs a, int nsteps, unsigned int epoch0) {
  extern __shared__ __align__(16) unsigned char dsm[];
  DecodeSmem s = carve_smem(dsm, a.dims, a.ncols);
  __shared__ unsigned int epoch;
  if (threadIdx.x == 0) epoch = epoch0;
  dec_sync();
  const int cta = blockIdx.x, ncta = gridDim.x;
  int bar = 0;
  for (int step = 0; step < nsteps; ++step) {
    for (int layer = 0; layer < a.dims.n_layers; ++layer) {
      phase_qkv(a, s, layer, cta, ncta);
      grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
      phase_attn(a, s, layer, cta, ncta);
      grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
      phase_oproj(a, s, layer, cta, ncta);
      grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
      phase_gateup(a, s, layer, cta, ncta);
      grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
      phase_down(a, s, layer, cta, ncta);
      grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
    }
    phase_head(a, s, cta, ncta);
    grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
    if (cta == 0) phase_argmax(a, ncta);
    grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
  }
}

}  // namespace b200lm

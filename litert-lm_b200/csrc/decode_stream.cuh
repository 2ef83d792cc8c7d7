// Streaming persistent decode kernel.
//
// Same phases as decode_ops.cuh (A qkv, B attention, C o-proj, D gate/up, E down,
// H head), one cooperative launch for one or more steps, a grid barrier between
// phases.  What differs is where the bytes come from and who fetches them:
//
//  * every read of HBM-resident data -- int4 weight tiles, their scales, norm
//    gains, cached K/V rows, the RoPE row -- arrives as 1-D bulk async copies
//    (cp.async.bulk, completion on an mbarrier) in a two-halves staging area in
//    shared memory, one or two "fills" ahead of its use;
//  * a dedicated PRODUCER WARP walks the static fill sequence on its own
//    (full / empty mbarriers per half, a small descriptor per fill published in
//    shared memory), so the 16 compute warps never compute addresses or issue
//    copies: after a grid barrier they touch L2-resident activations and shared
//    memory only;
//  * the norm prologues need ONE block reduction: with f the incoming branch
//    output and x = xin + rmsnorm(f) g_post, the sums of f^2, xin^2, xin f g_post
//    and (f g_post)^2 give both RMS factors; activations are quantised against
//    the static bound |rmsnorm(x)_i g_i| <= sqrt(d) max|g|, so no max-reduction.
//
// Fills form one static sequence per CTA: for every phase max(1, rounds) fills,
// fill n lands in half n & 1 and completes full[n & 1] exactly once (empty fills
// just arrive), consumers release the half through empty[n & 1].
#pragma once
#include "common.cuh"
#include "decode_ops.cuh"
#include "prefill_ops.cuh"

namespace b200lm {

#define B2_TP(k)                                                                          \
  do {                                                                                    \
    if (a.trace_pts && threadIdx.x == 0)                                                  \
      a.trace_pts[((size_t)bar * gridDim.x + blockIdx.x) * 8 + (k)] = clock64();          \
  } while (0)

enum StreamPhase { kSA = 0, kSB = 1, kSC = 2, kSD = 3, kSE = 4, kSH = 5 };
constexpr int kStreamThreads = kDecThreads + 32;   // 16 compute warps + 1 producer warp
constexpr int kStreamMaxStagedRows = 1024;         // cap on K/V rows staged per chunk
constexpr int kMaxV4 = 3;                          // float4 per thread held in registers by the norm prologue

struct PhasePlan {     // this CTA's share of one GEMV phase
  int N, K, slices, epilogue, has_gains;
  int work, slice, t0, t1, ktn, tpr, rounds;
};

struct StreamCursor {
  int step, layer, ph, round;
};

struct FillDesc {      // published by the producer for the consumers of one fill
  int ph, layer, round, valid;
  int ta, ntile, ktn, has_gains;          // GEMV fills
  int col, kvh, split, nsplit, k0, npre, is_global, pos;   // attention fills
};

struct StreamCtx {
  DecodeSmem s;                 // activation staging shared with the per-phase kernels
  unsigned char* half[2];
  int half_bytes;
  uint64_t* full;               // [2] bytes of a fill have landed
  uint64_t* empty;              // [2] consumers are done with the half
  uint64_t* aux;                // synchronous fetches inside the attention phase
  FillDesc* slot;               // [2]
  volatile int* step_ready;     // steps whose token / position are final
  LayerWeights* lw;             // [n_layers] copy in shared memory
  LayerKv* lkv;                 // [n_layers]
  PhasePlan* plan;              // [6] indexed by StreamPhase (kSB unused)
  int npre_max;                 // K/V rows a half can hold
  unsigned wait_no;             // fills consumed
  unsigned aux_cnt;
};

__host__ __device__ inline int stream_kmax(const ModelDims& d) {
  int kmax = d.ffn > d.d ? d.ffn : d.d;
  if (d.hq * d.hd > kmax) kmax = d.hq * d.hd;
  return kmax;
}

__host__ __device__ inline size_t stream_attn_bytes(const ModelDims& d) {
  int G = d.hq / d.hkv;
  return ((size_t)(G + 2) * d.hd + (size_t)G * (kStreamMaxStagedRows + 1) + 4 * G) * 4;   // q, k, v, scores
}

__host__ __device__ inline size_t stream_fixed_bytes(const ModelDims& d, int ncols) {
  int kmax = stream_kmax(d);
  size_t act = (size_t)ncols * kmax * 4;                          // xf
  act += (size_t)ncols * 3 * dec_xstride(kmax);                   // xq (three terms)
  size_t attn = stream_attn_bytes(d);
  if (attn > act) act = attn;                                     // attention aliases xf / xq only
  act += (size_t)kMaxRoundUnits * 16 * kQCols * 4 + 16;           // red (kept zero between rounds: never aliased)
  size_t b = act + 64 * 4 + kMaxCols * 4 + 2 * kDecThreads * 4;   // scratch, colscale, argbuf
  b += (size_t)d.n_layers * (sizeof(LayerWeights) + sizeof(LayerKv)) + 6 * sizeof(PhasePlan);
  b += 128 + 2 * sizeof(FillDesc) + 64;                           // mbarriers, descriptors, flags
  return b + 1024;
}

__device__ __forceinline__ void stream_carve(unsigned char* base, const ModelDims& d, int ncols, int half_bytes,
                                             StreamCtx& c) {
  unsigned char* p = reinterpret_cast<unsigned char*>(((uintptr_t)base + 127) & ~(uintptr_t)127);
  c.half[0] = p; p += half_bytes;
  c.half[1] = p; p += half_bytes;
  c.half_bytes = half_bytes;
  c.full = reinterpret_cast<uint64_t*>(p);
  c.empty = c.full + 2;
  c.aux = c.full + 4;
  p += 128;
  c.slot = reinterpret_cast<FillDesc*>(p); p += 2 * sizeof(FillDesc);
  c.step_ready = reinterpret_cast<volatile int*>(p); p += 64;
  int kmax = stream_kmax(d);
  unsigned char* act0 = p;
  c.s.xf = reinterpret_cast<float*>(p); p += (size_t)ncols * kmax * 4;
  c.s.xstride = dec_xstride(kmax);
  c.s.xq = reinterpret_cast<int8_t*>(p); p += (size_t)ncols * 3 * c.s.xstride;
  size_t attn = stream_attn_bytes(d);
  if ((size_t)(p - act0) < attn) p = act0 + attn;
  p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 15) & ~(uintptr_t)15);
  c.s.attn = reinterpret_cast<float*>(act0);
  c.s.red = reinterpret_cast<int*>(p); p += (size_t)kMaxRoundUnits * 16 * kQCols * 4;
  c.s.scratch = reinterpret_cast<float*>(p); p += 64 * 4;
  c.s.colscale = reinterpret_cast<float*>(p); p += kMaxCols * 4;
  c.s.colsum = nullptr;
  c.s.argbuf = reinterpret_cast<float*>(p); p += 2 * kDecThreads * 4;
  c.lw = reinterpret_cast<LayerWeights*>(p); p += (size_t)d.n_layers * sizeof(LayerWeights);
  c.lkv = reinterpret_cast<LayerKv*>(p); p += (size_t)d.n_layers * sizeof(LayerKv);
  c.plan = reinterpret_cast<PhasePlan*>(p);
}

__host__ __device__ inline void stream_phase_shape(const ModelDims& d, int o_slices, int down_slices, int ph, int* N,
                                                   int* K, int* slices, int* epi, int* gains) {
  switch (ph) {
    case kSA: *N = d.nqkv(); *K = d.d; *slices = 1; *epi = kEpiPlain; *gains = 1; break;
    case kSC: *N = d.d; *K = d.nq(); *slices = o_slices; *epi = kEpiPlain; *gains = 0; break;
    case kSD: *N = 2 * d.ffn; *K = d.d; *slices = 1; *epi = kEpiGeglu; *gains = 1; break;
    case kSE: *N = d.d; *K = d.ffn; *slices = down_slices; *epi = kEpiPlain; *gains = 0; break;
    default: *N = d.vocab; *K = d.d; *slices = 1; *epi = kEpiHead; *gains = 1; break;
  }
}

// Tiles of one phase that fit one staging half (0: the model does not fit this kernel).
__host__ __device__ inline int stream_tiles_per_round(const ModelDims& d, int half_bytes, int K, int slices, int epi,
                                                      int gains) {
  int ktn = K / 64 / slices;
  int cap = half_bytes - (gains ? 2 * d.d * 4 : 0);
  int per_tile = ktn * 512 + 64;
  int tpr = cap / per_tile;
  if (tpr > kMaxRoundUnits) tpr = kMaxRoundUnits;
  if (epi == kEpiGeglu) tpr &= ~1;
  return tpr;
}

__host__ inline bool stream_model_fits(const ModelDims& d, int o_slices, int down_slices, int half_bytes) {
  const int phases[5] = {kSA, kSC, kSD, kSE, kSH};
  for (int ph : phases) {
    int N, K, sl, epi, gains;
    stream_phase_shape(d, o_slices, down_slices, ph, &N, &K, &sl, &epi, &gains);
    if (stream_tiles_per_round(d, half_bytes, K, sl, epi, gains) < (epi == kEpiGeglu ? 2 : 1)) return false;
  }
  if (d.d / 4 > kMaxV4 * kDecThreads) return false;
  if (d.hq / d.hkv * d.hd > 2 * kDecThreads) return false;
  int esz = d.kv_dtype == 0 ? 4 : 2;
  if (half_bytes < (int)((size_t)kDecThreads * (d.hq / d.hkv) * 4 + 1024)) return false;   // key-part reduction of the attention
  return half_bytes >= 2 * d.hd * esz + 3 * d.hd * 4 + 64;   // at least one staged K/V row pair + RoPE row + gains
}

__device__ __noinline__ void stream_make_plans(const DecodeArgs& a, StreamCtx& c, int cta, int ncta) {
  const int phases[5] = {kSA, kSC, kSD, kSE, kSH};
  for (int i = 0; i < 5; ++i) {
    PhasePlan& p = c.plan[phases[i]];
    stream_phase_shape(a.dims, a.o_slices, a.down_slices, phases[i], &p.N, &p.K, &p.slices, &p.epilogue, &p.has_gains);
    GemvJob j{nullptr, nullptr, p.N, p.K, p.slices, nullptr, p.epilogue};
    p.work = gemv_assignment(j, cta, ncta, &p.slice, &p.t0, &p.t1) ? 1 : 0;
    p.ktn = p.K / 64 / p.slices;
    p.tpr = stream_tiles_per_round(a.dims, c.half_bytes, p.K, p.slices, p.epilogue, p.has_gains);
    p.rounds = p.work ? (p.t1 - p.t0 + p.tpr - 1) / p.tpr : 0;
  }
}

__device__ __forceinline__ void stream_advance(StreamCursor& cur, const StreamCtx& c, int n_layers) {
  int fills = cur.ph == kSB ? 1 : (c.plan[cur.ph].rounds > 1 ? c.plan[cur.ph].rounds : 1);
  if (++cur.round < fills) return;
  cur.round = 0;
  if (cur.ph == kSH) { cur.ph = kSA; cur.layer = 0; ++cur.step; return; }
  if (cur.ph == kSE) {
    if (cur.layer + 1 < n_layers) { ++cur.layer; cur.ph = kSA; } else { cur.ph = kSH; }
    return;
  }
  ++cur.ph;
}

// ------------------------------------------------------------ producer warp

__device__ __noinline__ void stream_producer(const DecodeArgs& a, StreamCtx& c, int cta, int nsteps) {
  const int lane = threadIdx.x & 31;
  const ModelDims& dm = a.dims;
  const int last = dm.n_layers - 1;
  StreamCursor cur{0, 0, kSA, 0};
  for (unsigned n = 0; cur.step < nsteps; ++n) {
    const unsigned h = n & 1u;
    if (n >= 2 && !mbar_wait(&c.empty[h], ((n >> 1) - 1u) & 1u, &a.st->err)) return;
    unsigned char* dst = c.half[h];
    uint64_t* bar = &c.full[h];
    FillDesc d;
    d.ph = cur.ph; d.layer = cur.layer; d.round = cur.round; d.valid = 0;
    d.ta = d.ntile = d.ktn = d.has_gains = 0;
    d.col = d.kvh = d.split = d.nsplit = d.k0 = d.npre = d.is_global = d.pos = 0;
    if (cur.ph == kSB) {
      // token / position of this step must be final before its rows are chosen
      for (long spins = 0; *c.step_ready <= cur.step; ++spins) {
        __nanosleep(40);
        if (spins > 20000000L) { atomicExch(&a.st->err, (int)kDevBarrierTimeout); return; }
      }
      d.is_global = c.lw[cur.layer].is_global;
      d.nsplit = d.is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
      const int items = a.ncols * dm.hkv * d.nsplit;
      if (cta < items) {
        d.valid = 1;
        d.split = cta % d.nsplit;
        int rest = cta / d.nsplit;
        d.kvh = rest % dm.hkv;
        d.col = rest / dm.hkv;
        int pos = __ldcg(&a.st->pos[d.col]);
        if (pos < 0 || pos >= dm.max_ctx) {
          if (lane == 0) atomicExch(&a.st->err, (int)kDevBadPosition);
          pos = 0;
        }
        int k0, k1;
        attn_split_range(dm, pos, d.is_global, d.nsplit, d.split, &k0, &k1);
        d.k0 = k0;
        d.pos = pos;
        int nold = min(k1, pos) - k0;        // the row of `pos` itself is not in the cache yet
        d.npre = nold < 0 ? 0 : min(nold, c.npre_max);
        if (lane == 0) c.slot[h] = d;
        __syncwarp();
        const int esz = dm.kv_dtype == 0 ? 4 : 2;
        const uint32_t row = (uint32_t)dm.hd * esz;
        const uint32_t rope_row = (uint32_t)(dm.hd / 2) * 4;
        const uint32_t gain_row = (uint32_t)dm.hd * 4;
        if (lane == 0) mbar_arrive_expect_tx(bar, 2u * d.npre * row + 2u * rope_row + 2u * gain_row);
        __syncwarp();
        const int* ptab = a.page_table + (size_t)d.col * a.pages_per_seq;
        const unsigned char* kb = reinterpret_cast<const unsigned char*>(c.lkv[cur.layer].k);
        const unsigned char* vb = reinterpret_cast<const unsigned char*>(c.lkv[cur.layer].v);
        for (int i = lane; i < 2 * d.npre; i += 32) {
          int r = i >> 1, isv = i & 1, key = d.k0 + r;
          size_t off = ((((size_t)ptab[key / kPage] * dm.hkv + d.kvh) * kPage + (key % kPage)) * dm.hd) * esz;
          bulk_load_1d(dst + (size_t)(isv ? c.npre_max : 0) * row + (size_t)r * row, (isv ? vb : kb) + off, row, bar);
        }
        if (lane == 31) {
          const int t = d.is_global ? 1 : 0;
          unsigned char* rp = dst + (size_t)2 * c.npre_max * row;
          bulk_load_1d(rp, a.rope_cos[t] + (size_t)pos * (dm.hd / 2), rope_row, bar);
          bulk_load_1d(rp + rope_row, a.rope_sin[t] + (size_t)pos * (dm.hd / 2), rope_row, bar);
        }
        if (lane == 30) {     // QK-norm gains behind the RoPE rows
          unsigned char* gp = dst + (size_t)2 * c.npre_max * row + 2u * rope_row;
          bulk_load_1d(gp, c.lw[cur.layer].g_q, gain_row, bar);
          bulk_load_1d(gp + gain_row, c.lw[cur.layer].g_k, gain_row, bar);
        }
      }
    } else {
      const PhasePlan& p = c.plan[cur.ph];
      if (p.work && cur.round < p.rounds) {
        const LayerWeights& L = c.lw[cur.ph == kSH ? last : cur.layer];
        const uint4* w;
        const float* wscale;
        const float *g_post = nullptr, *g_pre = nullptr;
        switch (cur.ph) {
          case kSA: w = L.wqkv; wscale = L.sqkv; g_pre = L.g_pre_attn;
                    g_post = cur.layer > 0 ? c.lw[cur.layer - 1].g_post_ffn : nullptr; break;
          case kSC: w = L.wo; wscale = L.so; break;
          case kSD: w = L.wgu; wscale = L.sgu; g_pre = L.g_pre_ffn; g_post = L.g_post_attn; break;
          case kSE: w = L.wdown; wscale = L.sdown; break;
          default: w = a.head_w; wscale = a.embed_scale; g_pre = a.g_final; g_post = L.g_post_ffn; break;
        }
        d.valid = 1;
        d.ktn = p.ktn;
        d.ta = p.t0 + cur.round * p.tpr;
        d.ntile = min(p.tpr, p.t1 - d.ta);
        d.has_gains = (p.has_gains && cur.round == 0) ? 1 : 0;
        if (lane == 0) c.slot[h] = d;
        __syncwarp();
        const int KT = p.K / 64, kt0 = p.slice * p.ktn;
        const uint32_t tile_bytes = (uint32_t)p.ktn * 512u;
        const uint32_t wbytes = (uint32_t)d.ntile * tile_bytes;
        const uint32_t sbytes = (uint32_t)d.ntile * 64u;
        const uint32_t gbytes = (uint32_t)dm.d * 4u;
        uint32_t total = wbytes + sbytes + (d.has_gains ? (g_post ? 2u : 1u) * gbytes : 0u);
        if (lane == 0) mbar_arrive_expect_tx(bar, total);
        __syncwarp();
        if (p.slices == 1) {
          // one contiguous run of ntile * KT tiles, cut into 8 KiB pieces over the lanes
          const unsigned char* src = reinterpret_cast<const unsigned char*>(w + (size_t)d.ta * KT * 32);
          const uint32_t piece = 8192u;
          const uint32_t npieces = (wbytes + piece - 1) / piece;
          for (uint32_t i = lane; i < npieces; i += 32) {
            uint32_t o = i * piece, nb = min(piece, wbytes - o);
            bulk_load_1d(dst + o, src + o, nb, bar);
          }
        } else {
          for (int i = lane; i < d.ntile; i += 32) {
            const unsigned char* src = reinterpret_cast<const unsigned char*>(w + ((size_t)(d.ta + i) * KT + kt0) * 32);
            bulk_load_1d(dst + (size_t)i * tile_bytes, src, tile_bytes, bar);
          }
        }
        if (lane == 31) bulk_load_1d(dst + wbytes, wscale + (size_t)d.ta * 16, sbytes, bar);
        if (d.has_gains) {
          if (lane == 30) bulk_load_1d(dst + wbytes + sbytes, g_pre, gbytes, bar);
          if (lane == 29 && g_post) bulk_load_1d(dst + wbytes + sbytes + gbytes, g_post, gbytes, bar);
        }
      }
    }
    if (!d.valid) {
      if (lane == 0) {
        c.slot[h] = d;
        mbar_arrive(bar);      // an empty fill still completes its barrier phase
      }
      __syncwarp();
    }
    stream_advance(cur, c, dm.n_layers);
  }
}

// ------------------------------------------------------------ consumer side

__device__ __forceinline__ const FillDesc* stream_acquire(StreamCtx& c, unsigned char** hb, int* err) {
  const unsigned n = c.wait_no, h = n & 1u;
  mbar_wait(&c.full[h], (n >> 1) & 1u, err);
  *hb = c.half[h];
  return &c.slot[h];
}
// All compute threads are done with the half of the current fill.
__device__ __forceinline__ void stream_release(StreamCtx& c) {
  const unsigned h = c.wait_no & 1u;
  ++c.wait_no;
  dec_sync();
  if (threadIdx.x == 0) mbar_arrive(&c.empty[h]);
}
// The same, with the block barrier and the arrive left to the grid barrier that follows at once
// (stream_grid_barrier): one block barrier less per phase.
__device__ __forceinline__ uint64_t* stream_release_deferred(StreamCtx& c) {
  const unsigned h = c.wait_no & 1u;
  ++c.wait_no;
  return &c.empty[h];
}

// grid_barrier (decode_ops.cuh) that first hands a staging half back to the producer: the block barrier
// at its entry is the one that release needs.
__device__ __forceinline__ void stream_grid_barrier(DecodeState* st, unsigned int* epoch, int ncta, uint64_t* release,
                                                    long long* trace, int bar_idx) {
  dec_sync();
  if (threadIdx.x == 0) {
    if (release) mbar_arrive(release);
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

// tiles in shared memory: tile u at wsm + u * ktn * 32 (uint4 units)
__device__ __forceinline__ void gemv_tiles_smem(const uint4* wsm, int ktn, int nu, QuantCols xc, int* red) {
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
  int un = beg / ktn, kt = beg - un * ktn - 1;
#pragma unroll 2
  for (int b = beg; b < end; ++b) {
    if (++kt == ktn) { kt = 0; ++un; }
    uint4 w = wsm[(size_t)b * 32 + lane];
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
    mma_tile_words(acc, w, b0, b1, b2, b3);
  }
  if (cur >= 0) flush_tile(red, cur, acc, lane, xc.nq);
}

// Four sums in one block reduction.
__device__ __forceinline__ void block_sum4(float (&v)[4], float* scratch) {
#pragma unroll
  for (int k = 0; k < 4; ++k) v[k] = warp_sum(v[k]);
  dec_sync();
  if ((threadIdx.x & 31) == 0) {
#pragma unroll
    for (int k = 0; k < 4; ++k) scratch[k * kDecWarps + (threadIdx.x >> 5)] = v[k];
  }
  dec_sync();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float s = scratch[k * kDecWarps + (threadIdx.x & (kDecWarps - 1))];
#pragma unroll
    for (int o = kDecWarps / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    v[k] = s;
  }
}

// Quantises four consecutive values (already divided by the scale) and stores each term as one word.
__device__ __forceinline__ void quantize4(float4 r, int nterms, int8_t* q0, int stride) {
  float v[4] = {r.x, r.y, r.z, r.w};
  uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float t0 = fminf(fmaxf(rintf(v[k]), -127.f), 127.f);
    w0 |= ((uint32_t)(int)t0 & 0xFFu) << (8 * k);
    float r1 = (v[k] - t0) * 128.0f;
    float t1 = fminf(fmaxf(rintf(r1), -127.f), 127.f);
    w1 |= ((uint32_t)(int)t1 & 0xFFu) << (8 * k);
    float r2 = (r1 - t1) * 128.0f;
    float t2 = fminf(fmaxf(rintf(r2), -127.f), 127.f);
    w2 |= ((uint32_t)(int)t2 & 0xFFu) << (8 * k);
  }
  *reinterpret_cast<uint32_t*>(q0) = w0;
  if (nterms > 1) *reinterpret_cast<uint32_t*>(q0 + stride) = w1;
  if (nterms > 2) *reinterpret_cast<uint32_t*>(q0 + 2 * stride) = w2;
}

// x = xin + rmsnorm(sum parts) * g_post ; xout <- x (cta 0) ; xq <- quantised rmsnorm(x) * g_pre.
// One pass over L2 (16-byte loads held in registers), one block reduction.
__device__ __forceinline__ void stream_prologue_resid(const DecodeArgs& a, StreamCtx& c, int cta, const float* parts,
                                                      int nparts, const float* xin, float* xout, const float* g_post,
                                                      const float* g_pre, float gmax_pre, int bar) {
  const int d = a.dims.d, d4 = d / 4;
  const DecodeSmem& s = c.s;
  const float bound = sqrtf((float)d) * gmax_pre * 1.0001f;     // |rmsnorm(x)_i g_i| never exceeds it
  const float inv = bound > 0.f ? 127.0f / bound : 0.f;
  for (int col = 0; col < a.ncols; ++col) {
    float4 f[kMaxV4], xi[kMaxV4], gp[kMaxV4];
    float sums[4] = {0.f, 0.f, 0.f, 0.f};    // f^2, xin^2, xin f g_post, (f g_post)^2
#pragma unroll
    for (int u = 0; u < kMaxV4; ++u) {
      const int i = threadIdx.x + u * kDecThreads;
      f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      xi[u] = f[u];
      gp[u] = f[u];
      if (i < d4) {
        for (int p = 0; p < nparts; ++p) {
          float4 v = __ldcg(reinterpret_cast<const float4*>(parts + ((size_t)p * a.ncols + col) * d) + i);
          f[u].x += v.x; f[u].y += v.y; f[u].z += v.z; f[u].w += v.w;
        }
        xi[u] = __ldcg(reinterpret_cast<const float4*>(xin + (size_t)col * d) + i);
        gp[u] = reinterpret_cast<const float4*>(g_post)[i];
      }
    }
#pragma unroll
    for (int u = 0; u < kMaxV4; ++u) {
      float4 fg = make_float4(f[u].x * gp[u].x, f[u].y * gp[u].y, f[u].z * gp[u].z, f[u].w * gp[u].w);
      sums[0] += f[u].x * f[u].x + f[u].y * f[u].y + f[u].z * f[u].z + f[u].w * f[u].w;
      sums[1] += xi[u].x * xi[u].x + xi[u].y * xi[u].y + xi[u].z * xi[u].z + xi[u].w * xi[u].w;
      sums[2] += xi[u].x * fg.x + xi[u].y * fg.y + xi[u].z * fg.z + xi[u].w * fg.w;
      sums[3] += fg.x * fg.x + fg.y * fg.y + fg.z * fg.z + fg.w * fg.w;
      gp[u] = fg;
    }
    if (col == 0) B2_TP(2);
    block_sum4(sums, s.scratch);
    if (col == 0) B2_TP(7);
    const float r = rsqrtf(sums[0] / (float)d + a.dims.eps);
    const float ss2 = fmaxf(sums[1] + 2.0f * r * sums[2] + r * r * sums[3], 0.f);
    const float r2 = rsqrtf(ss2 / (float)d + a.dims.eps);
    int8_t* q0 = s.xq + (size_t)(col * a.nterms) * s.xstride;
#pragma unroll
    for (int u = 0; u < kMaxV4; ++u) {
      const int i = threadIdx.x + u * kDecThreads;
      if (i < d4) {
        float4 x = make_float4(xi[u].x + r * gp[u].x, xi[u].y + r * gp[u].y, xi[u].z + r * gp[u].z, xi[u].w + r * gp[u].w);
        if (cta == 0) reinterpret_cast<float4*>(xout + (size_t)col * d)[i] = x;
        float4 gq = reinterpret_cast<const float4*>(g_pre)[i];
        const float k = r2 * inv;
        quantize4(make_float4(x.x * gq.x * k, x.y * gq.y * k, x.z * gq.z * k, x.w * gq.w * k), a.nterms, q0 + 4 * i, s.xstride);
      }
    }
    if (threadIdx.x == 0) s.colscale[col] = bound / 127.0f;
  }
  dec_sync();
}

__device__ __noinline__ void stream_prologue_embed(const DecodeArgs& a, StreamCtx& c, int cta, float* xout,
                                                      const float* g_pre, float gmax_pre) {
  const int d = a.dims.d;
  const DecodeSmem& s = c.s;
  const float emb = sqrtf((float)d);
  const float bound = sqrtf((float)d) * gmax_pre * 1.0001f;
  const float inv = bound > 0.f ? 127.0f / bound : 0.f;
  for (int col = 0; col < a.ncols; ++col) {
    int tok = __ldcg(&a.st->token[col]);
    if (tok < 0 || tok >= a.dims.vocab) {
      if (threadIdx.x == 0) atomicExch(&a.st->err, (int)kDevBadToken);
      tok = 0;
    }
    const uint8_t* row = a.embed_rows + (size_t)tok * (d / 2);
    const float sc = a.embed_scale[tok] * emb;
    float* x = s.xf + (size_t)col * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += kDecThreads) {
      int b = row[i >> 1];
      int nib = (i & 1) ? (b >> 4) : (b & 0xF);
      float v = (float)(nib >= 8 ? nib - 16 : nib) * sc;
      x[i] = v;
      ss += v * v;
      if (cta == 0) xout[(size_t)col * d + i] = v;
    }
    ss = block_sum(ss, s.scratch);
    const float k = rsqrtf(ss / (float)d + a.dims.eps) * inv;
    int8_t* q0 = s.xq + (size_t)(col * a.nterms) * s.xstride;
    for (int i = threadIdx.x; i < d; i += kDecThreads) quantize_value(x[i] * g_pre[i] * k, a.nterms, q0 + i, s.xstride);
    if (threadIdx.x == 0) s.colscale[col] = bound / 127.0f;
  }
  dec_sync();
}

// ---------------------------------------------------------------- attention
// One (query, kv head, split) item with its K/V rows staged in shared memory.
// Scores: one thread per (head, key) walks the row in a lane-rotated order, so
// the 32 rows a warp touches fall into different banks.  One softmax per CTA
// per chunk (no per-warp partial states), then one thread per output element
// accumulates P.V.  Splits longer than the staging half are processed in
// chunks with an online softmax; chunks that were not prefetched are fetched
// synchronously (compute warp 0 issues, everybody waits on the aux barrier).
template <typename T>
__device__ __forceinline__ float4 load4_smem(const T* p) {
  if constexpr (sizeof(T) == 4) {
    return *reinterpret_cast<const float4*>(p);
  } else {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    __nv_bfloat162 x = *reinterpret_cast<__nv_bfloat162*>(&v.x);
    __nv_bfloat162 y = *reinterpret_cast<__nv_bfloat162*>(&v.y);
    return make_float4(__low2float(x), __high2float(x), __low2float(y), __high2float(y));
  }
}

// This lane's DPL elements of a row of HD = 32 * DPL values: a staged K row (cache type T), or an fp32
// row in shared memory when `row` is null.  For DPL >= 4 the lane takes 4-element groups 128 elements
// apart (group c = elements c*128 + 4*lane ..), so a warp's 16-byte loads fall on consecutive addresses.
template <typename T, int DPL>
__device__ __forceinline__ void stream_load_dims(const T* row, const float* fresh, int lane, float (&out)[DPL]) {
  if constexpr (DPL % 4 == 0) {
#pragma unroll
    for (int c = 0; c < DPL / 4; ++c) {
      float4 t = row ? load4_smem<T>(row + c * 128 + 4 * lane) : *reinterpret_cast<const float4*>(fresh + c * 128 + 4 * lane);
      out[4 * c] = t.x; out[4 * c + 1] = t.y; out[4 * c + 2] = t.z; out[4 * c + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < DPL; ++i) out[i] = row ? kv_to_float<T>(row[lane * DPL + i]) : fresh[lane * DPL + i];
  }
}

struct AttnItem {
  int layer, col, kvh, split, nsplit, is_global;
  int bar;                  // barrier index of the phase (timeline stamps)
  int pos;                  // position of the query
  int nstaged;              // rows of chunk 0 already in the half (prefetched), else -1
  const float *cos_r, *sin_r;   // RoPE row of the query position (shared or global memory)
  const float *g_q, *g_k;       // QK-norm gains (shared or global memory)
};

template <typename T, int HD, int G>
__device__ __forceinline__ void attn_smem_item(const DecodeArgs& a, StreamCtx& c, const AttnItem& it, unsigned char* hb) {
  const ModelDims& dm = a.dims;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int half = HD / 2, C4 = HD / 4;
  const int qi = it.col, kvh = it.kvh;
  const int bar = it.bar;
  const LayerWeights& L = c.lw[it.layer];
  const LayerKv kv = c.lkv[it.layer];
  const int pos = it.pos;
  const int cap = c.npre_max;
  float* q_s = c.s.attn;               // [G][HD]
  float* k_s = q_s + G * HD;           // [HD] new key (normed, roped)
  float* v_s = k_s + HD;               // [HD]
  float* sc = v_s + HD;                // [G][cap + 1] probabilities exp(score - bound)
  const size_t rowb = (size_t)HD * sizeof(T);
  const T* kpre = reinterpret_cast<const T*>(hb);
  const T* vpre = reinterpret_cast<const T*>(hb + (size_t)cap * rowb);
  const float* row = a.qkv + (size_t)qi * dm.nqkv();
  const float att_scale = rsqrtf((float)HD);
  // Q and K are RMS-normalised, so every score is at most L.attn_bound in magnitude: the softmax is
  // shifted by that constant instead of a running maximum, and the partial sums of the splits
  // simply add up (no per-split maximum, no rescaling).
  const float shift = L.attn_bound;
  // ---- stage q heads, the new key and value
  for (int h = warp; h < G + 2; h += kDecWarps) {
    if (h <= G) {
      const float* src = h < G ? row + (size_t)(kvh * G + h) * HD : row + dm.nq() + (size_t)kvh * HD;
      const float* gain = h < G ? it.g_q : it.g_k;
      float* dst = h < G ? q_s + h * HD : k_s;
      float v[HD / 32];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < HD / 32; ++i) { v[i] = __ldcg(src + lane + 32 * i); ss += v[i] * v[i]; }
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / (float)HD + dm.eps);
      const float post = h < G ? att_scale : 1.0f;
      if constexpr (HD == 32) {                 // the pair of element e sits 16 lanes away
        float x = v[0] * r * gain[lane];
        float y = __shfl_xor_sync(0xffffffffu, x, 16);
        if (lane < 16) {
          float cs = it.cos_r[lane], sn = it.sin_r[lane];
          dst[lane] = (x * cs - y * sn) * post;
          dst[lane + 16] = (y * cs + x * sn) * post;
        }
      } else {
#pragma unroll
        for (int i = 0; i < HD / 64; ++i) {     // element e = lane + 32 i pairs with e + half
          const int e = lane + 32 * i;
          float a0 = v[i] * r * gain[e], b0 = v[i + HD / 64] * r * gain[e + half];
          float cs = it.cos_r[e], sn = it.sin_r[e];
          dst[e] = (a0 * cs - b0 * sn) * post;
          dst[e + half] = (b0 * cs + a0 * sn) * post;
        }
      }
    } else {
      const float* src = row + dm.nq() + dm.nkv() + (size_t)kvh * HD;
#pragma unroll
      for (int i = 0; i < HD / 32; ++i) v_s[lane + 32 * i] = __ldcg(src + lane + 32 * i);
    }
  }
  dec_sync();
  B2_TP(2);
  const int* ptab = a.page_table + (size_t)qi * a.pages_per_seq;
  if (it.split == 0) {     // KV append: exactly one CTA per (query, kv head)
    T* kbase = reinterpret_cast<T*>(kv.k);
    T* vbase = reinterpret_cast<T*>(kv.v);
    const int page = ptab[pos / kPage], slot = pos % kPage;
    size_t off = (((size_t)page * dm.hkv + kvh) * kPage + slot) * HD;
    for (int e = threadIdx.x; e < HD; e += kDecThreads) {
      if constexpr (sizeof(T) == 4) {
        kbase[off + e] = k_s[e];
        vbase[off + e] = v_s[e];
        if (kv.k16) kv.k16[off + e] = __float2bfloat16(k_s[e]);
      } else {
        kbase[off + e] = __float2bfloat16(k_s[e]);
        vbase[off + e] = __float2bfloat16(v_s[e]);
      }
      if (kv.v16) kv.v16[(((size_t)page * dm.hkv + kvh) * HD + e) * kPage + slot] = __float2bfloat16(v_s[e]);
    }
    asm volatile("fence.proxy.async.global;" ::: "memory");   // later steps fetch these rows with bulk async copies
  }
  int k0, k1;
  attn_split_range(dm, pos, it.is_global, it.nsplit, it.split, &k0, &k1);
  const bool has_new = k1 == pos + 1 && k1 > k0;      // this split ends with the new key
  const int n_old = (has_new ? k1 - 1 : k1) - k0;     // rows that live in the cache
  if constexpr (sizeof(T) == 2) {                     // what a bf16 cache would hand back
    for (int e = threadIdx.x; e < HD; e += kDecThreads) {
      k_s[e] = __bfloat162float(__float2bfloat16(k_s[e]));
      v_s[e] = __bfloat162float(__float2bfloat16(v_s[e]));
    }
    dec_sync();
  }
  // P.V ownership: thread = (element e of the head dimension, key part kp); it accumulates all G heads
  constexpr int KP = kDecThreads / HD;               // key parts
  constexpr int DPL = HD / 32;                       // dims of a row per lane in the score stage
  const int pv_e = threadIdx.x % HD, pv_part = threadIdx.x / HD;
  float o[G], lsum[G];
#pragma unroll
  for (int g = 0; g < G; ++g) { o[g] = 0.f; lsum[g] = 0.f; }
  // the score stage keeps this lane's dims of every q head in registers
  float qreg[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) stream_load_dims<float, DPL>(nullptr, q_s + g * HD, lane, qreg[g]);
  const int nchunks = n_old <= 0 ? 1 : (n_old + cap - 1) / cap;
  for (int ch = 0; ch < nchunks; ++ch) {
    const int c0 = ch * cap;
    const int nrows = max(0, min(cap, n_old - c0));
    const bool staged = ch == 0 && it.nstaged >= nrows;
    if (!staged && nrows > 0) {       // fetch these rows into the half now
      dec_sync();
      if (threadIdx.x < 32) {
        if (lane == 0) mbar_arrive_expect_tx(c.aux, 2u * (uint32_t)nrows * (uint32_t)rowb);
        __syncwarp();
        const unsigned char* kb = reinterpret_cast<const unsigned char*>(kv.k);
        const unsigned char* vb = reinterpret_cast<const unsigned char*>(kv.v);
        for (int i = lane; i < 2 * nrows; i += 32) {
          int r = i >> 1, isv = i & 1, key = k0 + c0 + r;
          size_t off = ((((size_t)ptab[key / kPage] * dm.hkv + kvh) * kPage + (key % kPage)) * HD) * sizeof(T);
          bulk_load_1d(hb + (size_t)(isv ? cap : 0) * rowb + (size_t)r * rowb, (isv ? vb : kb) + off, (uint32_t)rowb, c.aux);
        }
      }
      unsigned par = c.aux_cnt & 1u;
      ++c.aux_cnt;
      mbar_wait(c.aux, par, &a.st->err);
    }
    const bool lastc = ch == nchunks - 1;
    const int nk = nrows + ((lastc && has_new) ? 1 : 0);
    if (ch == 0) B2_TP(7);
    // ---- probabilities p[key][head] = exp(q_head . k_key - shift): a warp takes two keys at a time,
    //      lane l the dims [l*DPL, (l+1)*DPL) of both rows against all G heads; each K row is read once
    for (int kp = warp; 2 * kp < nk; kp += kDecWarps) {
      const int ka = 2 * kp, kb_ = min(2 * kp + 1, nk - 1);
      float xa[DPL], xb[DPL];
      stream_load_dims<T, DPL>(ka < nrows ? kpre + (size_t)ka * HD : nullptr, k_s, lane, xa);
      stream_load_dims<T, DPL>(kb_ < nrows ? kpre + (size_t)kb_ * HD : nullptr, k_s, lane, xb);
      float acc[2 * G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) { sa += qreg[g][i] * xa[i]; sb += qreg[g][i] * xb[i]; }
        acc[2 * g] = sa;
        acc[2 * g + 1] = sb;
      }
#pragma unroll
      for (int j = 0; j < 2 * G; ++j) acc[j] = warp_sum(acc[j]);
      if (lane < 2 * G) {
        const int g = lane >> 1, second = lane & 1;
        float v = acc[0];
#pragma unroll
        for (int j = 1; j < 2 * G; ++j) v = lane == j ? acc[j] : v;
        const int kk = second ? 2 * kp + 1 : ka;
        if (kk < nk) sc[kk * G + g] = __expf(v - shift);
      }
    }
    dec_sync();
    if (ch == 0) B2_TP(3);
    // ---- P.V and the row sums: this thread's element of V against the probabilities of all heads
    for (int kk = pv_part; kk < nk; kk += KP) {
      const float v = kk < nrows ? kv_to_float<T>(vpre[(size_t)kk * HD + pv_e]) : v_s[pv_e];
      float pg[G];
      if constexpr (G == 4) {          // one 16-byte broadcast load for the four heads
        const float4 t = *reinterpret_cast<const float4*>(sc + kk * 4);
        pg[0] = t.x; pg[1] = t.y; pg[2] = t.z; pg[3] = t.w;
      } else {
#pragma unroll
        for (int g = 0; g < G; ++g) pg[g] = sc[kk * G + g];
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        o[g] += pg[g] * v;
        lsum[g] += pg[g];
      }
    }
    if (ch + 1 < nchunks) dec_sync();      // the next chunk overwrites the rows and the probabilities
  }
  B2_TP(5);
  // ---- the key parts meet in shared memory (over the K rows, which are not needed any more),
  //      then part 0 writes the split's partial result: row sum l and unnormalised o, both relative to the shift
  dec_sync();
  float* ored = reinterpret_cast<float*>(hb);                  // [KP][G][HD]
  float* lred = ored + (size_t)KP * G * HD;                    // [KP][G]
  if (pv_part > 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) ored[((size_t)pv_part * G + g) * HD + pv_e] = o[g];
  }
  if (pv_e == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) lred[pv_part * G + g] = lsum[g];
  }
  dec_sync();
  if (pv_part == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float acc = o[g];
      for (int kp = 1; kp < KP; ++kp) acc += ored[((size_t)kp * G + g) * HD + pv_e];
      size_t pi = (((size_t)qi * dm.hkv + kvh) * it.nsplit + it.split) * G + g;
      a.part_o[pi * HD + pv_e] = acc;
      if (pv_e == 0) {
        float ls = 0.f;
        for (int kp = 0; kp < KP; ++kp) ls += lred[kp * G + g];
        a.part_ml[pi * 2] = shift;
        a.part_ml[pi * 2 + 1] = ls;
      }
    }
  }
  dec_sync();
  B2_TP(6);
}

// Input of the down projection: this CTA's K slice of the GeGLU activations, quantised per session
// with its own maximum.  The values stay in registers between the maximum and the quantisation
// (up to kMaxV4Down float4 per thread); wider slices go through the shared staging vector.
constexpr int kMaxV4Down = 4;
__device__ __forceinline__ void stream_prologue_down(const DecodeArgs& a, StreamCtx& c, int slice) {
  const ModelDims& dm = a.dims;
  const int Ks = dm.ffn / a.down_slices, n4 = Ks / 4;
  if (n4 > kMaxV4Down * kDecThreads) {
    for (int col = 0; col < a.ncols; ++col)
      for (int i = threadIdx.x; i < n4; i += kDecThreads)
        reinterpret_cast<float4*>(c.s.xf + (size_t)col * Ks)[i] =
            __ldcg(reinterpret_cast<const float4*>(a.act + (size_t)col * dm.ffn + (size_t)slice * Ks) + i);
    dec_sync();
    quantize_cols(c.s, Ks, a.ncols, a.nterms);
    return;
  }
  for (int col = 0; col < a.ncols; ++col) {
    const float4* src = reinterpret_cast<const float4*>(a.act + (size_t)col * dm.ffn + (size_t)slice * Ks);
    float4 v[kMaxV4Down];
    float m = 0.f;
#pragma unroll
    for (int u = 0; u < kMaxV4Down; ++u) {
      const int i = threadIdx.x + u * kDecThreads;
      v[u] = i < n4 ? __ldcg(src + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      m = fmaxf(m, fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w))));
    }
    m = block_max(m, c.s.scratch);
    const float inv = m > 0.f ? 127.0f / m : 0.f;
    int8_t* q0 = c.s.xq + (size_t)(col * a.nterms) * c.s.xstride;
#pragma unroll
    for (int u = 0; u < kMaxV4Down; ++u) {
      const int i = threadIdx.x + u * kDecThreads;
      if (i < n4) quantize4(make_float4(v[u].x * inv, v[u].y * inv, v[u].z * inv, v[u].w * inv), a.nterms, q0 + 4 * i, c.s.xstride);
    }
    if (threadIdx.x == 0) c.s.colscale[col] = m > 0.f ? m / 127.0f : 0.f;
    dec_sync();               // scratch is reused by the next session's maximum; xq is complete
  }
}

// Combine of the split partials of one head slice into xf (then quantised).  All splits share one
// softmax shift, so the combine is sum(o) / sum(l).  The splits of an output are dealt to as many
// threads as the block has per output and every load of a thread is independent of the others.
// The row sums l are fetched by ONE warp per head of the slice (a lane per split): they are a few
// cache lines that every CTA of the grid reads, so each CTA asks for them once, not once per thread.
__device__ __forceinline__ void stream_prologue_combine(const DecodeArgs& a, StreamCtx& c, int layer, int bar) {
  const ModelDims& dm = a.dims;
  const PhasePlan& p = c.plan[kSC];
  const int Ks = dm.nq() / a.o_slices, hps = Ks / dm.hd, G = dm.group();
  const int nsplit = c.lw[layer].is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int tpo = 1;                                    // threads per output: a power of two
  while (tpo * 2 * Ks <= kDecThreads && tpo * 2 <= nsplit && tpo < 8) tpo *= 2;
  float* part = c.s.argbuf;                       // [tpo][Ks] partial o: tpo * Ks <= kDecThreads
  float* lsum = c.s.argbuf + kDecThreads;         // [hps] row sums over all splits (hps <= kDecThreads)
  for (int col = 0; col < a.ncols; ++col) {
    if (col > 0) dec_sync();
    for (int hh = warp; hh < hps; hh += kDecWarps) {
      int h = p.slice * hps + hh, kvh = h / G, g = h % G;
      const float* pl = a.part_ml + ((((size_t)col * dm.hkv + kvh) * nsplit) * G + g) * 2 + 1;
      float ls = 0.f;
      for (int sp = lane; sp < nsplit; sp += 32) ls += __ldcg(pl + (size_t)sp * G * 2);
      ls = warp_sum(ls);
      if (lane == 0) lsum[hh] = ls;
    }
    const int i = threadIdx.x % Ks, part_id = threadIdx.x / Ks;
    if (part_id < tpo && Ks <= kDecThreads) {
      int hh = i / dm.hd, e = i - hh * dm.hd;
      int h = p.slice * hps + hh, kvh = h / G, g = h % G;
      const size_t pi0 = (((size_t)col * dm.hkv + kvh) * nsplit) * G + g;
      const float* po = a.part_o + pi0 * dm.hd + e;
      const size_t stride = (size_t)G * dm.hd;
      const int per = (nsplit + tpo - 1) / tpo;
      const int s0 = part_id * per, s1 = min(nsplit, s0 + per);
      float acc = 0.f;
      int sp = s0;
      for (; sp + 16 <= s1; sp += 16) {
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = __ldcg(po + (size_t)(sp + u) * stride);
#pragma unroll
        for (int u = 0; u < 16; ++u) acc += v[u];
      }
      for (; sp + 4 <= s1; sp += 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = __ldcg(po + (size_t)(sp + u) * stride);
        acc += (v[0] + v[1]) + (v[2] + v[3]);
      }
      for (; sp < s1; ++sp) acc += __ldcg(po + (size_t)sp * stride);
      part[(size_t)part_id * Ks + i] = acc;
    }
    dec_sync();
    if (col == 0) B2_TP(2);
    for (int j = threadIdx.x; j < Ks; j += kDecThreads) {
      const int hh = j / dm.hd;
      float acc = 0.f;
      if (Ks <= kDecThreads) {
        for (int t = 0; t < tpo; ++t) acc += part[(size_t)t * Ks + j];
      } else {                                     // wide slices: one thread walks all splits of an output
        int e = j - hh * dm.hd;
        int h = p.slice * hps + hh, kvh = h / G, g = h % G;
        const size_t pi0 = (((size_t)col * dm.hkv + kvh) * nsplit) * G + g;
        for (int sp = 0; sp < nsplit; ++sp) acc += __ldcg(a.part_o + (pi0 + (size_t)sp * G) * dm.hd + e);
      }
      const float ls = lsum[hh];
      c.s.xf[(size_t)col * Ks + j] = ls > 0.f ? acc / ls : 0.f;
    }
    if (Ks <= kDecThreads) {
      // one output per thread: its value is still at hand for the maximum and the quantisation
      dec_sync();
      const bool mine = (int)threadIdx.x < Ks;
      const float val = mine ? c.s.xf[(size_t)col * Ks + threadIdx.x] : 0.f;
      const float m = block_max(fabsf(val), c.s.scratch);
      const float inv = m > 0.f ? 127.0f / m : 0.f;
      if (mine) quantize_value(val * inv, a.nterms, c.s.xq + (size_t)(col * a.nterms) * c.s.xstride + threadIdx.x, c.s.xstride);
      if (threadIdx.x == 0) c.s.colscale[col] = m > 0.f ? m / 127.0f : 0.f;
    }
  }
  dec_sync();
  B2_TP(7);
  if (Ks > kDecThreads) quantize_cols(c.s, Ks, a.ncols, a.nterms);
}

// One GEMV phase of the stream: for every round acquire / (prologue) / MMA / epilogue / release.
// Called from ONE place (the phase loop of the kernel), so its code exists once.
// Returns the staging half whose release is left to the grid barrier (null when it was released here).
__device__ __forceinline__ uint64_t* stream_gemv_phase(const DecodeArgs& a, StreamCtx& c, int ph, int layer, int cta,
                                                       float* best_val, int* best_idx, int bar) {
  const PhasePlan& p = c.plan[ph];
  const ModelDims& dm = a.dims;
  const int ncols = a.ncols, nterms = a.nterms;
  const int fills = p.rounds > 1 ? p.rounds : 1;
  float* y = ph == kSA ? a.qkv : ph == kSC ? a.opart : ph == kSD ? a.act : ph == kSE ? a.fpart : a.logits;
  for (int r = 0; r < fills; ++r) {
    unsigned char* hb;
    if (r == 0) B2_TP(0);
    const FillDesc* fd = stream_acquire(c, &hb, &a.st->err);
    if (r == 0) B2_TP(1);
    if (fd->ph != ph && threadIdx.x == 0) atomicExch(&a.st->err, (int)kDevBarrierTimeout);   // sequence out of step
    if (fd->valid && fd->ph == ph) {
      const int ntile = fd->ntile, ktn = fd->ktn, ta = fd->ta;
      const uint4* wsm = reinterpret_cast<const uint4*>(hb);
      const float* ssm = reinterpret_cast<const float*>(hb + (size_t)ntile * ktn * 512);
      const float* g_pre = ssm + ntile * 16;          // first pass of norm phases: g_pre then g_post
      const float* g_post = g_pre + dm.d;
      if (r == 0) {
        const LayerWeights& L = c.lw[layer];
        if (ph == kSA && layer == 0) {
          stream_prologue_embed(a, c, cta, a.xres[1], g_pre, L.gmax_pre_attn);
        } else if (ph == kSC) {
          stream_prologue_combine(a, c, layer, bar);
        } else if (ph == kSE) {
          stream_prologue_down(a, c, p.slice);
        } else {
          // A (layer > 0), D and H: residual update + two norms, one reduction
          const bool isD = ph == kSD;
          const float* parts = isD ? a.opart : a.fpart;
          const int nparts = isD ? a.o_slices : a.down_slices;
          const float* xin = isD ? a.xres[1] : a.xres[0];
          float* xout = isD ? a.xres[0] : a.xres[1];
          const float gmax = ph == kSH ? a.gmax_final : isD ? L.gmax_pre_ffn : L.gmax_pre_attn;
          stream_prologue_resid(a, c, cta, parts, nparts, xin, xout, g_post, g_pre, gmax, bar);
        }
        B2_TP(3);
      }
      QuantCols xc{c.s.xq, c.s.xstride, ncols * nterms};
      gemv_tiles_smem(wsm, ktn, ntile, xc, c.s.red);
      dec_sync();
      if (r == 0) B2_TP(4);
      if (p.epilogue == kEpiGeglu) {
        const int npair = ntile / 2;
        for (int col = 0; col < ncols; ++col)
        for (int i = threadIdx.x; i < npair * 16; i += kDecThreads) {
          int pr = i >> 4, row = i & 15;
          float gate = finalize_value(c.s, 2 * pr, row, col, nterms) * ssm[(2 * pr) * 16 + row];
          float up = finalize_value(c.s, 2 * pr + 1, row, col, nterms) * ssm[(2 * pr + 1) * 16 + row];
          y[(size_t)col * (p.N / 2) + (size_t)(ta / 2 + pr) * 16 + row] = gelu_tanh(gate) * up;
          for (int t = 0; t < nterms; ++t) {           // leave the accumulators clean for the next round
            c.s.red[((2 * pr) * 16 + row) * kQCols + col * nterms + t] = 0;
            c.s.red[((2 * pr + 1) * 16 + row) * kQCols + col * nterms + t] = 0;
          }
        }
      } else {
        for (int col = 0; col < ncols; ++col)
        for (int i = threadIdx.x; i < ntile * 16; i += kDecThreads) {
          int un = i >> 4, row = i & 15;
          int n = (ta + un) * 16 + row;
          float v = finalize_value(c.s, un, row, col, nterms) * ssm[un * 16 + row];
          y[((size_t)p.slice * ncols + col) * p.N + n] = v;
          for (int t = 0; t < nterms; ++t) c.s.red[(un * 16 + row) * kQCols + col * nterms + t] = 0;
          if (p.epilogue == kEpiHead && col < kMaxCols) {
            if (v > best_val[col] || (v == best_val[col] && n < best_idx[col])) { best_val[col] = v; best_idx[col] = n; }
          }
        }
      }
    }
    if (r == fills - 1 && ph != kSH) {
      if (r == 0) B2_TP(5);
      B2_TP(6);
      return stream_release_deferred(c);       // the grid barrier follows immediately
    }
    stream_release(c);
    if (r == 0) B2_TP(5);
  }
  B2_TP(6);
  return nullptr;
}

// The kernel is instantiated per cache type / head_dim / GQA group, so the loop
// over phases carries exactly one attention variant and one GEMV phase body:
// every phase's code runs once per layer, and a small loop body stays in the
// instruction cache.
template <typename T, int HD, int G>
__global__ void __launch_bounds__(kStreamThreads, 1)
decode_stream_kernel(const __grid_constant__ DecodeArgs a, int nsteps, unsigned int epoch0, int half_bytes) {
  extern __shared__ __align__(128) unsigned char ssm_raw[];
  __shared__ unsigned int epoch;
  StreamCtx c;
  stream_carve(ssm_raw, a.dims, a.ncols, half_bytes, c);
  const int cta = blockIdx.x, ncta = gridDim.x;
  const ModelDims& dm = a.dims;
  if (threadIdx.x == 0) {
    epoch = epoch0;
    for (int i = 0; i < 2; ++i) { mbar_init(&c.full[i], 1); mbar_init(&c.empty[i], 1); }
    mbar_init(c.aux, 1);
    *c.step_ready = 1;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = threadIdx.x; i < dm.n_layers; i += kStreamThreads) {
    c.lw[i] = a.layers[i];
    c.lkv[i] = a.kv[i];
  }
  for (int i = threadIdx.x; i < kMaxRoundUnits * 16 * kQCols; i += kStreamThreads) c.s.red[i] = 0;
  constexpr int esz_kv = (int)sizeof(T);
  c.npre_max = min(kStreamMaxStagedRows, (half_bytes - 3 * HD * 4) / (2 * HD * esz_kv));
  c.wait_no = 0;
  c.aux_cnt = 0;
  __syncthreads();
  if (threadIdx.x == 0) stream_make_plans(a, c, cta, ncta);
  __syncthreads();

  if (threadIdx.x >= kDecThreads) {       // ---- producer warp
    stream_producer(a, c, cta, nsteps);
    return;
  }

  int bar = 0;
  const int n_phases = 5 * dm.n_layers + 1;
  for (int step = 0; step < nsteps; ++step) {
    if (threadIdx.x == 0) *c.step_ready = step + 1;
    float bv[kMaxCols];
    int bi[kMaxCols];
#pragma unroll
    for (int cc = 0; cc < kMaxCols; ++cc) { bv[cc] = -INFINITY; bi[cc] = 0x7fffffff; }
#pragma unroll 1
    for (int pi = 0; pi < n_phases; ++pi) {
      uint64_t* release = nullptr;                   // staging half handed back inside the grid barrier
      int layer = pi / 5, ph = pi - layer * 5;       // A, B, C, D, E of each layer ...
      if (pi == n_phases - 1) { layer = dm.n_layers - 1; ph = kSH; }   // ... then the head
      if (ph == kSB) {
        // ---- attention (K/V rows and the RoPE row staged by the producer)
        const LayerWeights& L = c.lw[layer];
        unsigned char* hb;
        B2_TP(0);
        const FillDesc* fd = stream_acquire(c, &hb, &a.st->err);
        B2_TP(1);
        if (fd->ph != kSB && threadIdx.x == 0) atomicExch(&a.st->err, (int)kDevBarrierTimeout);
        const int is_global = L.is_global;
        const int nsplit = is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
        const int items = a.ncols * dm.hkv * nsplit;
        const size_t rowb = (size_t)HD * esz_kv;
        for (int itx = cta; itx < items; itx += ncta) {
          AttnItem it;
          it.layer = layer;
          it.split = itx % nsplit;
          int rest = itx / nsplit;
          it.kvh = rest % dm.hkv;
          it.col = rest / dm.hkv;
          it.nsplit = nsplit;
          it.is_global = is_global;
          it.bar = bar;
          if (itx == cta && fd->valid && fd->ph == kSB) {
            it.nstaged = fd->npre;
            it.pos = fd->pos;
            it.cos_r = reinterpret_cast<const float*>(hb + (size_t)2 * c.npre_max * rowb);
            it.sin_r = it.cos_r + HD / 2;
            it.g_q = it.sin_r + HD / 2;
            it.g_k = it.g_q + HD;
          } else {            // further items of this CTA: rows fetched on the spot
            int pos = __ldcg(&a.st->pos[it.col]);
            if (pos < 0 || pos >= dm.max_ctx) {
              if (threadIdx.x == 0) atomicExch(&a.st->err, (int)kDevBadPosition);
              pos = 0;
            }
            it.pos = pos;
            it.nstaged = -1;
            it.cos_r = a.rope_cos[is_global ? 1 : 0] + (size_t)pos * (HD / 2);
            it.sin_r = a.rope_sin[is_global ? 1 : 0] + (size_t)pos * (HD / 2);
            it.g_q = L.g_q;
            it.g_k = L.g_k;
          }
          attn_smem_item<T, HD, G>(a, c, it, hb);
        }
        B2_TP(4);
        release = stream_release_deferred(c);
      } else {
        release = stream_gemv_phase(a, c, ph, layer, cta, bv, bi, bar);
      }
      if (ph == kSH) {       // CTA-level arg-max (lowest index wins ties), one slot per CTA
        float* sv = c.s.argbuf;
        int* si = reinterpret_cast<int*>(c.s.argbuf + kDecThreads);
        for (int col = 0; col < a.ncols; ++col) {
          dec_sync();
          sv[threadIdx.x] = bv[col];
          si[threadIdx.x] = bi[col];
          dec_sync();
          for (int stp = kDecThreads / 2; stp > 0; stp >>= 1) {
            if (threadIdx.x < stp) {
              float ov = sv[threadIdx.x + stp];
              int oi = si[threadIdx.x + stp];
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
      stream_grid_barrier(a.st, &epoch, ncta, release, a.trace, bar++);
    }
    if (cta == 0) phase_argmax(a, ncta);
    grid_barrier(a.st, &epoch, ncta, a.trace, bar++);
  }
}

// Host-side selection of the instantiation for a model.
inline const void* decode_stream_kernel_for(const ModelDims& d) {
  const int G = d.hq / d.hkv;
#define B2_PICK_G(T, HD)                                                                  \
  (G == 1 ? (const void*)decode_stream_kernel<T, HD, 1>                                   \
          : G == 2 ? (const void*)decode_stream_kernel<T, HD, 2> : (const void*)decode_stream_kernel<T, HD, 4>)
#define B2_PICK_HD(T)                                                                     \
  (d.hd == 32 ? B2_PICK_G(T, 32) : d.hd == 64 ? B2_PICK_G(T, 64) : d.hd == 128 ? B2_PICK_G(T, 128) : B2_PICK_G(T, 256))
  return d.kv_dtype == 0 ? B2_PICK_HD(float) : B2_PICK_HD(__nv_bfloat16);
#undef B2_PICK_HD
#undef B2_PICK_G
}

}  // namespace b200lm

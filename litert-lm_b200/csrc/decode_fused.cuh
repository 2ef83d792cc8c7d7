// Chained persistent decode kernel: no grid barriers.
//
// One cooperative launch runs one or more decode steps on every SM (16 compute
// warps + 1 copy-producer warp per CTA).  A step is a chain of dependent phases
// per layer -- A qkv, B attention, C o-proj, DE gate/up + GeGLU + down, R
// reduce -- then H, the LM head with its arg-max.  What distinguishes it from
// the barrier-per-phase kernels (decode_ops.cuh, decode_stream.cuh):
//
//  * Phases hand their results over in FLAG-CARRYING WORDS: every value is an
//    8-byte store of (fp32 bits, tag), the tag naming the (step, layer) that
//    produced it.  A consumer polls the words it needs and proceeds as soon as
//    their tags match, so "wait for the producers" and "fetch their output"
//    are ONE L2 round trip; there is no grid-wide barrier anywhere.  Buffers
//    alternate between two copies by layer parity, and every poll is bounded.
//  * Gate/up, GeGLU and the down projection are one phase: a CTA owns 64*m ffn
//    features, computes their activations and multiplies them by its K slice of
//    W_down at once; the partial d-vectors are summed by reducer CTAs in a fixed
//    order (deterministic fp32) and published once.
//  * The residual stream lives in every CTA's shared memory (all CTAs apply both
//    updates of a layer), so it never travels.
//  * Weights, scales, gains, cached K/V rows and the RoPE row arrive by 1-D bulk
//    async copies into a ring of equal slots, issued by the producer warp as far
//    ahead as the ring allows; both sides derive the same static fill sequence,
//    so no descriptors are exchanged.  In the head phase each warp consumes whole
//    slots (one 16-row tile each) on its own, without block-wide barriers.
//  * int4 x int8 tiles run on mma.sync m16n8k32; the quantised activations are
//    stored permuted so that one 16-byte shared-memory load yields a lane's four
//    B words of a 64-wide k tile.
#pragma once
#include "common.cuh"
#include "decode_ops.cuh"
#include "prefill_ops.cuh"
#include "decode_stream.cuh"

namespace b200lm {

constexpr int kFuThreads = kDecThreads + 32;   // 16 compute warps + 1 producer warp
constexpr int kFuMaxSlots = 32;
constexpr int kFuMaxV4 = 3;                    // float4 of the residual per thread (d <= 6144)
constexpr long kFuSpinLimit = 1L << 21;        // polls of ~0.5 us each: about a second

typedef unsigned long long fu_u64;

// Geometry of the chain for one model / session count; computed on the host, the same for all CTAs.
struct FusedPlan {
  int slot_bytes, nslots;
  int xstride;              // bytes between rows of the quantised activations (== 64 mod 128)
  int a_per;                // qkv row tiles per working CTA
  int c_cps, c_per, c_tps;  // o-proj: CTAs per K slice, row tiles per working CTA, row tiles per slot
  int ffn_m, nprod;         // down-projection k tiles (64 features) per FFN CTA, FFN CTAs
  int d_tps;                // down-projection row tiles per slot
  int r_per, nred;          // elements of d per reducer CTA, reducer CTAs
  int kps;                  // cached keys (K row + V row) per slot
  int round_fills;          // fills a phase keeps resident at once
  int part_stride;          // 8-byte words per attention partial (G*hd outputs + G row sums, even)
  int max_items;            // attention work items (sessions * kv heads * splits) at most
  int ll_qkv, ll_part, ll_o, ll_fpart, ll_f, ll_amax;   // offsets (8-byte words) of ONE parity copy in the exchange area
  int ll_words;             // words of one parity copy
  unsigned tag0;            // tag of (step 0, layer 0) of this launch is tag0 + 1
};

__host__ __device__ inline int fu_round_up(int v, int a) { return (v + a - 1) / a * a; }
__host__ __device__ inline int fu_pow2_floor(int v) { int p = 1; while (p * 2 <= v) p *= 2; return p; }
__host__ __device__ inline int fu_log2(int v) { int l = 0; while ((1 << (l + 1)) <= v) ++l; return l; }

// ------------------------------------------------------------ flag-carrying words

__device__ __forceinline__ void ll_store(fu_u64* p, float v, unsigned tag) {
  fu_u64 w = ((fu_u64)tag << 32) | (fu_u64)__float_as_uint(v);
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_store_bits(fu_u64* p, unsigned bits, unsigned tag) {
  fu_u64 w = ((fu_u64)tag << 32) | (fu_u64)bits;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_load2(const fu_u64* p, fu_u64& a, fu_u64& b) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ fu_u64 ll_load1(const fu_u64* p) {
  fu_u64 a;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(a) : "l"(p) : "memory");
  return a;
}
__device__ __forceinline__ float ll_val(fu_u64 w) { return __uint_as_float((unsigned)w); }
__device__ __forceinline__ bool ll_ok(fu_u64 w, unsigned tag) { return (unsigned)(w >> 32) == tag; }

// ------------------------------------------------------------------ CTA context

// One copy per CTA, in SHARED memory: every field is uniform over the CTA, and a context in registers
// would be spilled to local memory by the out-of-line phase functions (local memory has almost no L1
// left beside a 227 KiB shared-memory carve-out, so each access would be an L2 round trip).
struct FusedCtx {
  unsigned char* ring;
  uint64_t* full;            // [nslots]
  uint64_t* empty;           // [nslots]
  volatile int* dead;        // a bounded wait gave up: every later wait returns at once
  volatile int* step_ready;  // steps whose cache rows may be fetched (producer gate)
  int* pos0;                 // [kMaxCols] position of step 0
  int* tok;                  // [kMaxCols] token of the current step
  float* xres;               // [ncols][d] residual stream
  int8_t* xq;                // [ncols*nterms][xstride] quantised activations, k-permuted per 64
  int* red;                  // [16][16][8] accumulator fragments
  float* scratch;            // [128]
  float* colscale;           // [kMaxCols]
  float* gu;                 // [8m][16][ncols] gate / up values of this CTA's features
  float* act;                // [ncols][64m]; also the combine's staging [ncols][Ks]
  float* attn;               // q_s [G][hd], k_s [hd], v_s [hd], probabilities, key-part reduction
  LayerWeights* lw;
  LayerKv* lkv;
  ChainedLayer* cl;
  int slot_bytes, nslots, nslots_log2, xstride;
  float* fpart;              // [16 warps][16] partial outputs of a GEMV whose k range is split over warps
  int* err;
  fu_u64* ll_base;           // exchange area (two parity copies)
  int* gave_up;              // DecodeState::gave_up
  int* progress;             // DecodeArgs::progress
  long long* fill_log;       // development timeline of CTA 0: per fill (issue, wait start, wait end) in SM clocks, or null
  int where;                 // phase code * 1000 + layer, for the report of a wait that gave up
};

__host__ __device__ inline size_t fu_attn_floats(const ModelDims& d, const FusedPlan& pl) {
  const int G = d.hq / d.hkv;
  const int maxkeys = pl.round_fills * pl.kps + 1;
  return (size_t)(G + 2) * d.hd + (size_t)G * maxkeys + 4 * G + (size_t)kDecThreads * G + (size_t)(kDecThreads / d.hd + 1) * G + 64;
}

__host__ __device__ inline size_t fu_fixed_bytes(const ModelDims& d, int ncols, int nterms, const FusedPlan& pl) {
  size_t b = 0;
  b += 2 * (size_t)kFuMaxSlots * 8 + 128;                              // mbarriers, flags, pos0, tok
  b += (size_t)ncols * d.d * 4;                                        // xres
  b += (size_t)ncols * nterms * pl.xstride + 128;                      // xq
  b += (size_t)16 * 16 * kQCols * 4 + 16 * 16 * 4;                     // red, fpart
  b += 128 * 4 + kMaxCols * 4 + 64;                                    // scratch, colscale
  b += (size_t)8 * pl.ffn_m * 16 * ncols * 4;                          // gu
  size_t act = (size_t)ncols * 64 * pl.ffn_m * 4;
  size_t comb = (size_t)ncols * 512 * 4 + 512 * 4 * 4;                 // combine staging (Ks <= 512) + partial sums
  b += (act > comb ? act : comb) + 64;
  b += fu_attn_floats(d, pl) * 4 + 64;
  b += (size_t)d.n_layers * (sizeof(LayerWeights) + sizeof(LayerKv) + sizeof(ChainedLayer)) + 64;
  return b + 512;                                                      // alignment slack
}

__device__ __forceinline__ void fu_carve(unsigned char* base, const ModelDims& d, int ncols, int nterms, const FusedPlan& pl,
                                         FusedCtx& c) {
  unsigned char* p = reinterpret_cast<unsigned char*>(((uintptr_t)base + 127) & ~(uintptr_t)127);
  c.ring = p; p += (size_t)pl.nslots * pl.slot_bytes;
  c.full = reinterpret_cast<uint64_t*>(p); p += (size_t)kFuMaxSlots * 8;
  c.empty = reinterpret_cast<uint64_t*>(p); p += (size_t)kFuMaxSlots * 8;
  c.dead = reinterpret_cast<volatile int*>(p);
  c.step_ready = reinterpret_cast<volatile int*>(p + 4);
  c.pos0 = reinterpret_cast<int*>(p + 16);
  c.tok = reinterpret_cast<int*>(p + 16 + kMaxCols * 4);
  p += 128;
  c.xres = reinterpret_cast<float*>(p); p += (size_t)ncols * d.d * 4;
  p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 127) & ~(uintptr_t)127);
  c.xq = reinterpret_cast<int8_t*>(p); p += (size_t)ncols * nterms * pl.xstride;
  p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 15) & ~(uintptr_t)15);
  c.red = reinterpret_cast<int*>(p); p += (size_t)16 * 16 * kQCols * 4;
  c.fpart = reinterpret_cast<float*>(p); p += 16 * 16 * 4;
  c.scratch = reinterpret_cast<float*>(p); p += 128 * 4;
  c.colscale = reinterpret_cast<float*>(p); p += kMaxCols * 4;
  p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 15) & ~(uintptr_t)15);
  c.gu = reinterpret_cast<float*>(p); p += (size_t)8 * pl.ffn_m * 16 * ncols * 4;
  c.act = reinterpret_cast<float*>(p);
  {
    size_t act = (size_t)ncols * 64 * pl.ffn_m * 4;
    size_t comb = (size_t)ncols * 512 * 4 + 512 * 4 * 4;
    p += act > comb ? act : comb;
  }
  p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 15) & ~(uintptr_t)15);
  c.attn = reinterpret_cast<float*>(p); p += fu_attn_floats(d, pl) * 4;
  p = reinterpret_cast<unsigned char*>(((uintptr_t)p + 15) & ~(uintptr_t)15);
  c.lw = reinterpret_cast<LayerWeights*>(p); p += (size_t)d.n_layers * sizeof(LayerWeights);
  c.lkv = reinterpret_cast<LayerKv*>(p); p += (size_t)d.n_layers * sizeof(LayerKv);
  c.cl = reinterpret_cast<ChainedLayer*>(p);
  c.slot_bytes = pl.slot_bytes;
  c.nslots = pl.nslots;
  c.nslots_log2 = fu_log2(pl.nslots);
  c.xstride = pl.xstride;
}

// ------------------------------------------------------------------ host-side plan

// Fills `pl` for a model; returns false when the model does not fit this kernel (the caller then
// uses the barrier-per-phase kernels).  `smem_optin` is the device's opt-in shared memory per block.
__host__ inline bool fused_make_plan(const ModelDims& d, int ncols, int nterms, int ncta, int o_slices, int nsplit_local,
                                     int nsplit_global, size_t smem_optin, FusedPlan* out, size_t* smem_bytes) {
  FusedPlan pl{};
  const int G = d.hq / d.hkv;
  if (d.d % 64 || d.ffn % 64 || d.nq() % 64 || d.nqkv() % 16 || d.vocab % 16) return false;
  if (d.d / 4 > kFuMaxV4 * kDecThreads) return false;
  if (ncols * nterms > kQCols || ncols > kMaxCols) return false;
  if (G != 1 && G != 2 && G != 4) return false;
  if (d.hd != 32 && d.hd != 64 && d.hd != 128 && d.hd != 256) return false;
  const int esz = d.kv_dtype == 0 ? 4 : 2;
  const int ktn = d.d / 64;
  pl.slot_bytes = fu_round_up(ktn * 512 + 64, 128);
  if (pl.slot_bytes < 2 * d.d * 4) pl.slot_bytes = fu_round_up(2 * d.d * 4, 128);              // two gain vectors
  if (pl.slot_bytes < 2 * d.hd * esz) pl.slot_bytes = fu_round_up(2 * d.hd * esz, 128);        // one cached key
  if (pl.slot_bytes < 3 * d.hd * 4) pl.slot_bytes = fu_round_up(3 * d.hd * 4, 128);            // RoPE row + QK gains
  const int ntA = d.nqkv() / 16;
  pl.a_per = (ntA + ncta - 1) / ncta;
  // o-proj: K split by head slices (o_slices), row tiles over the CTAs of a slice
  const int Ks = d.nq() / o_slices;
  if (Ks % 64 || Ks > 512) return false;
  pl.c_cps = ncta / o_slices;
  if (pl.c_cps < 1) return false;
  pl.c_per = (d.d / 16 + pl.c_cps - 1) / pl.c_cps;
  pl.c_tps = pl.slot_bytes / ((Ks / 64) * 512 + 64);
  if (pl.c_tps < 1) return false;
  pl.c_tps = fu_pow2_floor(pl.c_tps);          // tiles-per-slot counts and the slot count are powers of two:
  if (pl.c_tps > 64) pl.c_tps = 64;            // the kernel locates tiles and slots with shifts, not divisions
  // ffn: 64*m features per producer CTA
  const int KTd = d.ffn / 64;
  pl.ffn_m = (KTd + ncta - 1) / ncta;
  pl.nprod = (KTd + pl.ffn_m - 1) / pl.ffn_m;
  pl.d_tps = pl.slot_bytes / (pl.ffn_m * 512 + 64);     // row tiles of the K slice with their 16 scales each
  if (pl.d_tps < 1) return false;
  pl.d_tps = fu_pow2_floor(pl.d_tps);
  if (pl.d_tps > 64) pl.d_tps = 64;
  pl.r_per = fu_round_up((d.d + ncta - 1) / ncta, 4);
  pl.nred = (d.d + pl.r_per - 1) / pl.r_per;
  pl.kps = fu_pow2_floor(pl.slot_bytes / (2 * d.hd * esz));
  if (pl.kps > 64) pl.kps = 64;
  pl.part_stride = G * d.hd + fu_round_up(G, 2);
  const int max_split = nsplit_local > nsplit_global ? nsplit_local : nsplit_global;
  pl.max_items = ncols * d.hkv * max_split;
  if (pl.max_items > ncta) return false;
  // widest activation vector that is quantised
  int kmax = d.d;
  if (64 * pl.ffn_m > kmax) kmax = 64 * pl.ffn_m;
  if (Ks > kmax) kmax = Ks;
  pl.xstride = fu_round_up(kmax, 128) + 64;
  // ring: what the fixed part leaves; a phase keeps at most round_fills slots at once
  pl.round_fills = 8;
  size_t fixed = 0;
  for (int pass = 0; pass < 2; ++pass) {
    fixed = fu_fixed_bytes(d, ncols, nterms, pl);
    if (fixed + 6 * (size_t)pl.slot_bytes > smem_optin) return false;
    pl.nslots = (int)((smem_optin - fixed) / pl.slot_bytes);
    if (pl.nslots > kFuMaxSlots) pl.nslots = kFuMaxSlots;
    pl.nslots = fu_pow2_floor(pl.nslots);
    int rf = pl.nslots - 2;
    if (rf > 16) rf = 16;
    if (rf == pl.round_fills) break;
    pl.round_fills = rf;
  }
  if (pl.nslots < 8 || pl.round_fills + 2 > pl.nslots) return false;
  // exchange area (8-byte words per parity copy)
  int off = 0;
  pl.ll_qkv = off; off += fu_round_up(ncols * d.nqkv(), 2);
  pl.ll_part = off; off += pl.max_items * pl.part_stride;
  pl.ll_o = off; off += o_slices * ncols * d.d;
  pl.ll_fpart = off; off += pl.nprod * ncols * d.d;
  pl.ll_f = off; off += ncols * d.d;
  pl.ll_amax = off; off += fu_round_up(2 * ncta * ncols, 2);
  pl.ll_words = fu_round_up(off, 2);
  *out = pl;
  *smem_bytes = fixed + (size_t)pl.nslots * pl.slot_bytes;
  return true;
}

// ------------------------------------------------------------------ slot helpers

// The fields of the context that the ring helpers need, read ONCE per phase function into registers:
// reading them from the shared-memory context at every use would chain several dependent shared-memory
// loads in front of each barrier test.  nslots is a power of two: slot = fill & mask, phase parity =
// bit log2(nslots) of the fill number.
struct FusedRing {
  unsigned char* ring;
  uint64_t* full;
  uint64_t* empty;
  int slot_bytes;
  unsigned mask;
  int log2;
};
__device__ __forceinline__ FusedRing fu_ring(const FusedCtx& c) {
  return FusedRing{c.ring, c.full, c.empty, c.slot_bytes, (unsigned)(c.nslots - 1), c.nslots_log2};
}
__device__ __forceinline__ unsigned char* fu_slot(const FusedRing& r, unsigned fill) {
  return r.ring + (size_t)(fill & r.mask) * r.slot_bytes;
}
// Records the first wait that gave up (kind 1: a poll of flag-carrying words, 2: a ring slot that never
// filled, 3: the producer waiting for a free slot or for the previous step).
__device__ __noinline__ void fu_gave_up(FusedCtx& c, int kind) {
  if (atomicCAS(c.gave_up + 3, 0, kind) == 0) {
    c.gave_up[0] = c.where / 1000;
    c.gave_up[1] = c.where % 1000;
    c.gave_up[2] = blockIdx.x;
    // where every CTA stood at that moment (the second half of the progress array): after a first
    // give-up the CTAs stop waiting and run through, so the live words say nothing any more
    volatile int* pr = c.progress;
    for (unsigned i = 0; i < gridDim.x; ++i) pr[gridDim.x + i] = pr[i];
  }
  *c.dead = 1;
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.b32 %0, 1, 0, p;\n}"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// The slot has not filled yet: bounded wait, with the development log of CTA 0.
__device__ __noinline__ void fu_acquire_slow(FusedCtx& c, unsigned fill) {
  if (*c.dead) return;
  const unsigned s = fill & (unsigned)(c.nslots - 1), par = (fill >> c.nslots_log2) & 1u;
  const bool log = c.fill_log && (threadIdx.x & 31) == 0 && fill < 4000u;
  if (log) c.fill_log[3 * fill + 1] = clock64();
  if (!mbar_wait(&c.full[s], par, c.err)) fu_gave_up(c, 2);
  if (log) c.fill_log[3 * fill + 2] = clock64();
}
// Weights are normally staged long before their phase: one non-blocking test, the slow path only if it fails.
__device__ __forceinline__ void fu_acquire(const FusedRing& r, FusedCtx& c, unsigned fill) {
  if (mbar_test(&r.full[fill & r.mask], (fill >> r.log2) & 1u)) return;
  fu_acquire_slow(c, fill);
}
// All compute threads are done with fills [f0, f0 + n): one block barrier, then one arrive per slot.
__device__ __forceinline__ void fu_release(const FusedRing& r, unsigned f0, int n) {
  dec_sync();
  if ((int)threadIdx.x < n) mbar_arrive(&r.empty[(f0 + threadIdx.x) & r.mask]);
}

// ------------------------------------------------------------------ bounded polls

__device__ __forceinline__ bool fu_spin_check(FusedCtx& c, long& spins) {
  ++spins;
  if ((spins & 63) == 0 && *c.dead) return false;
  if (spins > kFuSpinLimit) {
    atomicExch(c.err, (int)kDevBarrierTimeout);
    fu_gave_up(c, 1);
    return false;
  }
  return true;
}

// Two values at p (16-byte aligned) once both carry `tag`.
__device__ __forceinline__ float2 ll_wait2(FusedCtx& c, const fu_u64* p, unsigned tag) {
  fu_u64 w0 = 0, w1 = 0;
  long spins = 0;
  while (true) {
    ll_load2(p, w0, w1);
    if (ll_ok(w0, tag) && ll_ok(w1, tag)) break;
    if (!fu_spin_check(c, spins)) break;
  }
  return make_float2(ll_val(w0), ll_val(w1));
}
__device__ __forceinline__ fu_u64 ll_wait1(FusedCtx& c, const fu_u64* p, unsigned tag) {
  fu_u64 w = 0;
  {
    long spins = 0;
    while (true) {
      w = ll_load1(p);
      if (ll_ok(w, tag)) break;
      if (!fu_spin_check(c, spins)) break;
    }
  }
  return w;
}
// Four values at p (32-byte aligned): both 16-byte loads are in flight together.
__device__ __forceinline__ float4 ll_wait4(FusedCtx& c, const fu_u64* p, unsigned tag) {
  fu_u64 w0 = 0, w1 = 0, w2 = 0, w3 = 0;
  {
    long spins = 0;
    while (true) {
      ll_load2(p, w0, w1);
      ll_load2(p + 2, w2, w3);
      if (ll_ok(w0, tag) && ll_ok(w1, tag) && ll_ok(w2, tag) && ll_ok(w3, tag)) break;
      if (!fu_spin_check(c, spins)) break;
    }
  }
  return make_float4(ll_val(w0), ll_val(w1), ll_val(w2), ll_val(w3));
}

// ------------------------------------------------------------------ quantisation

// Byte offset of element k in a k-permuted row: inside each 64-wide k tile, lane t of an MMA quad finds
// its words for k = 4t, 16+4t, 32+4t, 48+4t next to each other (one 16-byte load).
__device__ __forceinline__ int fu_perm(int k) {
  const int kk = k & 63;
  return (k & ~63) + ((kk >> 2) & 3) * 16 + (kk >> 4) * 4 + (kk & 3);
}

// Four consecutive values (k multiple of 4), already scaled into [-127, 127], into nterms int8 terms
// (x = t0 + t1 / 128 + t2 / 16384 up to 2^-15): the residuals never exceed 64 in magnitude, so nothing clamps.
__device__ __forceinline__ void fu_quantize4(float4 r, int nterms, int8_t* row0, int k, int stride) {
  float v[4] = {r.x, r.y, r.z, r.w};
  uint32_t w0 = 0, w1 = 0, w2 = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float t0 = rintf(v[i]);
    const float r1 = (v[i] - t0) * 128.0f;
    const float t1 = rintf(r1);
    const float t2 = rintf((r1 - t1) * 128.0f);
    w0 |= ((uint32_t)(int)t0 & 0xFFu) << (8 * i);
    w1 |= ((uint32_t)(int)t1 & 0xFFu) << (8 * i);
    w2 |= ((uint32_t)(int)t2 & 0xFFu) << (8 * i);
  }
  int8_t* q = row0 + fu_perm(k);
  *reinterpret_cast<uint32_t*>(q) = w0;
  if (nterms > 1) *reinterpret_cast<uint32_t*>(q + stride) = w1;
  if (nterms > 2) *reinterpret_cast<uint32_t*>(q + 2 * stride) = w2;
}

// ------------------------------------------------------------------ int4 x int8 tiles

// mma.sync m16n8k32 s8 x s8 -> s32 as a pure function of its operands (no volatile: the compiler may
// interleave the chains of several tiles).
__device__ __forceinline__ void fu_mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void fu_mma_tile(int (&acc)[4], const uint4& w, const uint4& b) {
  const uint32_t m = 0xF0F0F0F0u;   // high nibble of every byte = 16 * q as int8
  fu_mma_s8(acc, (w.x << 4) & m, w.x & m, (w.y << 4) & m, w.y & m, b.x, b.y);
  fu_mma_s8(acc, (w.z << 4) & m, w.z & m, (w.w << 4) & m, w.w & m, b.z, b.w);
}

// Tile blocks [kt0, kt1) of one 16-row tile (block kt at wt + kt * kstride) against the quantised columns.
// Two accumulator chains (even / odd k tiles) hide the MMA latency.
__device__ __forceinline__ int4 fu_mma_run(const uint4* wt, int kstride, int kt0, int kt1, const int8_t* xq, int xstride, int nq,
                                        int lane) {
  const int g = lane >> 2, t = lane & 3;
  const bool ok = g < nq;
  const uint4* bp = reinterpret_cast<const uint4*>(xq + (size_t)(ok ? g : 0) * xstride + t * 16);
  int a0[4] = {0, 0, 0, 0}, a1[4] = {0, 0, 0, 0};
  const uint4 zero = make_uint4(0, 0, 0, 0);
  int kt = kt0;
  for (; kt + 1 < kt1; kt += 2) {
    const uint4 w0 = wt[(size_t)kt * kstride + lane], w1 = wt[(size_t)(kt + 1) * kstride + lane];
    const uint4 b0 = ok ? bp[kt * 4] : zero, b1 = ok ? bp[(kt + 1) * 4] : zero;
    fu_mma_tile(a0, w0, b0);
    fu_mma_tile(a1, w1, b1);
  }
  if (kt < kt1) {
    const uint4 w0 = wt[(size_t)kt * kstride + lane];
    const uint4 b0 = ok ? bp[kt * 4] : zero;
    fu_mma_tile(a0, w0, b0);
  }
  return make_int4(a0[0] + a1[0], a0[1] + a1[1], a0[2] + a1[2], a0[3] + a1[3]);
}

// Accumulator fragment of a warp into red[slot][16][kQCols].
__device__ __forceinline__ void fu_store_frag(int* red, int slot, int4 acc, int lane) {
  const int g = lane >> 2, t = lane & 3;
  int* base = red + slot * 16 * kQCols;
  *reinterpret_cast<int2*>(base + g * kQCols + 2 * t) = make_int2(acc.x, acc.y);
  *reinterpret_cast<int2*>(base + (g + 8) * kQCols + 2 * t) = make_int2(acc.z, acc.w);
}
// Value of (row, col) summed over `parts` consecutive fragments starting at `slot`.
__device__ __forceinline__ float fu_finalize(const int* red, int slot, int parts, int row, int col, int nterms, float colscale) {
  int s0 = 0, s1 = 0, s2 = 0;
  for (int p = 0; p < parts; ++p) {
    const int* r = red + ((slot + p) * 16 + row) * kQCols + col * nterms;
    s0 += r[0];
    if (nterms > 1) s1 += r[1];
    if (nterms > 2) s2 += r[2];
  }
  float v = (float)s0;
  if (nterms > 1) v += (float)s1 * (1.0f / 128.0f);
  if (nterms > 2) v += (float)s2 * (1.0f / 16384.0f);
  return v * (colscale * (1.0f / 16.0f));      // weights entered the MMA as 16 * q
}


// Where the outputs of a GEMV round go: flag-carrying words in the exchange area (out) or plain floats
// in shared memory (out_f); element (tile, row, col) lands at col * ld + row0 + tile * 16 + row.
struct FusedOut {
  fu_u64* out;
  float* out_f;
  int ld, row0;
  unsigned tag;
};

// One round of a GEMV phase over resident fills [fill0, fill0 + nfills): `ntiles` row tiles of `ktn` k
// tiles each, `tpf` tiles per fill (tile j of a fill at j * ktn * 512 bytes; with kmajor, k tile kk of tile j
// at (kk * tiles_in_fill + j) * 512).  scales == nullptr: the 16 scales of each tile follow the tiles of its
// fill; else scales[tile * 16 + row], tile counted from the start of the round.  With fewer than nine tiles
// the k range of a tile is split over several warps (latency), else a warp owns whole tiles and finalises
// them on its own (throughput).  The caller acquires before and releases after.  One copy of this code
// serves every GEMV phase: the step's instruction footprint matters more than a specialised inner loop.
__device__ __noinline__ void fu_gemv_round(FusedCtx& c, unsigned fill0, int tpf, int ntiles, int ktn, const float* scales,
                                           bool kmajor, int ncols, int nterms, FusedOut o) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const FusedRing rg = fu_ring(c);
  const int nq = ncols * nterms;
  int kw = 1;
  while (kw * 2 * ntiles <= kDecWarps && kw * 2 <= ktn) kw *= 2;
  const size_t tile_bytes = (size_t)ktn * 512;
  if (kw == 1) {
    for (int tile = warp; tile < ntiles; tile += kDecWarps) {
      const int f = tile / tpf, j = tile - f * tpf;
      const int in_fill = min(tpf, ntiles - f * tpf);
      const unsigned char* base = fu_slot(rg, fill0 + f);
      const int4 acc = fu_mma_run(reinterpret_cast<const uint4*>(base + (kmajor ? (size_t)j * 512 : (size_t)j * tile_bytes)),
                                  kmajor ? in_fill * 32 : 32, 0, ktn, c.xq, c.xstride, nq, lane);
      fu_store_frag(c.red, warp, acc, lane);
      __syncwarp();
      const float* sc = scales ? scales + tile * 16 : reinterpret_cast<const float*>(base + (size_t)in_fill * tile_bytes) + j * 16;
      for (int i = lane; i < 16 * ncols; i += 32) {
        const int row = i & 15, col = i >> 4;
        const float v = fu_finalize(c.red, warp, 1, row, col, nterms, c.colscale[col]) * sc[row];
        const size_t idx = (size_t)col * o.ld + o.row0 + tile * 16 + row;
        if (o.out_f) o.out_f[idx] = v;
        else ll_store(o.out + idx, v, o.tag);
      }
      __syncwarp();
    }
  } else {
    if (warp < ntiles * kw) {
      const int tile = warp / kw, part = warp - tile * kw;
      const int f = tile / tpf, j = tile - f * tpf;
      const int in_fill = min(tpf, ntiles - f * tpf);
      const unsigned char* base = fu_slot(rg, fill0 + f);
      const int k0 = part * ktn / kw, k1 = (part + 1) * ktn / kw;
      const int4 acc = fu_mma_run(reinterpret_cast<const uint4*>(base + (kmajor ? (size_t)j * 512 : (size_t)j * tile_bytes)),
                                  kmajor ? in_fill * 32 : 32, k0, k1, c.xq, c.xstride, nq, lane);
      fu_store_frag(c.red, warp, acc, lane);
    }
    dec_sync();
    for (int i = threadIdx.x; i < ntiles * 16 * ncols; i += kDecThreads) {
      const int row = i & 15, tile = (i >> 4) % ntiles, col = (i >> 4) / ntiles;
      const int f = tile / tpf, j = tile - f * tpf;
      const int in_fill = min(tpf, ntiles - f * tpf);
      const unsigned char* base = fu_slot(rg, fill0 + f);
      const float* sc = scales ? scales + tile * 16 : reinterpret_cast<const float*>(base + (size_t)in_fill * tile_bytes) + j * 16;
      const float v = fu_finalize(c.red, tile * kw, kw, row, col, nterms, c.colscale[col]) * sc[row];
      const size_t idx = (size_t)col * o.ld + o.row0 + tile * 16 + row;
      if (o.out_f) o.out_f[idx] = v;
      else ll_store(o.out + idx, v, o.tag);
    }
  }
}

// ---- one session, three int8 terms: outputs finalised in registers
//
// After the MMAs lane (g, t) holds acc.x = (row g, column 2t), acc.y = (row g, column 2t + 1) and acc.z / acc.w
// the same for row g + 8.  The three terms are columns 0, 1, 2: the lanes with t == 0 own columns 0 and 1 and
// take column 2 from the lane next to them.  Returns (row g, row g + 8), valid in the lanes with t == 0,
// still to be multiplied by colscale / 16 and the row's weight scale.
__device__ __forceinline__ float2 fu_terms(int4 acc) {
  const int lo2 = __shfl_down_sync(0xffffffffu, acc.x, 1);
  const int hi2 = __shfl_down_sync(0xffffffffu, acc.z, 1);
  return make_float2((float)acc.x + (float)acc.y * (1.0f / 128.0f) + (float)lo2 * (1.0f / 16384.0f),
                     (float)acc.z + (float)acc.w * (1.0f / 128.0f) + (float)hi2 * (1.0f / 16384.0f));
}

// fu_gemv_round for one session with three terms: no trip through shared memory when a warp owns whole
// tiles, one float per (warp, row) when the k range of a tile is split.  tpf is a power of two.
__device__ __forceinline__ void fu_gemv_fast(FusedCtx& c, unsigned fill0, int tpf_log2, int ntiles, int ktn, const float* scales,
                                             bool kmajor, FusedOut o) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const FusedRing rg = fu_ring(c);
  const int g = lane >> 2, t = lane & 3;
  const int tpf = 1 << tpf_log2;
  int kw_log2 = 0;
  while ((2 << kw_log2) * ntiles <= kDecWarps && (2 << kw_log2) <= ktn) ++kw_log2;
  const int kw = 1 << kw_log2;
  const size_t tile_bytes = (size_t)ktn * 512;
  const float cs = c.colscale[0] * (1.0f / 16.0f);       // weights entered the MMA as 16 * q
  if (kw == 1) {
    for (int tile = warp; tile < ntiles; tile += kDecWarps) {
      const int f = tile >> tpf_log2, j = tile & (tpf - 1);
      const int in_fill = min(tpf, ntiles - (f << tpf_log2));
      const unsigned char* base = fu_slot(rg, fill0 + f);
      const int4 acc = fu_mma_run(reinterpret_cast<const uint4*>(base + (kmajor ? (size_t)j * 512 : (size_t)j * tile_bytes)),
                                  kmajor ? in_fill * 32 : 32, 0, ktn, c.xq, c.xstride, 3, lane);
      const float2 v = fu_terms(acc);
      if (t == 0) {
        const float* sc = scales ? scales + tile * 16 : reinterpret_cast<const float*>(base + (size_t)in_fill * tile_bytes) + j * 16;
        const int idx = o.row0 + tile * 16 + g;
        const float lo = v.x * cs * sc[g], hi = v.y * cs * sc[g + 8];
        if (o.out_f) { o.out_f[idx] = lo; o.out_f[idx + 8] = hi; }
        else { ll_store(o.out + idx, lo, o.tag); ll_store(o.out + idx + 8, hi, o.tag); }
      }
    }
  } else {
    if (warp < (ntiles << kw_log2)) {
      const int tile = warp >> kw_log2, part = warp & (kw - 1);
      const int f = tile >> tpf_log2, j = tile & (tpf - 1);
      const int in_fill = min(tpf, ntiles - (f << tpf_log2));
      const unsigned char* base = fu_slot(rg, fill0 + f);
      const int k0 = (part * ktn) >> kw_log2, k1 = ((part + 1) * ktn) >> kw_log2;
      const int4 acc = fu_mma_run(reinterpret_cast<const uint4*>(base + (kmajor ? (size_t)j * 512 : (size_t)j * tile_bytes)),
                                  kmajor ? in_fill * 32 : 32, k0, k1, c.xq, c.xstride, 3, lane);
      const float2 v = fu_terms(acc);
      if (t == 0) { c.fpart[warp * 16 + g] = v.x; c.fpart[warp * 16 + g + 8] = v.y; }
    }
    dec_sync();
    if ((int)threadIdx.x < ntiles * 16) {
      const int tile = threadIdx.x >> 4, row = threadIdx.x & 15;
      const int f = tile >> tpf_log2, j = tile & (tpf - 1);
      const int in_fill = min(tpf, ntiles - (f << tpf_log2));
      const unsigned char* base = fu_slot(rg, fill0 + f);
      const float* sc = scales ? scales + tile * 16 : reinterpret_cast<const float*>(base + (size_t)in_fill * tile_bytes) + j * 16;
      float v = 0.f;
      for (int pt = 0; pt < kw; ++pt) v += c.fpart[((tile << kw_log2) + pt) * 16 + row];
      v *= cs * sc[row];
      const int idx = o.row0 + tile * 16 + row;
      if (o.out_f) o.out_f[idx] = v;
      else ll_store(o.out + idx, v, o.tag);
    }
  }
}

// ------------------------------------------------------------------ more polls

// Sum over `nparts` partial vectors of the four values at p + part * stride (words); up to four parts
// are in flight together, the sum runs over the parts in ascending order.
__device__ __forceinline__ float4 ll_sum4_parts(FusedCtx& c, const fu_u64* p, size_t stride, int nparts, unsigned tag) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p0 = 0; p0 < nparts; p0 += 4) {
    const int nb = min(4, nparts - p0);
    fu_u64 w[4][4];
#pragma unroll
    for (int q = 0; q < 4; ++q) w[q][0] = w[q][1] = w[q][2] = w[q][3] = 0;
    {
      long spins = 0;
      while (true) {
        bool ok = true;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (q < nb) {
            const fu_u64* s = p + (size_t)(p0 + q) * stride;
            ll_load2(s, w[q][0], w[q][1]);
            ll_load2(s + 2, w[q][2], w[q][3]);
            ok = ok && ll_ok(w[q][0], tag) && ll_ok(w[q][1], tag) && ll_ok(w[q][2], tag) && ll_ok(w[q][3], tag);
          }
        }
        if (ok) break;
        if (!fu_spin_check(c, spins)) {
          if (c.gave_up[2] == (int)blockIdx.x && atomicCAS(c.gave_up + 7, 0, (int)threadIdx.x + 1) == 0) {
            int bad = 0;
            for (int q = 0; q < 4; ++q)
              for (int e = 0; e < 4; ++e)
                if (q < nb && !ll_ok(w[q][e], tag) && bad == 0) {
                  bad = 1;
                  c.gave_up[4] = (int)(unsigned)(w[q][e] >> 32);
                  c.gave_up[5] = (int)tag;
                  c.gave_up[6] = (int)((p + (size_t)(p0 + q) * stride + e) - c.ll_base);
                }
          }
          break;
        }
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (q < nb) {
        acc.x += ll_val(w[q][0]); acc.y += ll_val(w[q][1]); acc.z += ll_val(w[q][2]); acc.w += ll_val(w[q][3]);
      }
    }
  }
  return acc;
}

// Sums of the two values at p + i * stride for i = first, first + step, ... < count (ascending), four in flight.
__device__ __forceinline__ float2 ll_sum2_strided(FusedCtx& c, const fu_u64* p, size_t stride, int first, int step, int count,
                                              unsigned tag) {
  float s0 = 0.f, s1 = 0.f;
  for (int i0 = first; i0 < count; i0 += 4 * step) {
    fu_u64 w[4][2];
#pragma unroll
    for (int q = 0; q < 4; ++q) w[q][0] = w[q][1] = 0;
    {
      long spins = 0;
      while (true) {
        bool ok = true;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = i0 + q * step;
          if (i < count) {
            ll_load2(p + (size_t)i * stride, w[q][0], w[q][1]);
            ok = ok && ll_ok(w[q][0], tag) && ll_ok(w[q][1], tag);
          }
        }
        if (ok) break;
        if (!fu_spin_check(c, spins)) break;
      }
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (i0 + q * step < count) { s0 += ll_val(w[q][0]); s1 += ll_val(w[q][1]); }
    }
  }
  return make_float2(s0, s1);
}

__device__ __forceinline__ ulonglong2 ll_wait2w(FusedCtx& c, const fu_u64* p, unsigned tag) {
  fu_u64 w0 = 0, w1 = 0;
  {
    long spins = 0;
    while (true) {
      ll_load2(p, w0, w1);
      if (ll_ok(w0, tag) && ll_ok(w1, tag)) break;
      if (!fu_spin_check(c, spins)) break;
    }
  }
  return make_ulonglong2(w0, w1);
}

// ------------------------------------------------------------------ prologues

__device__ __noinline__ void fu_stamp(long long* pts, int bar, int k) {
  pts[((size_t)bar * gridDim.x + blockIdx.x) * 8 + k] = clock64();
}
#define FU_TP(k)                                                                          \
  do {                                                                                    \
    if (a.trace_pts && threadIdx.x == 0) fu_stamp(a.trace_pts, bar, (k));                 \
  } while (0)
#define FU_ARRIVE() FU_TP(7)
#define FU_SEEN(b) do { } while (0)

// x = xres + rmsnorm(f) g_post, f = the sum of `nparts` vectors polled from the exchange area (tag);
// xres <- x; with want_q, xq <- int8 terms of rmsnorm(x) g_pre against the static bound sqrt(d) max|g_pre|.
// One pass, one block reduction: the sums of f^2, xres^2, xres f g_post and (f g_post)^2 give both factors.
template <int NV4>
__device__ __forceinline__ void fu_prologue_resid(const DecodeArgs& a, FusedCtx& c, const fu_u64* src, int nparts, unsigned tag,
                                                  const float* g_post, const float* g_pre, float gmax_pre, bool want_q,
                                                  int bar) {
  const int d = a.dims.d, d4 = d / 4;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nact = NV4 == 1 ? (d4 + 31) >> 5 : kDecWarps;        // warps that hold elements of the vector
  const float bound = sqrtf((float)d) * gmax_pre * 1.0001f;     // |rmsnorm(x)_i g_i| never exceeds it
  const float inv = bound > 0.f ? 127.0f / bound : 0.f;
  for (int col = 0; col < a.ncols; ++col) {
    float4 f[NV4], xi[NV4], gp[NV4];
    float* xr = c.xres + (size_t)col * d;
    if (warp < nact) {
      float sums[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int u = 0; u < NV4; ++u) {
        const int i = threadIdx.x + u * kDecThreads;
        f[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        xi[u] = f[u];
        gp[u] = f[u];
        if (i < d4) {
          f[u] = ll_sum4_parts(c, src + (size_t)col * d + 4 * (size_t)i, (size_t)a.ncols * d, nparts, tag);
          xi[u] = reinterpret_cast<const float4*>(xr)[i];
          gp[u] = reinterpret_cast<const float4*>(g_post)[i];
        }
      }
      if (col == 0) FU_TP(1);
#pragma unroll
      for (int u = 0; u < NV4; ++u) {
        float4 fg = make_float4(f[u].x * gp[u].x, f[u].y * gp[u].y, f[u].z * gp[u].z, f[u].w * gp[u].w);
        sums[0] += f[u].x * f[u].x + f[u].y * f[u].y + f[u].z * f[u].z + f[u].w * f[u].w;
        sums[1] += xi[u].x * xi[u].x + xi[u].y * xi[u].y + xi[u].z * xi[u].z + xi[u].w * xi[u].w;
        sums[2] += xi[u].x * fg.x + xi[u].y * fg.y + xi[u].z * fg.z + xi[u].w * fg.w;
        sums[3] += fg.x * fg.x + fg.y * fg.y + fg.z * fg.z + fg.w * fg.w;
        gp[u] = fg;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) sums[k] = warp_sum(sums[k]);
      if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) c.scratch[k * kDecWarps + warp] = sums[k];
      }
    }
    dec_sync();
    if (warp < nact) {
      float tot[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float sv = (lane & (kDecWarps - 1)) < nact ? c.scratch[k * kDecWarps + (lane & (kDecWarps - 1))] : 0.f;
#pragma unroll
        for (int o = kDecWarps / 2; o > 0; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
        tot[k] = sv;
      }
      const float r = rsqrtf(tot[0] / (float)d + a.dims.eps);
      const float ss2 = fmaxf(tot[1] + 2.0f * r * tot[2] + r * r * tot[3], 0.f);
      const float r2 = rsqrtf(ss2 / (float)d + a.dims.eps);
      int8_t* q0 = c.xq + (size_t)(col * a.nterms) * c.xstride;
#pragma unroll
      for (int u = 0; u < NV4; ++u) {
        const int i = threadIdx.x + u * kDecThreads;
        if (i < d4) {
          float4 x = make_float4(xi[u].x + r * gp[u].x, xi[u].y + r * gp[u].y, xi[u].z + r * gp[u].z, xi[u].w + r * gp[u].w);
          reinterpret_cast<float4*>(xr)[i] = x;
          if (want_q) {
            float4 gq = reinterpret_cast<const float4*>(g_pre)[i];
            const float k = r2 * inv;
            fu_quantize4(make_float4(x.x * gq.x * k, x.y * gq.y * k, x.z * gq.z * k, x.w * gq.w * k), a.nterms, q0, 4 * i, c.xstride);
          }
        }
      }
      if (threadIdx.x == 0) c.colscale[col] = bound / 127.0f;
    }
    dec_sync();        // xq, xres and colscale are complete; scratch is free for the next session
  }
}

// x = dequant(E[token]) sqrt(d); xres <- x; xq <- int8 terms of rmsnorm(x) g_pre.
template <int NV4>
__device__ __forceinline__ void fu_prologue_embed(const DecodeArgs& a, FusedCtx& c, const float* g_pre, float gmax_pre, bool want_q) {
  const int d = a.dims.d, d4 = d / 4;
  const float emb = sqrtf((float)d);
  const float bound = sqrtf((float)d) * gmax_pre * 1.0001f;
  const float inv = bound > 0.f ? 127.0f / bound : 0.f;
  for (int col = 0; col < a.ncols; ++col) {
    int tok = c.tok[col];
    if (tok < 0 || tok >= a.dims.vocab) {
      if (threadIdx.x == 0) atomicExch(c.err, (int)kDevBadToken);
      tok = 0;
    }
    const unsigned short* row = reinterpret_cast<const unsigned short*>(a.embed_rows + (size_t)tok * (d / 2));
    const float sc = __ldg(a.embed_scale + tok) * emb;
    float* xr = c.xres + (size_t)col * d;
    float4 x[NV4];
    float ss = 0.f;
#pragma unroll
    for (int u = 0; u < NV4; ++u) {
      const int i = threadIdx.x + u * kDecThreads;
      x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (i < d4) {
        const unsigned b = __ldg(row + i);        // four nibbles: elements 4i .. 4i+3, low nibble first
        int q0 = b & 0xF, q1 = (b >> 4) & 0xF, q2 = (b >> 8) & 0xF, q3 = (b >> 12) & 0xF;
        x[u] = make_float4((float)(q0 >= 8 ? q0 - 16 : q0) * sc, (float)(q1 >= 8 ? q1 - 16 : q1) * sc,
                           (float)(q2 >= 8 ? q2 - 16 : q2) * sc, (float)(q3 >= 8 ? q3 - 16 : q3) * sc);
        reinterpret_cast<float4*>(xr)[i] = x[u];
        ss += x[u].x * x[u].x + x[u].y * x[u].y + x[u].z * x[u].z + x[u].w * x[u].w;
      }
    }
    ss = block_sum(ss, c.scratch);
    const float k = rsqrtf(ss / (float)d + a.dims.eps) * inv;
    int8_t* q0 = c.xq + (size_t)(col * a.nterms) * c.xstride;
    if (want_q) {
#pragma unroll
      for (int u = 0; u < NV4; ++u) {
        const int i = threadIdx.x + u * kDecThreads;
        if (i < d4) {
          float4 gq = reinterpret_cast<const float4*>(g_pre)[i];
          fu_quantize4(make_float4(x[u].x * gq.x * k, x[u].y * gq.y * k, x[u].z * gq.z * k, x[u].w * gq.w * k), a.nterms, q0, 4 * i,
                       c.xstride);
        }
      }
    }
    if (threadIdx.x == 0) c.colscale[col] = bound / 127.0f;
  }
  dec_sync();
}

// The residual fits one float4 per thread up to d = 2048: the narrow instantiation is a third of the code.
__device__ __forceinline__ void fu_resid(const DecodeArgs& a, FusedCtx& c, const fu_u64* src, int nparts, unsigned tag,
                                         const float* g_post, const float* g_pre, float gmax_pre, bool want_q, int bar) {
  if (a.dims.d <= 4 * kDecThreads) fu_prologue_resid<1>(a, c, src, nparts, tag, g_post, g_pre, gmax_pre, want_q, bar);
  else fu_prologue_resid<kFuMaxV4>(a, c, src, nparts, tag, g_post, g_pre, gmax_pre, want_q, bar);
}
__device__ __forceinline__ void fu_embed(const DecodeArgs& a, FusedCtx& c, const float* g_pre, float gmax_pre, bool want_q) {
  if (a.dims.d <= 4 * kDecThreads) fu_prologue_embed<1>(a, c, g_pre, gmax_pre, want_q);
  else fu_prologue_embed<kFuMaxV4>(a, c, g_pre, gmax_pre, want_q);
}

// Quantises `K` values per session held in shared memory (vals[col * K + k]) against each session's
// own maximum; K <= 4 * kDecThreads.
__device__ __forceinline__ void fu_quantize_dynamic(const DecodeArgs& a, FusedCtx& c, const float* vals, int K) {
  const int n4 = K / 4;
  for (int col = 0; col < a.ncols; ++col) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if ((int)threadIdx.x < n4) v = reinterpret_cast<const float4*>(vals + (size_t)col * K)[threadIdx.x];
    float m = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    m = block_max(m, c.scratch);
    const float inv = m > 0.f ? 127.0f / m : 0.f;
    if ((int)threadIdx.x < n4)
      fu_quantize4(make_float4(v.x * inv, v.y * inv, v.z * inv, v.w * inv), a.nterms,
                   c.xq + (size_t)(col * a.nterms) * c.xstride, 4 * threadIdx.x, c.xstride);
    if (threadIdx.x == 0) c.colscale[col] = m > 0.f ? m / 127.0f : 0.f;
    dec_sync();           // scratch is reused by the next session's maximum; xq and colscale are complete
  }
}

// ------------------------------------------------------------------ attention

// This CTA's attention work item of a layer, or item < 0.
struct FusedAttnItem {
  int item, col, kvh, split, nsplit;
  int pos, k0, n_old, has_new;      // query position, first key of the split, cached keys, new key in this split
  int nfills;                       // 1 (RoPE row + QK gains) + key slots
};

__device__ __forceinline__ FusedAttnItem fu_attn_item(const DecodeArgs& a, const FusedPlan& pl, const FusedCtx& c, int layer,
                                                      int cta, int step) {
  const ModelDims& dm = a.dims;
  FusedAttnItem it;
  const int is_global = c.lw[layer].is_global;
  it.nsplit = is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
  const int items = a.ncols * dm.hkv * it.nsplit;
  it.item = cta < items ? cta : -1;
  it.col = it.kvh = it.split = it.pos = it.k0 = it.n_old = it.has_new = it.nfills = 0;
  if (it.item < 0) return it;
  it.split = cta % it.nsplit;
  const int rest = cta / it.nsplit;
  it.kvh = rest % dm.hkv;
  it.col = rest / dm.hkv;
  int pos = c.pos0[it.col] + step;
  if (pos < 0 || pos >= dm.max_ctx) pos = 0;       // reported by the consumer side
  it.pos = pos;
  int k0, k1;
  attn_split_range(dm, pos, is_global, it.nsplit, it.split, &k0, &k1);
  it.k0 = k0;
  it.has_new = (k1 == pos + 1 && k1 > k0) ? 1 : 0;
  const int n_old = (it.has_new ? k1 - 1 : k1) - k0;
  it.n_old = n_old > 0 ? n_old : 0;
  it.nfills = 1 + (it.n_old + pl.kps - 1) / pl.kps;
  return it;
}

// One (session, kv head, split) item.  The split's cached K/V rows sit in ring slots (kps keys per slot:
// their K rows, then their V rows), processed in rounds of round_fills slots; all splits shift the softmax by
// the layer's static score bound, so the partial sums (sum p v, sum p) of splits and rounds simply add.
template <typename T, int HD, int G>
__device__ __forceinline__ unsigned fu_attention(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, int layer, int step,
                                              unsigned fill_no, fu_u64* ll, unsigned tag, int bar) {
  const ModelDims& dm = a.dims;
  const FusedAttnItem it = fu_attn_item(a, pl, c, layer, blockIdx.x, step);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const FusedRing rg = fu_ring(c);
  constexpr int half = HD / 2;
  constexpr int KP = kDecThreads / HD;               // key parts of the P.V stage
  constexpr int DPL = HD / 32;                       // dims of a row per lane in the score stage
  const LayerWeights& L = c.lw[layer];
  const LayerKv kv = c.lkv[layer];
  const int pos = it.pos, kvh = it.kvh, col = it.col;
  const int maxkeys = pl.round_fills * pl.kps + 1;
  float* q_s = c.attn;                               // [G][HD]
  float* k_s = q_s + G * HD;                         // [HD] new key (normed, roped)
  float* v_s = k_s + HD;                             // [HD]
  float* sc = v_s + HD;                              // [maxkeys][G] probabilities exp(score - bound)
  float* ored = sc + ((G * maxkeys + 3) & ~3);       // [KP][G][HD]
  float* lred = ored + (size_t)KP * G * HD;          // [KP][G]
  const size_t rowb = (size_t)HD * sizeof(T);
  // ---- RoPE row and QK-norm gains (first fill of the item)
  const unsigned aux_fill = fill_no;
  fu_acquire(rg, c, aux_fill);
  const float* cos_r = reinterpret_cast<const float*>(fu_slot(rg, aux_fill));
  const float* sin_r = cos_r + half;
  const float* g_q = sin_r + half;
  const float* g_k = g_q + HD;
  // ---- q heads of the group, new k and v of this kv head: polled straight into shared memory
  {
    const fu_u64* qkv = ll + pl.ll_qkv + (size_t)col * dm.nqkv();
    const int i = threadIdx.x;
    if (i < (G + 2) * HD / 4) {
      const int e = 4 * i;
      int src;
      float* dst;
      if (e < G * HD) { src = kvh * G * HD + e; dst = q_s + e; }
      else if (e < (G + 1) * HD) { src = dm.nq() + kvh * HD + (e - G * HD); dst = k_s + (e - G * HD); }
      else { src = dm.nq() + dm.nkv() + kvh * HD + (e - (G + 1) * HD); dst = v_s + (e - (G + 1) * HD); }
      *reinterpret_cast<float4*>(dst) = ll_wait4(c, qkv + src, tag);
    }
  }
  FU_SEEN(bar - 1);
  FU_TP(1);
  dec_sync();
  // ---- QK-RMSNorm, RoPE, attention scale (in place: a warp holds its head in registers)
  const float att_scale = rsqrtf((float)HD);
  if (warp <= G) {
    float* hp = warp < G ? q_s + warp * HD : k_s;
    const float* gain = warp < G ? g_q : g_k;
    float v[HD / 32];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < HD / 32; ++i) { v[i] = hp[lane + 32 * i]; ss += v[i] * v[i]; }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / (float)HD + dm.eps);
    const float post = warp < G ? att_scale : 1.0f;
    __syncwarp();
    if constexpr (HD == 32) {                 // the pair of element e sits 16 lanes away
      float x = v[0] * r * gain[lane];
      float y = __shfl_xor_sync(0xffffffffu, x, 16);
      if (lane < 16) {
        float cs = cos_r[lane], sn = sin_r[lane];
        hp[lane] = (x * cs - y * sn) * post;
        hp[lane + 16] = (y * cs + x * sn) * post;
      }
    } else {
#pragma unroll
      for (int i = 0; i < HD / 64; ++i) {     // element e = lane + 32 i pairs with e + half
        const int e = lane + 32 * i;
        float a0 = v[i] * r * gain[e], b0 = v[i + HD / 64] * r * gain[e + half];
        float cs = cos_r[e], sn = sin_r[e];
        hp[e] = (a0 * cs - b0 * sn) * post;
        hp[e + half] = (b0 * cs + a0 * sn) * post;
      }
    }
  }
  dec_sync();
  FU_TP(2);
  const int* ptab = a.page_table + (size_t)col * a.pages_per_seq;
  if (it.split == 0) {     // KV append: exactly one CTA per (session, kv head)
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
  if constexpr (sizeof(T) == 2) {                     // what a bf16 cache would hand back
    dec_sync();
    for (int e = threadIdx.x; e < HD; e += kDecThreads) {
      k_s[e] = __bfloat162float(__float2bfloat16(k_s[e]));
      v_s[e] = __bfloat162float(__float2bfloat16(v_s[e]));
    }
    dec_sync();
  }
  const float shift = L.attn_bound;
  const int pv_e = threadIdx.x % HD, pv_part = threadIdx.x / HD;
  float o[G], lsum[G];
#pragma unroll
  for (int g = 0; g < G; ++g) { o[g] = 0.f; lsum[g] = 0.f; }
  float qreg[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) stream_load_dims<float, DPL>(nullptr, q_s + g * HD, lane, qreg[g]);
  const int kps = pl.kps, kps_log2 = fu_log2(pl.kps);      // a power of two
  const int RK = pl.round_fills * kps;
  const int nrounds = it.n_old <= 0 ? 1 : (it.n_old + RK - 1) / RK;
  const unsigned key_fill0 = aux_fill + 1;
  for (int rd = 0; rd < nrounds; ++rd) {
    const int r0 = rd * RK;
    const int nrows = max(0, min(RK, it.n_old - r0));
    const int nf = (nrows + kps - 1) >> kps_log2;
    const unsigned f0 = key_fill0 + (unsigned)(r0 >> kps_log2);
    for (int f = 0; f < nf; ++f) fu_acquire(rg, c, f0 + f);
    const bool lastr = rd == nrounds - 1;
    const int nk = nrows + ((lastr && it.has_new) ? 1 : 0);
    if (rd == 0) FU_TP(3);
    // ---- probabilities p[key][head] = exp(q_head . k_key - shift): a warp takes two keys at a time
    for (int kp = warp; 2 * kp < nk; kp += kDecWarps) {
      const int ka = 2 * kp, kb_ = min(2 * kp + 1, nk - 1);
      const T* ra = nullptr;
      const T* rb = nullptr;
      if (ka < nrows) ra = reinterpret_cast<const T*>(fu_slot(rg, f0 + (ka >> kps_log2)) + (size_t)(ka & (kps - 1)) * rowb);
      if (kb_ < nrows) rb = reinterpret_cast<const T*>(fu_slot(rg, f0 + (kb_ >> kps_log2)) + (size_t)(kb_ & (kps - 1)) * rowb);
      float xa[DPL], xb[DPL];
      stream_load_dims<T, DPL>(ra, k_s, lane, xa);
      stream_load_dims<T, DPL>(rb, k_s, lane, xb);
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
    // ---- P.V and the row sums: this thread's element of V against the probabilities of all heads
    for (int kk = pv_part; kk < nk; kk += KP) {
      float v;
      if (kk < nrows) {
        const T* rv = reinterpret_cast<const T*>(fu_slot(rg, f0 + (kk >> kps_log2)) + (size_t)(kps + (kk & (kps - 1))) * rowb);
        v = kv_to_float<T>(rv[pv_e]);
      } else {
        v = v_s[pv_e];
      }
      float pg[G];
      if constexpr (G == 4) {
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
    // the slots of this round (and with them the probabilities) are free again; round 0 frees the first fill too
    if (rd == 0) fu_release(rg, aux_fill, nf + 1);
    else fu_release(rg, f0, nf);
  }
  FU_TP(4);
  // ---- the key parts meet in shared memory, part 0 publishes the split's partial result
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
    fu_u64* part = ll + pl.ll_part + (size_t)it.item * pl.part_stride;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float acc = o[g];
      for (int kp = 1; kp < KP; ++kp) acc += ored[((size_t)kp * G + g) * HD + pv_e];
      ll_store(part + g * HD + pv_e, acc, tag);
      if (pv_e == 0) {
        float ls = 0.f;
        for (int kp = 0; kp < KP; ++kp) ls += lred[kp * G + g];
        ll_store(part + G * HD + g, ls, tag);
      }
    }
  }
  FU_ARRIVE();
  dec_sync();
  return aux_fill + (unsigned)it.nfills;
}

// Combine of the split partials of one head slice (the o-proj input), quantised per session against its
// own maximum.  All splits share one softmax shift, so the combine is sum(o) / sum(l).
__device__ __forceinline__ void fu_prologue_combine(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, int layer, int slice,
                                                    const fu_u64* ll, unsigned tag, int bar) {
  const ModelDims& dm = a.dims;
  const int Ks = dm.nq() / a.o_slices, hps = Ks / dm.hd, G = dm.group();
  const int nsplit = c.lw[layer].is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int P = Ks / 2;                            // output pairs
  int tpo = 1;                                     // threads per pair: a power of two
  while (tpo * 2 * P <= kDecThreads && tpo * 2 <= nsplit) tpo *= 2;
  float* xf = c.act;                               // [ncols][Ks]
  float* part = c.act + (size_t)a.ncols * 512;     // [tpo][Ks]
  float* lsum = c.scratch + 64;                    // [hps]
  const size_t pstride = (size_t)pl.part_stride;
  for (int col = 0; col < a.ncols; ++col) {
    for (int hh = warp; hh < hps; hh += kDecWarps) {
      const int h = slice * hps + hh, kvh = h / G, g = h % G;
      const fu_u64* pl0 = ll + pl.ll_part + ((size_t)(col * dm.hkv + kvh) * nsplit) * pstride + G * dm.hd + g;
      float ls = 0.f;
      for (int sp = lane; sp < nsplit; sp += 32) ls += ll_val(ll_wait1(c, pl0 + (size_t)sp * pstride, tag));
      ls = warp_sum(ls);
      if (lane == 0) lsum[hh] = ls;
    }
    const int pair = threadIdx.x % P, part_id = threadIdx.x / P;
    if (part_id < tpo) {
      const int j = 2 * pair, hh = j / dm.hd, e = j - hh * dm.hd;
      const int h = slice * hps + hh, kvh = h / G, g = h % G;
      const fu_u64* po = ll + pl.ll_part + ((size_t)(col * dm.hkv + kvh) * nsplit) * pstride + g * dm.hd + e;
      const float2 s2 = ll_sum2_strided(c, po, pstride, part_id, tpo, nsplit, tag);
      part[(size_t)part_id * Ks + j] = s2.x;
      part[(size_t)part_id * Ks + j + 1] = s2.y;
    }
    if (col == 0) { FU_SEEN(bar - 1); FU_TP(1); }
    dec_sync();
    if ((int)threadIdx.x < Ks) {
      const int j = threadIdx.x, hh = j / dm.hd;
      float acc = 0.f;
      for (int t = 0; t < tpo; ++t) acc += part[(size_t)t * Ks + j];
      const float ls = lsum[hh];
      xf[(size_t)col * Ks + j] = ls > 0.f ? acc / ls : 0.f;
    }
    dec_sync();
  }
  fu_quantize_dynamic(a, c, xf, Ks);
}

// ------------------------------------------------------------------ per-CTA shares

struct FusedCta {
  int a_t0, a_n;                 // qkv row tiles
  int c_slice, c_t0, c_n;        // o-proj K slice and row tiles (c_n == 0: none)
  int f_prod, f_kt0, f_mk;       // ffn: producer index (-1: none), first 64-feature k tile, k tiles
  int r_e0, r_n;                 // reducer: first element of d, elements (0: none)
  int h_t0, h_n;                 // head row tiles
};

__device__ __forceinline__ FusedCta fu_cta_share(const DecodeArgs& a, const FusedPlan& pl, int cta, int ncta) {
  const ModelDims& dm = a.dims;
  FusedCta s;
  const int ntA = dm.nqkv() / 16;
  s.a_t0 = cta * pl.a_per;
  s.a_n = max(0, min(ntA, s.a_t0 + pl.a_per) - s.a_t0);
  s.c_slice = cta / pl.c_cps;
  s.c_t0 = (cta - s.c_slice * pl.c_cps) * pl.c_per;
  s.c_n = s.c_slice < a.o_slices ? max(0, min(dm.d / 16, s.c_t0 + pl.c_per) - s.c_t0) : 0;
  const int KTd = dm.ffn / 64;
  s.f_prod = cta < pl.nprod ? cta : -1;
  s.f_kt0 = cta * pl.ffn_m;
  s.f_mk = s.f_prod >= 0 ? min(pl.ffn_m, KTd - s.f_kt0) : 0;
  s.r_e0 = cta * pl.r_per;
  s.r_n = cta < pl.nred ? min(pl.r_per, dm.d - s.r_e0) : 0;
  const int ntH = dm.vocab / 16;
  s.h_t0 = (int)((long long)cta * ntH / ncta);
  s.h_n = (int)((long long)(cta + 1) * ntH / ncta) - s.h_t0;
  return s;
}

// ------------------------------------------------------------------ producer warp

// The slot of fill n is still in use: bounded wait.  False when it gave up (the CTA is then marked dead).
__device__ __noinline__ bool fu_prod_wait_slow(FusedCtx& c, unsigned n) {
  if (*c.dead) return false;
  const unsigned s = n & (unsigned)(c.nslots - 1);
  if (!mbar_wait(&c.empty[s], ((n >> c.nslots_log2) - 1u) & 1u, c.err)) {
    if ((threadIdx.x & 31) == 0 && atomicCAS(c.gave_up + 3, 0, 3) == 0) {
      c.gave_up[0] = 8;
      c.gave_up[1] = (int)n;
      c.gave_up[2] = blockIdx.x;
    }
    *c.dead = 1;
    return false;
  }
  return true;
}
// Waits for the slot of fill n to be free and arms its barrier for `bytes`; returns the slot, or nullptr
// when the wait gave up.
__device__ __forceinline__ unsigned char* fu_prod_begin(const FusedRing& r, FusedCtx& c, unsigned n, uint32_t bytes) {
  const unsigned s = n & r.mask;
  if (n > r.mask && !mbar_test(&r.empty[s], ((n >> r.log2) - 1u) & 1u)) {
    if (!fu_prod_wait_slow(c, n)) return nullptr;
  }
  if ((threadIdx.x & 31) == 0) {
    mbar_arrive_expect_tx(&r.full[s], bytes);
    if (c.fill_log && n < 4000u) c.fill_log[3 * n] = clock64();
  }
  __syncwarp();
  return r.ring + (size_t)s * r.slot_bytes;
}
__device__ __forceinline__ uint64_t* fu_prod_bar(const FusedRing& r, unsigned n) { return &r.full[n & r.mask]; }

template <typename T>
__device__ __noinline__ void fused_producer(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh, int nsteps) {
  const ModelDims& dm = a.dims;
  const int lane = threadIdx.x & 31, cta = blockIdx.x;
  const int ktn = dm.d / 64;
  const uint32_t rec_b = (uint32_t)ktn * 512u + 64u, gain_b = (uint32_t)dm.d * 4u;
  const FusedRing rg = fu_ring(c);
  unsigned n = 0;                    // next fill
  unsigned char* dst;
// one contiguous copy fills the slot
#define FU_FILL1(src, bytes)                                                      \
  do {                                                                            \
    dst = fu_prod_begin(rg, c, n, (bytes));                                           \
    if (!dst) return;                                                             \
    if (lane == 0) bulk_load_1d(dst, (src), (bytes), fu_prod_bar(rg, n));          \
    ++n;                                                                          \
  } while (0)
  for (int step = 0; step < nsteps; ++step) {
    for (int layer = 0; layer < dm.n_layers; ++layer) {
      const LayerWeights& L = c.lw[layer];
      const ChainedLayer& Cl = c.cl[layer];
      // ---- A: gains [pre | post], then this CTA's row-tile records of W_qkv
      FU_FILL1(Cl.gA, layer > 0 ? 2u * gain_b : gain_b);
      for (int i = 0; i < sh.a_n; ++i) FU_FILL1(Cl.wqkv_s + (size_t)(sh.a_t0 + i) * rec_b, rec_b);
      // ---- B
      {
        // cache rows of earlier steps are fetched only once those steps are complete
        for (long spins = 0; *c.step_ready <= step; ++spins) {
          __nanosleep(64);
          if (*c.dead) return;
          if (spins > (1L << 24)) { *c.dead = 1; return; }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        const FusedAttnItem it = fu_attn_item(a, pl, c, layer, cta, step);
        if (it.item >= 0) {
          const int t = L.is_global ? 1 : 0;
          const uint32_t rope_b = (uint32_t)dm.hd * 4u, qk_b = 2u * (uint32_t)dm.hd * 4u;
          dst = fu_prod_begin(rg, c, n, rope_b + qk_b);
          if (!dst) return;
          if (lane == 0) bulk_load_1d(dst, a.rope_cs[t] + (size_t)it.pos * dm.hd, rope_b, fu_prod_bar(rg, n));
          if (lane == 1) bulk_load_1d(dst + rope_b, Cl.qk, qk_b, fu_prod_bar(rg, n));
          ++n;
          // K rows of a slot's keys, then their V rows; keys of one page are contiguous in the cache
          const uint32_t rowb = (uint32_t)dm.hd * (uint32_t)sizeof(T);
          const int* ptab = a.page_table + (size_t)it.col * a.pages_per_seq;
          const unsigned char* kb = reinterpret_cast<const unsigned char*>(c.lkv[layer].k);
          const unsigned char* vb = reinterpret_cast<const unsigned char*>(c.lkv[layer].v);
          for (int r0 = 0; r0 < it.n_old; r0 += pl.kps) {
            const int nr = min(pl.kps, it.n_old - r0);
            dst = fu_prod_begin(rg, c, n, 2u * (uint32_t)nr * rowb);
            if (!dst) return;
            // lanes 0 / 1: K rows before / after a page boundary, lanes 2 / 3: V rows
            if (lane < 4) {
              const int key0 = it.k0 + r0;
              const int first = min(nr, kPage - (key0 % kPage));       // rows in the page of key0
              const int seg = lane & 1, isv = lane >> 1;
              const int rbeg = seg ? first : 0, rn = seg ? nr - first : first;
              if (rn > 0) {
                const int key = key0 + rbeg;
                const size_t off = ((((size_t)ptab[key / kPage] * dm.hkv + it.kvh) * kPage + (key % kPage)) * dm.hd) * sizeof(T);
                bulk_load_1d(dst + (size_t)((isv ? pl.kps : 0) + rbeg) * rowb, (isv ? vb : kb) + off, (uint32_t)rn * rowb,
                             fu_prod_bar(rg, n));
              }
            }
            ++n;
          }
        }
      }
      // ---- C: this CTA's row tiles of W_o restricted to its head slice (contiguous), then their scales
      if (sh.c_n > 0) {
        const int KTo = dm.nq() / 64, ktc = KTo / a.o_slices, RT = dm.d / 16;
        const uint32_t ctile = (uint32_t)ktc * 512u;
        for (int t0 = 0; t0 < sh.c_n; t0 += pl.c_tps) {
          const int nt = min(pl.c_tps, sh.c_n - t0);
          dst = fu_prod_begin(rg, c, n, (uint32_t)nt * (ctile + 64u));
          if (!dst) return;
          if (lane == 0)
            bulk_load_1d(dst, Cl.wo_s + (((size_t)sh.c_slice * RT + sh.c_t0 + t0) * ktc) * 32, (uint32_t)nt * ctile, fu_prod_bar(rg, n));
          if (lane == 1)
            bulk_load_1d(dst + (size_t)nt * ctile, L.so + (size_t)(sh.c_t0 + t0) * 16, (uint32_t)nt * 64u, fu_prod_bar(rg, n));
          ++n;
        }
      }
      // ---- DE: gains, gate / up records of this CTA's features, its K slice of W_down
      FU_FILL1(Cl.gD, 2u * gain_b);
      if (sh.f_prod >= 0) {
        for (int i = 0; i < 8 * sh.f_mk; ++i) FU_FILL1(Cl.wgu_s + (size_t)(8 * sh.f_kt0 + i) * rec_b, rec_b);
        // [k_tile][row_tile] order: a slot holds, for each k tile of the slice, `nt` consecutive row tiles,
        // then the scales of those rows
        const int nrt = dm.d / 16;
        for (int t0 = 0; t0 < nrt; t0 += pl.d_tps) {
          const int nt = min(pl.d_tps, nrt - t0);
          dst = fu_prod_begin(rg, c, n, (uint32_t)(nt * sh.f_mk) * 512u + (uint32_t)nt * 64u);
          if (!dst) return;
          if (lane < sh.f_mk)
            bulk_load_1d(dst + (size_t)lane * nt * 512, Cl.wdown_k + ((size_t)(sh.f_kt0 + lane) * nrt + t0) * 32, (uint32_t)nt * 512u,
                         fu_prod_bar(rg, n));
          if (lane == 31)
            bulk_load_1d(dst + (size_t)nt * sh.f_mk * 512, L.sdown + (size_t)t0 * 16, (uint32_t)nt * 64u, fu_prod_bar(rg, n));
          ++n;
        }
      }
    }
    // ---- H
    FU_FILL1(a.gH, 2u * gain_b);
    for (int i = 0; i < sh.h_n; ++i) FU_FILL1(a.head_ws + (size_t)(sh.h_t0 + i) * rec_b, rec_b);
  }
#undef FU_FILL1
}

// ------------------------------------------------------------------ the phases
//
// Every phase is one out-of-line function of (step, layer, fills consumed so far) that returns the new
// fill count: the kernel's main loop then keeps next to nothing live across the calls.

// Phase code * 1000 + layer for the report of a wait that gave up, and the CTA's progress word.
__device__ __forceinline__ void fu_mark(const DecodeArgs& a, FusedCtx& c, int step, int where) {
  if (threadIdx.x == 0) {
    c.where = where;
    a.progress[blockIdx.x] = step * 10000 + where;
  }
}

// Lowest index wins ties, NaN never wins.
__device__ __forceinline__ void fu_better(float& bv, int& bi, float v, int i) {
  if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
}

__device__ __forceinline__ unsigned fu_tag(const DecodeArgs& a, const FusedPlan& pl, int step, int layer) {
  return pl.tag0 + (unsigned)step * (unsigned)(a.dims.n_layers + 1) + (unsigned)layer + 1u;
}
// The exchange area alternates between two copies by layer parity.
__device__ __forceinline__ fu_u64* fu_ll(const FusedPlan& pl, FusedCtx& c, int layer) {
  return c.ll_base + (size_t)(layer & 1) * pl.ll_words;
}

// A: residual update (or embedding) + pre-attention norm -> this CTA's rows of the QKV projection.
__device__ __forceinline__ unsigned fu_phase_qkv(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh, int step,
                                              int layer, unsigned fill_no) {
  const ModelDims& dm = a.dims;
  const FusedRing rg = fu_ring(c);
  const int bar = layer * 5, d = dm.d;
  fu_mark(a, c, step, 1000 + layer);
  FU_TP(0);
  const unsigned tag = fu_tag(a, pl, step, layer);
  const unsigned gf = fill_no;
  fu_acquire(rg, c, gf);
  const float* g_pre = reinterpret_cast<const float*>(fu_slot(rg, gf));
  if (layer == 0) fu_embed(a, c, g_pre, c.lw[0].gmax_pre_attn, sh.a_n > 0);
  else fu_resid(a, c, fu_ll(pl, c, layer - 1) + pl.ll_f, 1, tag - 1u, g_pre + d, g_pre, c.lw[layer].gmax_pre_attn, sh.a_n > 0, bar);
  FU_TP(2);
  fu_release(rg, gf, 1);
  fill_no = gf + 1;
  for (int t0 = 0; t0 < sh.a_n; t0 += pl.round_fills) {
    const int nt = min(pl.round_fills, sh.a_n - t0);
    for (int f = 0; f < nt; ++f) fu_acquire(rg, c, fill_no + f);
    if (t0 == 0) FU_TP(5);
    const FusedOut o{fu_ll(pl, c, layer) + pl.ll_qkv, nullptr, dm.nqkv(), (sh.a_t0 + t0) * 16, tag};
    if (a.ncols == 1 && a.nterms == 3) fu_gemv_fast(c, fill_no, 0, nt, d / 64, nullptr, false, o);
    else fu_gemv_round(c, fill_no, 1, nt, d / 64, nullptr, false, a.ncols, a.nterms, o);
    fu_release(rg, fill_no, nt);
    fill_no += nt;
  }
  FU_ARRIVE();
  return fill_no;
}

// C: combine of the attention partials of this CTA's head slice -> its rows of the O projection.
__device__ __forceinline__ unsigned fu_phase_oproj(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh, int step,
                                                int layer, unsigned fill_no) {
  const ModelDims& dm = a.dims;
  const FusedRing rg = fu_ring(c);
  const int bar = layer * 5 + 2, d = dm.d;
  fu_mark(a, c, step, 3000 + layer);
  FU_TP(0);
  if (sh.c_n > 0) {
    const unsigned tag = fu_tag(a, pl, step, layer);
    fu_u64* ll = fu_ll(pl, c, layer);
    fu_prologue_combine(a, pl, c, layer, sh.c_slice, ll, tag, bar);
    FU_TP(2);
    const int ktc = dm.nq() / 64 / a.o_slices;
    const int nf_all = (sh.c_n + pl.c_tps - 1) / pl.c_tps;
    for (int fr = 0; fr < nf_all; fr += pl.round_fills) {
      const int nf = min(pl.round_fills, nf_all - fr);
      const int t0 = fr * pl.c_tps, nt = min(sh.c_n - t0, nf * pl.c_tps);
      for (int f = 0; f < nf; ++f) fu_acquire(rg, c, fill_no + f);
      const FusedOut o{ll + pl.ll_o + (size_t)sh.c_slice * a.ncols * d, nullptr, d, (sh.c_t0 + t0) * 16, tag};
      if (a.ncols == 1 && a.nterms == 3) fu_gemv_fast(c, fill_no, fu_log2(pl.c_tps), nt, ktc, nullptr, false, o);
      else fu_gemv_round(c, fill_no, pl.c_tps, nt, ktc, nullptr, false, a.ncols, a.nterms, o);
      fu_release(rg, fill_no, nf);
      fill_no += nf;
    }
  }
  FU_ARRIVE();
  return fill_no;
}

// Gate / up, GeGLU and down for one session, three terms and 64 features per CTA (eight gate / up row
// tiles, one k tile of W_down per row tile).  Warp (p, q) multiplies the gate AND the up tile of feature
// pair-tile p over k quarter q, so GeGLU needs no second exchange; warp 0 turns the 64 sums into
// quantised activations (their maximum is two shuffle rounds away); every warp then owns whole row tiles
// of the down projection and finalises them in registers.
__device__ __forceinline__ unsigned fu_ffn_fast(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh,
                                                unsigned fill_no, fu_u64* out, unsigned tag, int bar) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const FusedRing rg = fu_ring(c);
  const int g = lane >> 2, t = lane & 3;
  const int d = a.dims.d, ktn = d / 64;
  const unsigned mask = rg.mask;
  {
    const int p = warp & 3, q = warp >> 2;
    const unsigned fg = fill_no + 2u * p;
    fu_acquire(rg, c, fg);
    fu_acquire(rg, c, fg + 1);
    if (warp == 0) FU_TP(5);
    const int k0 = (q * ktn) >> 2, k1 = ((q + 1) * ktn) >> 2;
    const int4 ag = fu_mma_run(reinterpret_cast<const uint4*>(fu_slot(rg, fg)), 32, k0, k1, c.xq, c.xstride, 3, lane);
    const int4 au = fu_mma_run(reinterpret_cast<const uint4*>(fu_slot(rg, fg + 1)), 32, k0, k1, c.xq, c.xstride, 3, lane);
    const float2 vg = fu_terms(ag), vu = fu_terms(au);
    float* fp = c.act + ((q * 4 + p) * 2) * 16;          // [4 quarters][4 pair tiles][gate, up][16 rows]
    if (t == 0) { fp[g] = vg.x; fp[g + 8] = vg.y; fp[16 + g] = vu.x; fp[16 + g + 8] = vu.y; }
  }
  dec_sync();
  FU_TP(3);
  if (warp < 2) {                    // 64 features, one per lane of two warps
    const float cs = c.colscale[0] * (1.0f / 16.0f);
    const int f = threadIdx.x, pp = f >> 4, row = f & 15;
    float gate = 0.f, up = 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      gate += c.act[((q * 4 + pp) * 2) * 16 + row];
      up += c.act[((q * 4 + pp) * 2 + 1) * 16 + row];
    }
    const float sg = reinterpret_cast<const float*>(fu_slot(rg, fill_no + 2u * pp) + (size_t)ktn * 512)[row];
    const float su = reinterpret_cast<const float*>(fu_slot(rg, fill_no + 2u * pp + 1u) + (size_t)ktn * 512)[row];
    const float av = gelu_tanh(gate * cs * sg) * (up * cs * su);
    float m = warp_max(fabsf(av));
    if (lane == 0) c.scratch[warp] = m;
    asm volatile("bar.sync 2, 64;" ::: "memory");       // the two warps only
    m = fmaxf(c.scratch[0], c.scratch[1]);
    const float v = av * (m > 0.f ? 127.0f / m : 0.f);
    const float t0 = rintf(v), r1 = (v - t0) * 128.0f, t1 = rintf(r1), t2 = rintf((r1 - t1) * 128.0f);
    int8_t* q8 = c.xq + fu_perm(f);
    q8[0] = (int8_t)(int)t0;
    q8[c.xstride] = (int8_t)(int)t1;
    q8[2 * c.xstride] = (int8_t)(int)t2;
    if (threadIdx.x == 0) c.colscale[0] = m > 0.f ? m / 127.0f : 0.f;
  }
  dec_sync();
  FU_TP(4);
  if (threadIdx.x < 8) mbar_arrive(&rg.empty[(fill_no + threadIdx.x) & mask]);    // gate / up slots
  fill_no += 8;
  const int nrt = d / 16, nf = (nrt + pl.d_tps - 1) / pl.d_tps;      // the K slice of W_down with its scales
  for (int f = 0; f < nf; ++f) fu_acquire(rg, c, fill_no + f);
  if (warp == 0) FU_TP(6);
  fu_gemv_fast(c, fill_no, fu_log2(pl.d_tps), nrt, 1, nullptr, true, FusedOut{out, nullptr, d, 0, tag});
  fu_release(rg, fill_no, nf);
  return fill_no + nf;
}

// DE: residual update + pre-FFN norm -> gate / up rows of this CTA's features -> GeGLU -> its K slice of
// the down projection; the partial d-vector goes to the reducers.
__device__ __forceinline__ unsigned fu_phase_ffn(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh, int step,
                                              int layer, unsigned fill_no) {
  const ModelDims& dm = a.dims;
  const FusedRing rg = fu_ring(c);
  const int bar = layer * 5 + 3, d = dm.d, ncols = a.ncols;
  fu_mark(a, c, step, 4000 + layer);
  FU_TP(0);
  const unsigned tag = fu_tag(a, pl, step, layer);
  fu_u64* ll = fu_ll(pl, c, layer);
  const unsigned gf = fill_no;
  fu_acquire(rg, c, gf);
  const float* g_pre = reinterpret_cast<const float*>(fu_slot(rg, gf));
  fu_resid(a, c, ll + pl.ll_o, a.o_slices, tag, g_pre + d, g_pre, c.lw[layer].gmax_pre_ffn, sh.f_prod >= 0, bar);
  FU_TP(2);
  fu_release(rg, gf, 1);
  fill_no = gf + 1;
  const int nf_down = (d / 16 + pl.d_tps - 1) / pl.d_tps;
  if (sh.f_prod >= 0 && ncols == 1 && a.nterms == 3 && sh.f_mk == 1 && pl.round_fills >= 8 && nf_down <= pl.round_fills) {
    fill_no = fu_ffn_fast(a, pl, c, sh, fill_no, ll + pl.ll_fpart + (size_t)sh.f_prod * d, tag, bar);
  } else if (sh.f_prod >= 0) {
    const int ngu = 8 * sh.f_mk, K2 = 64 * sh.f_mk;
    for (int t0 = 0; t0 < ngu; t0 += pl.round_fills) {
      const int nt = min(pl.round_fills, ngu - t0);
      for (int f = 0; f < nt; ++f) fu_acquire(rg, c, fill_no + f);
      if (t0 == 0) FU_TP(5);
      fu_gemv_round(c, fill_no, 1, nt, d / 64, nullptr, false, ncols, a.nterms, FusedOut{nullptr, c.gu, ngu * 16, t0 * 16, tag});
      fu_release(rg, fill_no, nt);
      fill_no += nt;
    }
    FU_TP(3);
    // GeGLU: tiles alternate gate, up; feature p * 16 + row of this CTA's slice
    for (int i = threadIdx.x; i < ncols * K2; i += kDecThreads) {
      const int col = i / K2, f = i - col * K2, p = f >> 4, row = f & 15;
      const float gate = c.gu[((size_t)col * ngu + 2 * p) * 16 + row];
      const float up = c.gu[((size_t)col * ngu + 2 * p + 1) * 16 + row];
      c.act[(size_t)col * K2 + f] = gelu_tanh(gate) * up;
    }
    dec_sync();
    fu_quantize_dynamic(a, c, c.act, K2);
    FU_TP(4);
    const int nrt = d / 16, nf_all = (nrt + pl.d_tps - 1) / pl.d_tps;
    const int rf = pl.round_fills;
    fu_u64* out = ll + pl.ll_fpart + (size_t)sh.f_prod * ncols * d;
    for (int fr = 0; fr < nf_all; fr += rf) {
      const int nf = min(rf, nf_all - fr);
      const int t0 = fr * pl.d_tps, nt = min(nrt - t0, nf * pl.d_tps);
      for (int f = 0; f < nf; ++f) fu_acquire(rg, c, fill_no + f);
      if (fr == 0) FU_TP(6);
      fu_gemv_round(c, fill_no, pl.d_tps, nt, sh.f_mk, nullptr, true, ncols, a.nterms, FusedOut{out, nullptr, d, t0 * 16, tag});
      fu_release(rg, fill_no, nf);
      fill_no += nf;
    }
  }
  FU_ARRIVE();
  return fill_no;
}

// R: this CTA's elements of the FFN output: the sum of the producers' partial vectors, in a fixed order.
__device__ __forceinline__ void fu_phase_reduce(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh, int step,
                                             int layer) {
  const int bar = layer * 5 + 4, d = a.dims.d, ncols = a.ncols;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  fu_mark(a, c, step, 5000 + layer);
  FU_TP(0);
  if (sh.r_n > 0) {
    const unsigned tag = fu_tag(a, pl, step, layer);
    fu_u64* ll = fu_ll(pl, c, layer);
    const int np2 = sh.r_n / 2, groups = (pl.nprod + 31) / 32;
    const int tasks = ncols * np2 * groups;
    float* rs = c.act;
    const fu_u64* src = ll + pl.ll_fpart;
    for (int task = warp; task < tasks; task += kDecWarps) {
      const int grp = task % groups, rest = task / groups, ps = rest % np2, col = rest / np2;
      const int p = grp * 32 + lane;
      float x = 0.f, y = 0.f;
      if (p < pl.nprod) {
        const float2 xy = ll_wait2(c, src + ((size_t)p * ncols + col) * d + sh.r_e0 + 2 * ps, tag);
        x = xy.x;
        y = xy.y;
      }
      x = warp_sum(x);
      y = warp_sum(y);
      if (lane == 0) { rs[task * 2] = x; rs[task * 2 + 1] = y; }
    }
    FU_TP(1);
    dec_sync();
    for (int i = threadIdx.x; i < ncols * sh.r_n; i += kDecThreads) {
      const int col = i / sh.r_n, e = i - col * sh.r_n, ps = e >> 1, which = e & 1;
      float v = 0.f;
      for (int grp = 0; grp < groups; ++grp) v += rs[((col * np2 + ps) * groups + grp) * 2 + which];
      ll_store(ll + pl.ll_f + (size_t)col * d + sh.r_e0 + e, v, tag);
    }
    dec_sync();
  }
  FU_ARRIVE();
}

// H: final residual update + final norm -> this CTA's rows of the LM head (every warp streams its own
// row tiles) -> arg-max, exchanged so that every CTA knows the next token.
__device__ __forceinline__ unsigned fu_phase_head(const DecodeArgs& a, const FusedPlan& pl, FusedCtx& c, const FusedCta& sh, int step,
                                               int sd0, unsigned fill_no) {
  const ModelDims& dm = a.dims;
  const FusedRing rg = fu_ring(c);
  const int L = dm.n_layers, d = dm.d, ktn = d / 64, ncols = a.ncols, nterms = a.nterms;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int cta = blockIdx.x, ncta = gridDim.x;
  int bar = 5 * L;
  fu_mark(a, c, step, 6000);
  FU_TP(0);
  const unsigned tagh = fu_tag(a, pl, step, L);
  float bv[kMaxCols / 2];
  int bi[kMaxCols / 2];
#pragma unroll
  for (int k = 0; k < kMaxCols / 2; ++k) { bv[k] = -INFINITY; bi[k] = 0x7fffffff; }
  float bx = -INFINITY;      // candidates of the upper half-warp in the one-session register path
  int bj = 0x7fffffff;
  {
    const unsigned gf = fill_no;
    fu_acquire(rg, c, gf);
    const float* g_pre = reinterpret_cast<const float*>(fu_slot(rg, gf));
    fu_resid(a, c, fu_ll(pl, c, L - 1) + pl.ll_f, 1, tagh - 1u, g_pre + d, g_pre, a.gmax_final, true, bar);
    FU_TP(2);
    fu_release(rg, gf, 1);
    const unsigned f0 = gf + 1;
    const int nq = ncols * nterms;
    const bool timed = a.trace_pts != nullptr;      // the timeline tool asks where the warps spend the phase
    long long t_wait = 0, t_mma = 0, t_fin = 0;
    // A warp may wait for a slot only while the fill before it in that slot is already the warp's own
    // past (an mbarrier wait tells apart two consecutive phases, not three): with fewer slots than warps
    // only as many warps stream as there are slots.
    const int nstream = min(kDecWarps, c.nslots);
    for (int i = warp; i < sh.h_n && warp < nstream; i += nstream) {
      const unsigned fill = f0 + (unsigned)i;
      const long long t0 = timed ? clock64() : 0;
      fu_acquire(rg, c, fill);
      const long long t1 = timed ? clock64() : 0;
      const unsigned char* base = fu_slot(rg, fill);
      const int4 acc = fu_mma_run(reinterpret_cast<const uint4*>(base), 32, 0, ktn, c.xq, c.xstride, nq, lane);
      const float* scl = reinterpret_cast<const float*>(base + (size_t)ktn * 512);
      const int n0 = (sh.h_t0 + i) * 16;
      long long t2 = 0;
      if (ncols == 1 && nterms == 3) {          // finalised in registers: rows g and g + 8 in the lanes with t == 0
        const float2 v = fu_terms(acc);
        if (timed) t2 = clock64();
        if ((lane & 3) == 0) {
          const int gq = lane >> 2;
          const float cs = c.colscale[0] * (1.0f / 16.0f);
          const float lo = v.x * cs * scl[gq], hi = v.y * cs * scl[gq + 8];
          a.logits[n0 + gq] = lo;
          a.logits[n0 + gq + 8] = hi;
          if ((lane >> 4) == 0) { fu_better(bv[0], bi[0], lo, n0 + gq); fu_better(bv[0], bi[0], hi, n0 + gq + 8); }
          else { fu_better(bx, bj, lo, n0 + gq); fu_better(bx, bj, hi, n0 + gq + 8); }
        }
      } else {
        fu_store_frag(c.red, warp, acc, lane);
        __syncwarp();
        if (timed) t2 = clock64();
#pragma unroll
        for (int k = 0; k < kMaxCols / 2; ++k) {
          const int row = lane & 15, col = (lane >> 4) + 2 * k;
          if (col < ncols) {
            const float v = fu_finalize(c.red, warp, 1, row, col, nterms, c.colscale[col]) * scl[row];
            a.logits[(size_t)col * dm.vocab + n0 + row] = v;
            fu_better(bv[k], bi[k], v, n0 + row);
          }
        }
      }
      t_wait += t1 - t0;
      t_mma += t2 - t1;
      __syncwarp();
      if (lane == 0) mbar_arrive(&rg.empty[fill & rg.mask]);
      if (timed) t_fin += clock64() - t2;
    }
    fill_no = f0 + (unsigned)sh.h_n;
    FU_TP(3);
    if (timed && threadIdx.x == 0) {                // where warp 0 spent the head phase (cycles)
      long long* q = a.trace_pts + ((size_t)(bar + 1) * gridDim.x + blockIdx.x) * 8;
      q[4] = t_wait; q[5] = t_mma; q[6] = t_fin;
    }
  }
  if (ncols == 1 && nterms == 3) {       // hand the upper half-warp's candidate to the lane 16 below it
    const float ov = __shfl_down_sync(0xffffffffu, bx, 16);
    const int oi = __shfl_down_sync(0xffffffffu, bj, 16);
    if (lane < 16) fu_better(bv[0], bi[0], ov, oi);
  }
  // CTA-level arg-max per session, published as (value bits, index)
  float* sv = c.scratch;                                  // [16]
  int* si = reinterpret_cast<int*>(c.scratch + 16);       // [16]
  fu_u64* amax = c.ll_base + (size_t)(step & 1) * pl.ll_words + pl.ll_amax;
  for (int col = 0; col < ncols; ++col) {
    const int k = col >> 1;
    float v = -INFINITY;
    int ix = 0x7fffffff;
#pragma unroll
    for (int kk = 0; kk < kMaxCols / 2; ++kk)
      if (kk == k && (lane >> 4) == (col & 1)) { v = bv[kk]; ix = bi[kk]; }
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, v, o);
      int oi = __shfl_xor_sync(0xffffffffu, ix, o);
      fu_better(v, ix, ov, oi);
    }
    dec_sync();
    if (lane == 0) { sv[warp] = v; si[warp] = ix; }
    dec_sync();
    if (warp == 0) {
      float v2 = lane < kDecWarps ? sv[lane] : -INFINITY;
      int i2 = lane < kDecWarps ? si[lane] : 0x7fffffff;
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v2, o);
        int oi = __shfl_xor_sync(0xffffffffu, i2, o);
        fu_better(v2, i2, ov, oi);
      }
      if (lane == 0) {
        __threadfence();            // this CTA's cache rows of the step are visible before its candidate is
        ll_store(amax + ((size_t)cta * ncols + col) * 2, v2, tagh);
        ll_store_bits(amax + ((size_t)cta * ncols + col) * 2 + 1, (unsigned)i2, tagh);
      }
    }
  }
  FU_ARRIVE();
  // ---- every CTA reads all candidates: the token of the next step needs no further exchange
  ++bar;
  fu_mark(a, c, step, 7000);
  FU_TP(0);
  if (warp == 0) {
    for (int col = 0; col < ncols; ++col) {
      float v = -INFINITY;
      int ix = 0x7fffffff;
      for (int ct = lane; ct < ncta; ct += 32) {
        const ulonglong2 w = ll_wait2w(c, amax + ((size_t)ct * ncols + col) * 2, tagh);
        fu_better(v, ix, ll_val(w.x), (int)(unsigned)w.y);
      }
      for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, ix, o);
        fu_better(v, ix, ov, oi);
      }
      if (lane == 0) {
        if (ix == 0x7fffffff) ix = 0;
        if (a.advance) c.tok[col] = ix;
        if (cta == 0) {
          a.st->out_token[col] = ix;
          const int sd = sd0 + step;
          if (a.step_tokens && sd < a.step_capacity) a.step_tokens[(size_t)sd * ncols + col] = ix;
          if (a.advance) {
            a.st->token[col] = ix;
            a.st->pos[col] = c.pos0[col] + step + 1;
          }
        }
      }
    }
    if (lane == 0) {
      if (cta == 0) a.st->steps_done = sd0 + step + 1;
      FU_TP(1);
      __threadfence();              // candidates of every CTA observed: their cache rows may be fetched now
      *c.step_ready = step + 2;
    }
  }
  FU_ARRIVE();
  dec_sync();
  return fill_no;
}

// ------------------------------------------------------------------ the kernel

template <typename T, int HD, int G>
__global__ void __launch_bounds__(kFuThreads, 1)
decode_fused_kernel(const __grid_constant__ DecodeArgs a, const __grid_constant__ FusedPlan pl, fu_u64* ll_base, int nsteps) {
  extern __shared__ __align__(128) unsigned char fsm_raw[];
  __shared__ FusedCtx c;
  __shared__ FusedCta sh;
  const ModelDims& dm = a.dims;
  if (threadIdx.x == 0) {
    fu_carve(fsm_raw, dm, a.ncols, a.nterms, pl, c);
    c.err = &a.st->err;
    c.gave_up = a.st->gave_up;
    c.ll_base = ll_base;
    c.progress = a.progress;
    c.fill_log = (a.trace && blockIdx.x == (unsigned)a.advance * 0u + 0u) ? a.trace : nullptr;
    c.where = 0;
    sh = fu_cta_share(a, pl, blockIdx.x, gridDim.x);
    for (int i = 0; i < pl.nslots; ++i) { mbar_init(&c.full[i], 1); mbar_init(&c.empty[i], 1); }
    *c.dead = 0;
    *c.step_ready = 1;
    for (int col = 0; col < kMaxCols; ++col) {
      c.pos0[col] = col < a.ncols ? __ldcg(&a.st->pos[col]) : 0;
      c.tok[col] = col < a.ncols ? __ldcg(&a.st->token[col]) : 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dm.n_layers; i += kFuThreads) {
    c.lw[i] = a.layers[i];
    c.lkv[i] = a.kv[i];
    c.cl[i] = a.chained[i];
  }
  __syncthreads();

  if (threadIdx.x >= kDecThreads) {       // ---- producer warp
    fused_producer<T>(a, pl, c, sh, nsteps);
    return;
  }
  unsigned fill_no = 0;                   // fills consumed so far (the same in every compute thread)
  const int sd0 = (blockIdx.x == 0 && threadIdx.x == 0) ? __ldcg(&a.st->steps_done) : 0;
  for (int step = 0; step < nsteps; ++step) {
    if (threadIdx.x < a.ncols) {
      const int p = c.pos0[threadIdx.x] + step;
      if (p < 0 || p >= dm.max_ctx) atomicExch(c.err, (int)kDevBadPosition);
    }
    for (int layer = 0; layer < dm.n_layers; ++layer) {
      fill_no = fu_phase_qkv(a, pl, c, sh, step, layer, fill_no);
      {
        const int bar = layer * 5 + 1;
        fu_mark(a, c, step, 2000 + layer);
        const int nsp = c.lw[layer].is_global ? a.n_attn_splits_global : a.n_attn_splits_local;
        FU_TP(0);
        if ((int)blockIdx.x < a.ncols * dm.hkv * nsp)
          fill_no = fu_attention<T, HD, G>(a, pl, c, layer, step, fill_no, fu_ll(pl, c, layer), fu_tag(a, pl, step, layer), bar);
        else
          FU_ARRIVE();
      }
      fill_no = fu_phase_oproj(a, pl, c, sh, step, layer, fill_no);
      fill_no = fu_phase_ffn(a, pl, c, sh, step, layer, fill_no);
      fu_phase_reduce(a, pl, c, sh, step, layer);
    }
    fill_no = fu_phase_head(a, pl, c, sh, step, sd0, fill_no);
  }
}

// Host-side selection of the instantiation for a model.
inline const void* decode_fused_kernel_for(const ModelDims& d) {
  const int G = d.hq / d.hkv;
#define B2_PICK_G(T, HD)                                                                  \
  (G == 1 ? (const void*)decode_fused_kernel<T, HD, 1>                                    \
          : G == 2 ? (const void*)decode_fused_kernel<T, HD, 2> : (const void*)decode_fused_kernel<T, HD, 4>)
#define B2_PICK_HD(T)                                                                     \
  (d.hd == 32 ? B2_PICK_G(T, 32) : d.hd == 64 ? B2_PICK_G(T, 64) : d.hd == 128 ? B2_PICK_G(T, 128) : B2_PICK_G(T, 256))
  return d.kv_dtype == 0 ? B2_PICK_HD(float) : B2_PICK_HD(__nv_bfloat16);
#undef B2_PICK_HD
#undef B2_PICK_G
}

}  // namespace b200lm

// Int4 weight-only GEMM for prefill with the WEIGHTS as the tensor-core "A"
// operand held in tensor memory:
//
//   D[weight row][token] = sum_k W[row][k] * X[token][k]
//
// The int4 weight tile is expanded to bf16 in registers and written straight
// into TMEM (tcgen05.st); the activations are the K-major "B" operand, staged
// in shared memory by TMA.  Compared with expanding the weights into a shared
// memory tile this removes, per 64-wide k block, 16 KB of shared-memory writes
// and a 4 KB operand read per MMA, which is what bounded the shared-memory
// variant (an M128 N128 K16 MMA reading both operands from shared memory
// needs the full 128 B/clk of the SM by itself).
//
// The kernel is persistent: one CTA per SM walks a static list of output tiles
// (128 weight rows x 256 tokens x one K split).  Lane i of the accumulator is
// weight row i, so the per-channel scale is one scalar per epilogue thread and
// a warp's store covers 32 consecutive output features of one token.  The 16
// epilogue warps first pull the whole accumulator into registers (64 values
// per thread) and hand it back, so the scaling / GeGLU and the global stores
// of one tile run under the main loop of the next.
//
// Warp roles: 0 = TMA producer, 1 = TMEM owner + MMA issue, 2..5 = int4
// expansion, 6..21 = epilogue.
//
// TMEM columns: [0, NTOK) accumulator, then one slot of 32 columns per pipeline
// stage holding one expanded 128 x 64 weight tile each.
#pragma once
#include "prefill_ops.cuh"

namespace b200lm {

constexpr int kTsStages = 5;
constexpr int kTsRows = 128;                        // weight rows per tile
constexpr int kTsTok = 256;                         // tokens per tile
constexpr int kTsAcols = 32;                        // TMEM columns of one expanded 128 x 64 weight tile
// Warps per role and token width: narrow tiles give the warps their smaller epilogue does not need to the
// int4 expansion (two warps per 32 accumulator lanes, half a weight row each).  The epilogue needs one warp
// per 32 lanes x 64 token columns.
__host__ __device__ constexpr int ts_deq_warps(int ntok) { return ntok >= 256 ? 4 : 8; }
__host__ __device__ constexpr int ts_epi_warps(int ntok) { return 4 * (ntok / 64); }
__host__ __device__ constexpr int ts_threads(int ntok) { return 64 + 32 * (ts_deq_warps(ntok) + ts_epi_warps(ntok)); }
constexpr int kTsStageX = kTsTok * kGemmBK * 2;     // activation tile, 32 KB
constexpr int kTsTmemCols = 512;
// Pipeline depth per token width.  A stage holds one k block: NTOK x 64 activations and 4 KB of int4 weights.
// The weights come from HBM, so what bounds a narrow tile is the bytes in flight per SM (stages x 4 KB over a
// round trip of a few microseconds), not the MMA: narrow tiles spend the shared memory and the tensor-memory
// columns the accumulator leaves on more stages.
__host__ __device__ constexpr int ts_stages(int ntok) { return ntok >= 256 ? kTsStages : ntok == 128 ? 8 : 12; }
__host__ __device__ constexpr int ts_smem(int ntok) { return ts_stages(ntok) * (ntok * kGemmBK * 2 + kGemmStageQ) + 1024 + 512; }
static_assert(256 + ts_stages(256) * kTsAcols <= kTsTmemCols && 128 + ts_stages(128) * kTsAcols <= kTsTmemCols &&
                  64 + ts_stages(64) * kTsAcols <= kTsTmemCols, "TMEM budget");
static_assert(ts_smem(256) <= 227 * 1024 && ts_smem(128) <= 227 * 1024 && ts_smem(64) <= 227 * 1024, "shared memory budget");

// A operand in tensor memory, B through a shared-memory descriptor
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float gelu_tanh_fast(float x) {
  const float c = 0.7978845608028654f;
  float y = c * (x + 0.044715f * x * x * x), t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(y));
  return 0.5f * x * (1.0f + t);
}

// Tile list: tile = (ks * t_tiles + t_tile) * n_tiles + n_tile; CTA c takes
// tiles c, c + gridDim.x, ...
struct TsTile {
  int n_tile, t_tile, ks;
};
__device__ __forceinline__ TsTile ts_tile(int tile, int n_tiles, int t_tiles) {
  TsTile t;
  t.n_tile = tile % n_tiles;
  int r = tile / n_tiles;
  t.t_tile = r % t_tiles;
  t.ks = r / t_tiles;
  return t;
}

// EPI 0: fp32 partials outF[ks][T][N].  EPI 1: GeGLU; tile rows alternate
// gate (even) and up (odd) rows of one ffn feature, output bf16 outB[T][N/2].
//
// NTOK is the token width of a tile (the N of the MMA): 256 for prefill; 128 or 64 when the whole GEMM has
// no more token rows than that (the wide decode step, short prompts), which cuts the activation bytes every
// CTA re-reads per k block and the MMA time in proportion.  tmX must have a box of min(NTOK, 128) rows.
template <int EPI, int NTOK>
__global__ void __launch_bounds__(ts_threads(NTOK), 1)
gemm_w4_ts_kernel(const __grid_constant__ CUtensorMap tmX, GemmArgs g) {
  constexpr int kTsDeqWarps = ts_deq_warps(NTOK), kTsEpiWarps = ts_epi_warps(NTOK);
  constexpr int S = ts_stages(NTOK);
  constexpr int kStageX = NTOK * kGemmBK * 2;       // activation tile of one stage
  constexpr uint32_t kStageTx = NTOK * kGemmBK * 2 + kGemmStageQ;
  extern __shared__ unsigned char gsm_raw[];
  unsigned char* gsm = reinterpret_cast<unsigned char*>(((uintptr_t)gsm_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sX = gsm;
  unsigned char* sQ = gsm + S * kStageX;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sQ + S * kGemmStageQ);
  uint64_t* full_bar = bars;              // [S] TMA bytes landed
  uint64_t* deq_bar = bars + S;           // [S] expanded weights are in TMEM
  uint64_t* empty_bar = bars + 2 * S;     // [S] MMA finished with the stage (shared memory and TMEM slot)
  uint64_t* acc_full = bars + 3 * S;      // accumulator complete
  uint64_t* acc_empty = bars + 3 * S + 1; // accumulator read out by the epilogue warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = g.K / kGemmBK;
  const int nkb = KB / g.ksplit;
  const int n_tiles = (g.N + kTsRows - 1) / kTsRows;
  const int t_tiles = (g.T + NTOK - 1) / NTOK;
  const int total = n_tiles * t_tiles * g.ksplit;
  const int my_tiles = (int)blockIdx.x < total ? (total - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&deq_bar[s], kTsDeqWarps);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, kTsEpiWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTsTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_w = tmem_base + NTOK;         // weight slots follow the accumulator columns
  // barriers and TMEM are set up: from here on the kernel reads what its predecessor wrote
  pdl_wait();
  pdl_launch_dependents();

  if (warp == 0) {
    // ---- producer: one elected lane issues the copies, the warp stays together
    int it = 0;
    bool ok = true;
    for (int li = 0; li < my_tiles && ok; ++li) {
      const TsTile tl = ts_tile(blockIdx.x + li * gridDim.x, n_tiles, t_tiles);
      const uint8_t* wtile = g.w + ((size_t)tl.n_tile * KB + (size_t)tl.ks * nkb) * kGemmStageQ;
      for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
        const int s = it % S, n = it / S;
        if (n > 0) ok = mbar_wait(&empty_bar[s], (n - 1) & 1, g.err);
        if (ok && lane == 0) {
          mbar_arrive_expect_tx(&full_bar[s], kStageTx);
#pragma unroll
          for (int h = 0; h < (NTOK + 127) / 128; ++h)
            tma_load_2d(sX + s * kStageX + h * 128 * 128, &tmX, (tl.ks * nkb + kb) * kGemmBK,
                        tl.t_tile * NTOK + h * 128, &full_bar[s]);
          bulk_load_1d(sQ + s * kGemmStageQ, wtile + (size_t)kb * kGemmStageQ, kGemmStageQ, &full_bar[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue
    const uint32_t idesc = umma_idesc_bf16(kTsRows, NTOK);
    int it = 0;
    bool ok = true;
    for (int li = 0; li < my_tiles && ok; ++li) {
      if (li > 0) ok = mbar_wait(acc_empty, (li - 1) & 1, g.err);
      tc_fence_after();
      for (int kb = 0; kb < nkb && ok; ++kb, ++it) {
        const int s = it % S, n = it / S;
        ok = mbar_wait(&full_bar[s], n & 1, g.err) && mbar_wait(&deq_bar[s], n & 1, g.err);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) {
          const uint64_t xd = umma_desc_sw128(smem_u32(sX + s * kStageX));
#pragma unroll
          for (int k = 0; k < kGemmBK / 16; ++k)   // 16 bf16 along K per MMA: 8 TMEM columns, 32 bytes of X
            umma_bf16_ts(tmem_base, tmem_w + s * kTsAcols + k * 8, xd + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
          umma_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (ok && lane == 0) umma_commit(acc_full);
      __syncwarp();
    }
  } else if (warp < 2 + kTsDeqWarps) {
    // ---- int4 -> bf16 expansion into TMEM: this thread does the 64 k (32 columns) of its weight row, or one
    // half of them when two warps share the 32 lanes
    const int quarter = warp & 3;                  // TMEM lanes 32*quarter .. +31 belong to this warp
    constexpr int kHalves = 8 / kTsDeqWarps;       // halves of a row per thread: 2 with four warps, 1 with eight
    const int half0 = kTsDeqWarps == 8 ? (warp - 2) >> 2 : 0;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int iters = my_tiles * nkb;
    const __nv_bfloat162 bias = __float2bfloat162_rn(136.0f);
    bool ok = true;
    for (int it = 0; it < iters && ok; ++it) {
      const int s = it % S, n = it / S;
      ok = mbar_wait(&full_bar[s], n & 1, g.err);
      if (ok && n > 0) ok = mbar_wait(&empty_bar[s], (n - 1) & 1, g.err);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int hh = 0; hh < kHalves; ++hh) {
        const int half = half0 + hh;
        const uint4 q = *reinterpret_cast<const uint4*>(sQ + s * kGemmStageQ + row * 32 + half * 16);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint32_t v = ((qw[j] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;   // bf16(128 + nibble) pairs
            __nv_bfloat162 h = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&v), bias);
            r[j * 4 + i] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
        tmem_st16(tmem_w + lane_base + s * kTsAcols + half * 16, r);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&deq_bar[s]);
    }
  } else {
    // ---- epilogue: this warp takes 64 token columns of its 32 weight rows
    const int quarter = warp & 3;
    const int second = (warp - 2 - kTsDeqWarps) >> 2;      // 0..3
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = true;
    for (int li = 0; li < my_tiles && ok; ++li) {
      const TsTile tl = ts_tile(blockIdx.x + li * gridDim.x, n_tiles, t_tiles);
      ok = mbar_wait(acc_full, li & 1, g.err);
      if (!ok) break;
      tc_fence_after();
      const int c0 = second * 64;
      const int t0 = tl.t_tile * NTOK + c0;
      uint32_t v0[32], v1[32];
      if (c0 < NTOK) {
        tmem_ld32(tmem_base + lane_base + c0, v0);
        tmem_ld32(tmem_base + lane_base + c0 + 32, v1);
      }
      // the accumulator is in registers: hand it back before the stores
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty);
      if (c0 >= NTOK) continue;                      // a narrow tile has no columns for this warp
      const float sc = g.wscale[tl.n_tile * kTsRows + row];
      if constexpr (EPI == 0) {
        const int nrow = tl.n_tile * kTsRows + row;
        if (nrow < g.N) {
          float* dst = g.outF + ((size_t)tl.ks * g.T + t0) * g.N + nrow;
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (t0 + c < g.T) dst[(size_t)c * g.N] = __uint_as_float(v0[c]) * sc;
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (t0 + 32 + c < g.T) dst[(size_t)(32 + c) * g.N] = __uint_as_float(v1[c]) * sc;
        }
      } else {
        const int F = g.N / 2;
        const int f = tl.n_tile * (kTsRows / 2) + (row >> 1);
        const bool odd = lane & 1;
        __nv_bfloat16* dst = g.outB + (size_t)(t0 + (odd ? 1 : 0)) * F + f;
        const int tlim = g.T - t0 - (odd ? 1 : 0);          // columns c (even) with c < tlim are stored
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float a = __uint_as_float(v0[c]) * sc, bb = __uint_as_float(v0[c + 1]) * sc;
          float got = __shfl_xor_sync(0xffffffffu, odd ? a : bb, 1);
          float gate = odd ? got : a, up = odd ? bb : got;
          if (c < tlim && f < F) dst[(size_t)c * F] = __float2bfloat16(gelu_tanh_fast(gate) * up);
        }
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float a = __uint_as_float(v1[c]) * sc, bb = __uint_as_float(v1[c + 1]) * sc;
          float got = __shfl_xor_sync(0xffffffffu, odd ? a : bb, 1);
          float gate = odd ? got : a, up = odd ? bb : got;
          if (32 + c < tlim && f < F) dst[(size_t)(32 + c) * F] = __float2bfloat16(gelu_tanh_fast(gate) * up);
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
    tmem_dealloc(tmem_base, kTsTmemCols);
  }
}

}  // namespace b200lm

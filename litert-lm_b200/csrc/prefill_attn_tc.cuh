// Prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One CTA owns a 128-row query tile of one kv head: 128 / G consecutive tokens
// times the G query heads of the group (GQA packing: every K/V tile is loaded
// once for all heads that share it).  Keys are walked in tiles of 64:
//
//   S  = Q K^T        tcgen05.mma  M128 N64  K=hd   (Q, K tiles by TMA, K-major)
//   P  = exp(S - B)   softmax warps: tcgen05.ld, mask, exp2, bf16 -> shared memory
//   O += P V          tcgen05.mma  M128 N=hd K64    (V comes from a TRANSPOSED bf16
//                                                    copy of the cache, so it is K-major too)
//
// Q and K are RMS-normalised per head before the product, so every score obeys
// |s| <= B = sqrt(hd) max|g_q| max|g_k|.  The softmax is therefore shifted by the
// constant B instead of a running maximum: exact by shift invariance, no
// overflow, and the O accumulator in tensor memory never has to be rescaled.
// (Layers whose bound is too large for fp32 exponents use the CUDA-core kernel.)
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer (owns TMEM), warps 2-5
// softmax + epilogue (one thread per query row = TMEM lane).  K/V tiles are
// double buffered.  All waits are bounded.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "prefill_ops.cuh"

namespace b200lm {

constexpr int kFaThreads = 192;
constexpr int kFaBN = 64;            // keys per tile
constexpr float kFaMaxBound = 40.0f; // exp(-2 * 40) is still a normal fp32 number

template <int HD>
struct FaSmem {
  static constexpr int kQ = 128 * HD * 2;            // 128 rows, HD/64 sub-tiles of 128 B rows
  static constexpr int kK = kFaBN * HD * 2;          // per stage
  static constexpr int kV = HD * kFaBN * 2;          // per stage: HD rows of 64 keys
  static constexpr int kP = 128 * kFaBN * 2;
  static constexpr int kTotal = kQ + 2 * kK + 2 * kV + kP + 256 + 1024;
};

struct FaArgs {
  int T, start, hq, hkv, window, is_global;
  const int* page_table;
  __nv_bfloat16* out;      // [T][hq][hd]
  float bound;             // B
  int* err;
};

template <int HD>
__global__ void __launch_bounds__(kFaThreads, 1)
flash_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmVt, FaArgs g) {
  extern __shared__ unsigned char fa_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>(((uintptr_t)fa_raw + 1023) & ~(uintptr_t)1023);
  using L = FaSmem<HD>;
  unsigned char* sQ = sm;
  unsigned char* sK = sQ + L::kQ;
  unsigned char* sV = sK + 2 * L::kK;
  unsigned char* sP = sV + 2 * L::kV;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + L::kP);
  uint64_t* q_full = bars;            // Q tile landed
  uint64_t* kv_full = bars + 1;       // [2]
  uint64_t* kv_empty = bars + 3;      // [2] both MMAs of the tile are done with the stage
  uint64_t* s_full = bars + 5;        // S = Q K^T complete
  uint64_t* s_free = bars + 6;        // softmax has read S
  uint64_t* p_full = bars + 7;        // P written to shared memory
  uint64_t* p_empty = bars + 8;       // P V has consumed P
  uint64_t* o_full = bars + 9;        // all MMAs complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = g.hq / g.hkv;
  const int TT = 128 / G;                       // tokens per tile
  const int t0 = blockIdx.x * TT, kvh = blockIdx.y;
  constexpr int KB = HD / 64;                   // 64-column blocks of the head dimension
  constexpr uint32_t kTmemCols = HD + kFaBN <= 256 ? 256 : 512;
  constexpr uint32_t kSCol = 0, kOCol = kFaBN;

  // key range of this query tile
  const int qpos_min = g.start + t0;
  const int qpos_max = g.start + min(t0 + TT, g.T) - 1;
  const int k_lo = g.is_global ? 0 : max(0, qpos_min - g.window + 1);
  const int tile_lo = k_lo / kFaBN, tile_hi = qpos_max / kFaBN;
  const int ntiles = tile_hi - tile_lo + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(s_full, 1);
    mbar_init(s_free, 128);
    mbar_init(p_full, 128);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      // Q tile: KB boxes of 64 columns x (G heads x TT tokens) rows
      mbar_arrive_expect_tx(q_full, L::kQ);
      for (int kb = 0; kb < KB; ++kb) {
        asm volatile(
            "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
            ::"r"(smem_u32(sQ + kb * 128 * 128)), "l"(&tmQ), "r"(kb * 64), "r"(kvh * G), "r"(t0), "r"(smem_u32(q_full))
            : "memory");
      }
      for (int j = 0; j < ntiles; ++j) {
        const int s = j & 1, n = j >> 1;
        if (n > 0 && !mbar_wait(&kv_empty[s], (n - 1) & 1, g.err)) break;
        const int key0 = (tile_lo + j) * kFaBN;
        const int page = g.page_table[key0 / kPage], slot0 = key0 % kPage;
        mbar_arrive_expect_tx(&kv_full[s], L::kK + L::kV);
        const int krow = (page * g.hkv + kvh) * kPage + slot0;
        for (int kb = 0; kb < KB; ++kb)
          tma_load_2d(sK + s * L::kK + kb * kFaBN * 128, &tmK, kb * 64, krow, &kv_full[s]);
        tma_load_2d(sV + s * L::kV, &tmVt, slot0, (page * g.hkv + kvh) * HD, &kv_full[s]);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc_bf16(128, kFaBN);
      const uint32_t idesc_o = umma_idesc_bf16(128, HD);
      bool ok = mbar_wait(q_full, 0, g.err);
      for (int j = 0; j < ntiles && ok; ++j) {
        const int s = j & 1, n = j >> 1;
        ok = mbar_wait(&kv_full[s], n & 1, g.err);
        if (ok && j > 0) ok = mbar_wait(s_free, (j - 1) & 1, g.err);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
          const uint64_t qd = umma_desc_sw128(smem_u32(sQ + kb * 128 * 128));
          const uint64_t kd = umma_desc_sw128(smem_u32(sK + s * L::kK + kb * kFaBN * 128));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + kSCol, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
        }
        umma_commit(s_full);
        ok = mbar_wait(p_full, j & 1, g.err);
        if (!ok) break;
        tc_fence_after();
        const uint64_t pd = umma_desc_sw128(smem_u32(sP));
        const uint64_t vd = umma_desc_sw128(smem_u32(sV + s * L::kV));
#pragma unroll
        for (int k = 0; k < kFaBN / 16; ++k)
          umma_bf16(tmem + kOCol, pd + (uint64_t)(k * 2), vd + (uint64_t)(k * 2), idesc_o, (j | k) ? 1u : 0u);
        umma_commit(&kv_empty[s]);
        umma_commit(p_empty);
      }
      umma_commit(o_full);
    }
  } else {
    // ---- softmax warps: thread = one query row = one TMEM lane
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                 // row of the tile: token r / G, head r % G
    const int tok = t0 + r / G;
    const int qpos = g.start + tok;
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const float log2e = 1.4426950408889634f;
    const float shift = g.bound * log2e;
    float lsum = 0.f;
    bool ok = true;
    for (int j = 0; j < ntiles && ok; ++j) {
      ok = mbar_wait(s_full, j & 1, g.err);
      if (!ok) break;
      tc_fence_after();
      uint32_t v0[32], v1[32];
      tmem_ld32(lane_addr + kSCol, v0);
      tmem_ld32(lane_addr + kSCol + 32, v1);
      tc_fence_before();
      mbar_arrive(s_free);                              // S may be overwritten by the next Q K^T
      const int key0 = (tile_lo + j) * kFaBN;
      uint32_t packed[32];
#pragma unroll
      for (int c = 0; c < 64; c += 2) {
        float p[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int kpos = key0 + c + e;
          const float sv = __uint_as_float(c + e < 32 ? v0[(c + e) & 31] : v1[(c + e) & 31]);
          const bool open = kpos <= qpos && (g.is_global || qpos - kpos < g.window);
          p[e] = open ? exp2f(sv * log2e - shift) : 0.f;
        }
        __nv_bfloat162 h = __floats2bfloat162_rn(p[0], p[1]);
        // sum what the tensor core will actually multiply (the rounded values)
        lsum += __low2float(h) + __high2float(h);
        packed[c >> 1] = *reinterpret_cast<uint32_t*>(&h);
      }
      if (j > 0) ok = mbar_wait(p_empty, (j - 1) & 1, g.err);   // P V of the previous tile has read P
      if (!ok) break;
      unsigned char* prow = sP + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int chunk = c ^ (r & 7);
        *reinterpret_cast<uint4*>(prow + chunk * 16) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      }
      fence_async_smem();
      mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> bf16
    if (ok && mbar_wait(o_full, 0, g.err)) {
      tc_fence_after();
      const float inv = lsum > 0.f ? 1.0f / lsum : 0.f;
      const int head = kvh * G + (r % G);
      __nv_bfloat16* dst = g.out + ((size_t)tok * g.hq + head) * HD;
#pragma unroll 1
      for (int cb = 0; cb < HD / 32; ++cb) {
        uint32_t o[32];
        tmem_ld32(lane_addr + kOCol + cb * 32, o);
        if (tok < g.T) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            uint4 w;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
            w.x = *reinterpret_cast<uint32_t*>(&h0); w.y = *reinterpret_cast<uint32_t*>(&h1);
            w.z = *reinterpret_cast<uint32_t*>(&h2); w.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + cb * 32 + c) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*reinterpret_cast<volatile int*>(g.err) == (int)kDevBarrierTimeout) {
    for (int i = 0; i < 2000; ++i) __nanosleep(100);   // let copies in flight land before the CTA retires
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
}

}  // namespace b200lm

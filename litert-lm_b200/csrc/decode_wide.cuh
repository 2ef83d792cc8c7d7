// Wide lockstep decode: one greedy step for MANY sessions at once, with the projections on the
// tensor-core int4 GEMM of the prefill path (the sessions' current tokens are the GEMM's token rows)
// and one attention CTA per (session, kv head) over that session's own pages.  The weights stream
// once per step for the whole group, which is what a group of more sessions than the GEMV kernels
// carry (kMaxCols) needs.  Activations are bf16 as in prefill.
//
// This file holds the two small kernels the step adds to the prefill kernels; the step itself is
// Executor::launch_wide_steps.
#pragma once
#include "prefill_ops.cuh"

namespace b200lm {

constexpr int kWideMax = 128;          // sessions of one wide step (half a token tile of the GEMM)
constexpr int kWideArgThreads = 1024;

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

/*
 * b200lm_ops.h — operator-level C ABI of libb200lm.so.
 *
 * The reference hides its operators inside compiled_model_.Run
 * (runtime/executor/llm_litert_compiled_model_executor.cc:271,407,522), so these
 * entry points have no one-to-one reference symbol; each names the step of
 * that opaque graph it stands for.  They exist for the operator parity tests
 * and for the attention / GEMM micro-benchmarks.  All pointers are HOST
 * memory unless a name says "dev"; the calls copy in, run the kernel, copy out.
 * Same status-code and error-string conventions as b200lm.h.
 */
#ifndef B200LM_OPS_H_
#define B200LM_OPS_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Host-only repacks of canonical int4 rows ([n][k/2] bytes, element 2j in the
 * low nibble) into the decode layout (16x64 mma tiles) and the tensor-core GEMM
 * layout (128-row x 64-k blocks).  out must hold n_pad*k/2 bytes, n_pad = n
 * rounded up to 16 (W4T) or 128 (W4G).  No GPU needed. */
int B200LmOps_RepackW4T(const uint8_t* packed, int64_t n, int64_t k, uint8_t* out, char** err);
int B200LmOps_RepackW4G(const uint8_t* packed, int64_t n, int64_t k, uint8_t* out, char** err);

/* Bit-exact unpack gate: uploads canonical rows, repacks, and has the GPU
 * expand the decode layout back to int8 [n][k] with the same device function
 * the GEMV uses to address its tiles. */
int B200LmOps_UnpackW4(int32_t device, const uint8_t* packed, int64_t n, int64_t k, int8_t* out, char** err);

/* Decode GEMV (the int4 fully-connected op at batch 1..4):
 * y[c][n] = scale[n] * sum_k W[n][k] x[c][k], x quantised to `nterms` int8 terms. */
int B200LmOps_GemvW4(int32_t device, const uint8_t* packed, const float* scale, int64_t n, int64_t k,
                     const float* x, int32_t ncols, int32_t nterms, int32_t kslices, float* y, char** err);

/* Prefill GEMM (the int4 fully-connected op over T tokens), bf16 activations:
 * mode B200LM_GEMM_CHECK or B200LM_GEMM_TCGEN05.  out is [T][n] fp32.
 * repeat > 1 re-runs the kernel and, when ms_out != NULL, returns the mean
 * device time per run in milliseconds (CUDA events). */
int B200LmOps_GemmW4(int32_t device, int32_t mode, const uint8_t* packed, const float* scale, int64_t n,
                     int64_t k, const float* a, int32_t t, int32_t ksplit, int32_t repeat, float* out,
                     float* ms_out, char** err);

/* Fused gate/up GEMM + GeGLU: out[T][ffn] = gelu_tanh(A Wg^T) * (A Wu^T). */
int B200LmOps_GemmGegluW4(int32_t device, int32_t mode, const uint8_t* gate_packed, const float* gate_scale,
                          const uint8_t* up_packed, const float* up_scale, int64_t ffn, int64_t k,
                          const float* a, int32_t t, float* out, char** err);

/* Attention against a paged cache built from k, v [S][hkv][hd] (fp32 host,
 * stored as fp32 or bf16 pages): queries q [T][hq][hd] at positions
 * qpos0 + i (or all at qpos0 + T - 1 ... see below), causal, optional window
 * (window <= 0: global).  No QK-norm, no RoPE (raw q/k, as the attention-only
 * micro-benchmark specifies).  nsplit > 1 runs the split-KV decode kernel plus
 * the log-sum-exp combine (T is then a batch of independent single-token
 * queries all at position S - 1); nsplit == 1 runs the prefill kernel.
 * kv_bf16: bit 0 = bf16 pages (else fp32); bit 1 (decode only) = every query
 * gets its own physical copy of the cache and its own page table, i.e. a
 * batch of independent sequences instead of queries sharing one cache; bit 2
 * (decode only) = the streaming kernel of the wide decode step
 * (csrc/decode_wide.cuh: K / V in blocks of 16 positions by bulk async copies
 * into a shared-memory ring) instead of the register-resident split kernel
 * (two keys in flight per warp). */
int B200LmOps_Attention(int32_t device, const float* q, const float* k, const float* v, int32_t t, int32_t s,
                        int32_t hq, int32_t hkv, int32_t hd, int32_t qpos0, int32_t window,
                        int32_t kv_bf16, int32_t nsplit, int32_t repeat, float* out, float* ms_out,
                        char** err);

/* Causal self-attention over s tokens on the tensor cores (the prefill flash
 * kernel of the executor: TMA-staged K/V tiles, tcgen05 MMA with TMEM
 * accumulators, GQA-packed query tiles).  q [s][hq][hd], k, v [s][hkv][hd] fp32
 * host, rounded to bf16 on the device; scores are q.k / sqrt(hd); window <= 0
 * means global.  hd must be 128 or 256.  The kernel shifts the softmax by a
 * constant bound on the scores instead of a running maximum; inputs whose
 * scores could exceed 40 are rejected with FailedPrecondition.  repeat > 1
 * re-runs the kernel and returns the mean device time in ms_out. */
int B200LmOps_AttentionPrefillTc(int32_t device, const float* q, const float* k, const float* v, int32_t s,
                                 int32_t hq, int32_t hkv, int32_t hd, int32_t window, int32_t repeat, float* out,
                                 float* ms_out, char** err);

/* Split-KV decode attention that allocates nothing.  It has no counterpart in
 * the reference.  It is for callers that may not allocate device memory when
 * they call in: code running inside another runtime's execution callback, a
 * serving loop that bans allocator calls once it is warm, or a process whose
 * GPU memory was handed out completely at start-up.  The ordinary entry point
 * above allocates scratch for the per-split partial results on every call;
 * this one keeps them (with the query positions and an error word) in one
 * fixed 8 MiB device array that is part of the library image, so every GPU
 * that loads the library holds those 8 MiB until the process ends.
 *
 * All pointers are DEVICE memory owned by the caller:
 *   q_dev          [batch] rows of (hq + 2*hkv)*hd floats, the layout of a fused
 *                  QKV projection; only the first hq*hd floats of a row are read
 *   k_pages_dev,   paged cache [page][hkv][256][hd], fp32 or bf16 (kv_bf16),
 *   v_pages_dev    already holding positions 0 .. s-1
 *   page_table_dev [ceil(s/256)] physical page of each logical page
 *   out_dev        [batch][hq][hd] floats
 * Every query sits at position s-1 (causal; window <= 0 means global).  Work is
 * queued on `stream` (NULL: the default stream) and the call returns without
 * waiting.
 *
 * Limits: batch <= 16368 and batch*hq*nsplit*(hd+2)*4 bytes <= 8 MiB - 64 KiB;
 * larger requests are rejected with InvalidArgument.  The first call on a
 * device looks up the array's address and sets a kernel attribute; make that
 * first call before starting any stream capture.  All calls on a device share
 * the array, which keeps what the last call left in it (the call itself resets
 * the one word that must start at zero); two calls whose kernels overlap on
 * the GPU -- different streams, no ordering between them -- race on it.  The
 * caller's current device is left as it was.  The per-device set-up is done
 * under a lock, so first calls from several threads are safe. */
int B200LmOps_AttentionDecodeStatic(int32_t device, const float* q_dev, const void* k_pages_dev,
                                    const void* v_pages_dev, const int32_t* page_table_dev, int32_t batch, int32_t s,
                                    int32_t hq, int32_t hkv, int32_t hd, int32_t window, int32_t kv_bf16,
                                    int32_t nsplit, float* out_dev, void* stream, char** err);

/* Status of the work queued by B200LmOps_AttentionDecodeStatic on `stream`:
 * waits for the stream, then reads the error word its kernels keep in the
 * static array (no allocation either).  Returns OK, or InvalidArgument when a
 * query position lay outside the cache; *device_error (optional) receives the
 * raw word.  No counterpart in the reference. */
int B200LmOps_AttentionDecodeStaticStatus(int32_t device, void* stream, int32_t* device_error, char** err);

#ifdef __cplusplus
}
#endif
#endif /* B200LM_OPS_H_ */

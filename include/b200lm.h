/*
 * b200lm.h — C ABI of the B200 LlmExecutor backend for LiteRT-LM.
 *
 * The library (libb200lm.so) replaces, for one decoder model on one B200, the
 * work the reference does inside LlmLiteRtCompiledModelExecutor:
 * Prefill / Decode / DecodeLogits with the same token hold-back, step counting
 * and bucketed work groups, on hand-written sm_100a CUDA kernels.
 *
 * Conventions (those of the reference's one dynamic C boundary, the GPU
 * sampler in runtime/components/sampler_factory.cc:30-57):
 *   - every call returns an absl::StatusCode integer (0 OK, 1 Cancelled,
 *     3 InvalidArgument, 4 DeadlineExceeded, 5 NotFound, 9 FailedPrecondition,
 *     12 Unimplemented, 13 Internal);
 *   - on failure *err (when err != NULL) receives a malloc'd message that the
 *     caller releases with free();
 *   - handles are opaque; one handle is used from one thread at a time (the
 *     reference drives an executor from a single engine worker thread,
 *     runtime/core/engine_impl.cc:185-186); different handles are independent.
 * There is no CPU fallback: without a CUDA device every entry point that needs
 * one fails with FailedPrecondition.
 */
#ifndef B200LM_H_
#define B200LM_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct B200LmExecutor B200LmExecutor;

/* decode_mode: AUTO picks the chained persistent kernel when the model fits its
 * shared-memory ring, else the streaming persistent kernel, else one kernel per
 * phase replayed from a CUDA graph. */
enum {
  B200LM_DECODE_AUTO = 0,
  B200LM_DECODE_PHASE_KERNELS = 1,     /* one kernel per phase, CUDA graph per step */
  B200LM_DECODE_PERSISTENT = 2,        /* one cooperative kernel, grid barrier per phase, weights streamed by bulk async copies */
  B200LM_DECODE_PERSISTENT_BASIC = 3,  /* one cooperative kernel, grid barrier per phase, plain loads (comparison) */
  B200LM_DECODE_CHAINED = 4,           /* one cooperative kernel without grid barriers: phases hand results over in
                                          flag-carrying words, gate/up + down fused */
  B200LM_DECODE_WIDE = 5               /* lockstep groups of up to 128 sessions: the projections of a step run on the
                                          tensor-core int4 GEMM of the prefill path with the sessions as its token
                                          rows (bf16 activations), one attention CTA per (session, kv head), one CUDA
                                          graph per step.  AUTO picks it when n_sessions > 4.  Needs the tensor-core
                                          GEMM weights; no tensor parallelism. */
};
enum { B200LM_GEMM_AUTO = 0, B200LM_GEMM_CHECK = 1, B200LM_GEMM_TCGEN05 = 2 };

typedef struct B200LmConfig {
  int32_t struct_size;     /* sizeof(B200LmConfig), for forward compatibility */
  int32_t device;          /* CUDA device ordinal */
  int32_t max_num_tokens;  /* KV capacity; 0 = the model's context length.
                              Counterpart of LlmExecutorSettings::GetMaxNumTokens
                              (runtime/executor/llm_executor_settings.h:95-154). */
  int32_t decode_mode;     /* B200LM_DECODE_* */
  int32_t prefill_gemm;    /* B200LM_GEMM_* */
  int32_t page_order;      /* physical order of a session's KV pages: 0 = ascending (normal use),
                              1 = descending.  A test hook: with the table reversed, a wrong
                              (page, slot) computation cannot pass the KV indexing checks by
                              accident.  Results do not depend on it. */
  void* stream;            /* cudaStream_t to run on, or NULL for an own stream */
  int32_t n_sessions;      /* sessions held by this executor (0 = 1): 1..4 with the persistent decode
                              kernels, up to 128 in B200LM_DECODE_WIDE; see B200Lm_DecodeTokensBatch */
  int32_t reserved1;
  /* Tensor parallelism (BASELINE config 5).  tp_world > 1: this executor is rank tp_rank of tp_world and
   * the model image holds THAT RANK'S SHARD (query / kv heads and FFN columns split over the ranks, see
   * model_io.shard_for_tensor_parallel); the partial O and down projections of the ranks are summed with an
   * NCCL all-reduce on the executor's stream.  tp_unique_id points at the 128 bytes of an ncclUniqueId that
   * rank 0 obtained from B200Lm_TpUniqueId and handed to every rank.  One process per GPU; every rank makes
   * the same calls in the same order.  The reference has no multi-GPU path
   * (runtime/executor/llm_litert_compiled_model_executor.cc:95 checks batch 1). */
  int32_t tp_rank;
  int32_t tp_world;
  const void* tp_unique_id;
} B200LmConfig;

/* Replaces LlmLiteRtCompiledModelExecutor::Create
 * (runtime/executor/llm_litert_compiled_model_executor.cc:590-833): reads the
 * `.litertlm` image (bytes, or a file path when bytes == NULL), repacks the
 * int4 weights for the kernels and allocates the paged KV cache. */
int B200Lm_Create(const B200LmConfig* config, const void* litertlm_bytes, uint64_t n_bytes,
                  const char* path_or_null, B200LmExecutor** out, char** err);

/* A second executor (own KV cache, own step counter) over the weights of an
 * existing one: independent sessions on one GPU share one weight copy.  No
 * counterpart in the reference, whose engine shares one executor between
 * sessions and resets it (runtime/core/session_basic.cc:67-72). */
int B200Lm_CreateShared(B200LmExecutor* weights_owner, const B200LmConfig* config,
                        B200LmExecutor** out, char** err);

void B200Lm_Destroy(B200LmExecutor* e);

/* Replaces LlmLiteRtCompiledModelExecutor::Prefill(inputs, params)
 * (llm_litert_compiled_model_executor.cc:90-276).  ids is host memory, batch 1.
 * The last id of every work group is held back and consumed by the next
 * Prefill / Decode call.  wait_for_completion and cancel carry
 * ExecutorPrefillParams (runtime/executor/llm_executor_io_types.h:217-250);
 * *cancel is polled between work groups -> Cancelled. */
int B200Lm_Prefill(B200LmExecutor* e, const int32_t* ids, int32_t n_ids, int32_t wait_for_completion,
                   const volatile int32_t* cancel_or_null, char** err);

/* Replaces DecodeLogits(inputs) and Decode(inputs, logits)
 * (llm_litert_compiled_model_executor.cc:300-534): runs one step on *id (or on
 * the pending id when id == NULL; none pending -> InvalidArgument "No id
 * available to be decoded.") and writes vocab floats to host_logits, which may
 * be pageable or page-locked host memory (a page-locked buffer receives the
 * device-to-host copy directly). */
int B200Lm_DecodeLogits(B200LmExecutor* e, const int32_t* id_or_null, float* host_logits, char** err);

/* Replaces Decode(output_tokens) (llm_litert_compiled_model_executor.cc:278-298):
 * one step on the pending id, greedy arg-max on the device (lowest index wins
 * ties, as std::max_element in runtime/components/sampling_cpu_util.cc:32-41),
 * result becomes the pending id. */
int B200Lm_DecodeToken(B200LmExecutor* e, int32_t* out_id, char** err);

/* n_steps greedy steps with the arg-max fed back on the device, no host round
 * trip per step; ids come back at the end.  Equivalent to n_steps calls of
 * B200Lm_DecodeToken. */
int B200Lm_DecodeTokens(B200LmExecutor* e, int32_t n_steps, int32_t* out_ids, char** err);

/* Several sessions in one executor.  No counterpart in the reference, whose
 * engine gives every session the one executor in turn (runtime/core/
 * session_basic.cc:67-72).  An executor created with n_sessions = B holds B
 * independent sessions over one weight copy: each has its own KV pages, step
 * counter and pending id.  B200Lm_SelectSession makes one of them the session
 * that Prefill / DecodeLogits / DecodeToken(s) / Reset / GetCurrentStep /
 * GetLastPrefillPlan / ReadKvRow act on (session 0 after Create);
 * B200Lm_PrefillSession is Select + Prefill.  B200Lm_DecodeTokensBatch advances
 * ALL sessions by n_steps greedy steps in lockstep, reading the weights once
 * per step for the whole batch; out_ids is [n_steps][n_sessions].  Every
 * session must have a pending id (i.e. have been prefilled).  With three or
 * four sessions the decode activations are quantised to two int8 terms
 * instead of three (relative error 6e-5 instead of 5e-7); in B200LM_DECODE_WIDE
 * (more than four sessions) they are bf16, as in prefill. */
int B200Lm_SelectSession(B200LmExecutor* e, int32_t session, char** err);
int B200Lm_GetNumSessions(B200LmExecutor* e, int32_t* out, char** err);
int B200Lm_PrefillSession(B200LmExecutor* e, int32_t session, const int32_t* ids, int32_t n,
                          int32_t wait_for_completion, const volatile int32_t* cancel_or_null, char** err);
int B200Lm_DecodeTokensBatch(B200LmExecutor* e, int32_t n_steps, int32_t* out_ids, char** err);

/* Replaces Reset() (llm_litert_compiled_model_executor.cc:568-574): rewinds the
 * counters, leaves the cache contents in place. */
int B200Lm_Reset(B200LmExecutor* e, char** err);

/* GetVocabSize (:576-586), GetCurrentStep (llm_litert_compiled_model_executor.h:95-97:
 * processed tokens + 1 when an id is pending), GetExecutorSettings().GetMaxNumTokens(). */
int B200Lm_GetVocabSize(B200LmExecutor* e, int32_t* out, char** err);
int B200Lm_GetCurrentStep(B200LmExecutor* e, int32_t* out, char** err);
int B200Lm_GetMaxNumTokens(B200LmExecutor* e, int32_t* out, char** err);

/* 128 bytes of a fresh ncclUniqueId for a tensor-parallel group (call on one rank, give the bytes to all).
 * No counterpart in the reference. */
int B200Lm_TpUniqueId(void* out_128_bytes, char** err);

/* Mean device time (ms) of one all-reduce of `count` floats over the executor's tensor-parallel group,
 * measured with CUDA events over `iters` back-to-back calls: tells the share of the collectives in a
 * decode step (two per layer).  Every rank must call it.  No counterpart in the reference. */
int B200Lm_TpAllReduceProbe(B200LmExecutor* e, int64_t count, int32_t iters, float* ms_out, char** err);

/* The decode path this executor settled on (B200LM_DECODE_*): what AUTO resolved to, or
 * the fallback taken when the requested kernel does not fit the model.  No counterpart
 * in the reference. */
int B200Lm_GetDecodeMode(B200LmExecutor* e, int32_t* out, char** err);

/* ExecutorBackendName() (runtime/executor/llm_executor_base.h:79). */
const char* B200Lm_BackendName(void);

/* Waits for everything queued on the executor's stream; reports a device error
 * word set by a kernel (bounded wait that gave up, token or position out of
 * range) as DeadlineExceeded / InvalidArgument. */
int B200Lm_Synchronize(B200LmExecutor* e, char** err);

/* The work-group plan of the last Prefill: (bucket, ids) pairs as chosen by
 * GetOptimizedPrefillWorkGroups (litert_compiled_model_executor_utils.cc:300-330). */
int B200Lm_GetLastPrefillPlan(B200LmExecutor* e, int32_t* buckets, int32_t* lengths, int32_t capacity,
                              int32_t* n_groups, char** err);

/* Inspection: one cached K or V row (head_dim floats) and the physical page /
 * slot the position maps to.  Used by the KV-indexing parity tests. */
int B200Lm_ReadKvRow(B200LmExecutor* e, int32_t layer, int32_t is_v, int32_t kv_head, int32_t pos,
                     float* out_row, int32_t* out_page, int32_t* out_slot, char** err);

/* Device timeline of ONE greedy decode step run by a persistent decode mode
 * (equivalent to B200Lm_DecodeToken): for every grid barrier b and CTA c,
 * stamps[(b * n_cta + c) * 2 + {0,1}] = that SM's cycle counter when the CTA
 * arrived at / was released from the barrier.  Within one CTA,
 * arrive[b] - release[b-1] is the time it worked in phase b and
 * release[b] - arrive[b] the time it waited.  After those n_barriers * n_cta * 2
 * values come n_barriers * n_cta * 8 stamps taken inside the phase that ends
 * at barrier b (streaming mode: 0 phase start, 1 staged bytes arrived, 2 next
 * fill issued, 3 prologue done, 4 MMA done, 5 epilogue done, 6 phase end; 0
 * where a point was not reached).  The reference has no per-op
 * profiler hook (only wall-clock BenchmarkInfo marks, runtime/engine/io_types.h:104-163).
 * capacity is in int64 elements; sm_clock_khz converts cycles to time. */
int B200Lm_TraceDecodeStep(B200LmExecutor* e, int32_t* out_id, int64_t* stamps, int64_t capacity,
                           int32_t* n_barriers, int32_t* n_cta, int32_t* sm_clock_khz, char** err);

/* Number of kernels of this library launched on behalf of the handle so far. */
int B200Lm_GetLaunchCount(B200LmExecutor* e, int64_t* out, char** err);

#ifdef __cplusplus
}
#endif
#endif /* B200LM_H_ */

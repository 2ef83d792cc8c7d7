/* TEST / MEASUREMENT INFRASTRUCTURE, not part of the product path.
 *
 * A second CPU baseline for the timed comparison: the decoder's int4 matrices run through XNNPACK's
 * fully-connected operator with per-channel int4 weights and dynamically quantised int8 activations
 * (qd8-f32-qc8w), the kernel family the reference's CPU backend reaches through LiteRT's XNNPACK delegate.
 * The int4 values are handed over as int8 channel-wise weights: the int4 operator (qd8-f32-qc4w) of this
 * XNNPACK build returns wrong sums for 64 or more input channels (all-ones weights, ramp input, compared
 * with the qc8w operator on the same data), so it is not used.  Decode therefore reads twice the weight
 * bytes an int4 kernel would; prefill runs the same int8 VNNI arithmetic.  This is the XNNPACK build that ships inside torch (symbols exported
 * by libtorch_cpu.so, bound with dlsym after `import torch`), NOT LiteRT and NOT the reference's pinned
 * XNNPACK revision.  Everything that is not a matrix product (norms, RoPE, attention, GeGLU) stays the
 * plain C of oracle.c: this file only supplies the matmul hook (orc_set_matmul_hook).
 *
 * Activations are quantised to int8 per row here, so results differ from the fp32 oracle by the
 * quantisation error; it is a timing baseline, not a parity oracle.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <xnnpack.h>

typedef enum xnn_status (*fn_initialize)(const struct xnn_allocator*);
typedef enum xnn_status (*fn_create_fc)(size_t, size_t, size_t, size_t, const float*, const int8_t*, const float*, float, float,
                                        uint32_t, xnn_code_cache_t, xnn_weights_cache_t, xnn_operator_t*);
typedef enum xnn_status (*fn_reshape_fc)(xnn_operator_t, size_t, pthreadpool_t);
typedef enum xnn_status (*fn_setup_fc)(xnn_operator_t, const int8_t*, float*, const struct xnn_quantization_params*);
typedef enum xnn_status (*fn_create_cvt)(uint32_t, xnn_operator_t*);
typedef enum xnn_status (*fn_reshape_cvt)(xnn_operator_t, size_t, size_t, size_t, size_t, pthreadpool_t);
typedef enum xnn_status (*fn_setup_cvt)(xnn_operator_t, const float*, int8_t*, struct xnn_quantization_params*);
typedef enum xnn_status (*fn_run)(xnn_operator_t, pthreadpool_t);
typedef pthreadpool_t (*fn_pool_create)(size_t);
typedef void (*fn_pool_destroy)(pthreadpool_t);

static struct {
  fn_initialize initialize;
  fn_create_fc create_fc;
  fn_reshape_fc reshape_fc;
  fn_setup_fc setup_fc;
  fn_create_cvt create_cvt;
  fn_reshape_cvt reshape_cvt;
  fn_setup_cvt setup_cvt;
  fn_run run;
  fn_pool_create pool_create;
  fn_pool_destroy pool_destroy;
  pthreadpool_t pool;
  xnn_operator_t cvt;
  int ready;
} X;

#define XNNB_MAX_OPS 2048
static struct { const void* key; int N, K, T; xnn_operator_t op; } g_ops[XNNB_MAX_OPS];
static int g_nops = 0;
static int8_t* g_q = NULL;
static struct xnn_quantization_params* g_qp = NULL;
static size_t g_q_cap = 0, g_qp_cap = 0;
static int g_cvt_T = -1, g_cvt_K = -1;

/* Returns 0 when XNNPACK is bound and initialised with a pool of `threads` workers. */
int xnnb_init(int threads, const char* torch_cpu_lib) {
  if (X.ready) {
    if (X.pool) X.pool_destroy(X.pool);
    X.pool = X.pool_create((size_t)threads);
    g_cvt_T = -1;
    for (int i = 0; i < g_nops; ++i) g_ops[i].T = -1;      /* operators re-plan for the new pool */
    return X.pool ? 0 : -1;
  }
  /* Python loads torch's libraries with local visibility: take a handle on the already-loaded library. */
  void* h = torch_cpu_lib ? dlopen(torch_cpu_lib, RTLD_NOW | RTLD_NOLOAD) : NULL;
  if (!h) h = RTLD_DEFAULT;
#define BIND(field, type, name) X.field = (type)dlsym(h, name); if (!X.field) { fprintf(stderr, "xnnb: %s not found\n", name); return -1; }
  BIND(initialize, fn_initialize, "xnn_initialize")
  BIND(create_fc, fn_create_fc, "xnn_create_fully_connected_nc_qd8_f32_qc8w")
  BIND(reshape_fc, fn_reshape_fc, "xnn_reshape_fully_connected_nc_qd8_f32_qc8w")
  BIND(setup_fc, fn_setup_fc, "xnn_setup_fully_connected_nc_qd8_f32_qc8w")
  BIND(create_cvt, fn_create_cvt, "xnn_create_convert_nc_f32_qd8")
  BIND(reshape_cvt, fn_reshape_cvt, "xnn_reshape_convert_nc_f32_qd8")
  BIND(setup_cvt, fn_setup_cvt, "xnn_setup_convert_nc_f32_qd8")
  BIND(run, fn_run, "xnn_run_operator")
  BIND(pool_create, fn_pool_create, "pthreadpool_create")
  BIND(pool_destroy, fn_pool_destroy, "pthreadpool_destroy")
#undef BIND
  if (X.initialize(NULL) != xnn_status_success) return -2;
  X.pool = X.pool_create((size_t)threads);
  if (!X.pool) return -3;
  if (X.create_cvt(0, &X.cvt) != xnn_status_success) return -4;
  X.ready = 1;
  return 0;
}

/* The matmul hook of oracle.c: y[t][n] = scale[n] * sum_k w[n][k] x[t][k], w in [-7, 7] expanded to int8.
 * Returns 0 on success (non-zero makes the oracle fall back to its own loop). */
int xnnb_matmul(const void* key, const int8_t* w, const float* scale, int N, int K, const float* x, int T, float* y, int ldy) {
  if (!X.ready || ldy != N) return -1;
  int idx = -1;
  for (int i = 0; i < g_nops; ++i)
    if (g_ops[i].key == key && g_ops[i].N == N && g_ops[i].K == K) { idx = i; break; }
  if (idx < 0) {
    if (g_nops >= XNNB_MAX_OPS) return -1;
    xnn_operator_t op = NULL;
    float* bias = (float*)calloc((size_t)N, sizeof(float));
    enum xnn_status st = X.create_fc((size_t)K, (size_t)N, (size_t)K, (size_t)N, scale, w, bias, -INFINITY, INFINITY, 0, NULL, NULL, &op);
    free(bias);                                    /* XNNPACK keeps its own packed copy of weights and bias */
    if (st != xnn_status_success) return -1;
    idx = g_nops++;
    g_ops[idx].key = key; g_ops[idx].N = N; g_ops[idx].K = K; g_ops[idx].T = -1; g_ops[idx].op = op;
  }
  size_t need_q = (size_t)T * K + XNN_EXTRA_BYTES, need_qp = (size_t)T + XNN_EXTRA_QUANTIZATION_PARAMS;
  if (need_q > g_q_cap) { free(g_q); g_q = (int8_t*)malloc(need_q); g_q_cap = need_q; }
  if (need_qp > g_qp_cap) { free(g_qp); g_qp = (struct xnn_quantization_params*)malloc(need_qp * sizeof *g_qp); g_qp_cap = need_qp; }
  if (!g_q || !g_qp) return -1;
  if (g_cvt_T != T || g_cvt_K != K) {
    if (X.reshape_cvt(X.cvt, (size_t)T, (size_t)K, (size_t)K, (size_t)K, X.pool) != xnn_status_success) return -1;
    g_cvt_T = T; g_cvt_K = K;
  }
  if (X.setup_cvt(X.cvt, x, g_q, g_qp) != xnn_status_success) return -1;
  if (X.run(X.cvt, X.pool) != xnn_status_success) return -1;
  if (g_ops[idx].T != T) {
    if (X.reshape_fc(g_ops[idx].op, (size_t)T, X.pool) != xnn_status_success) return -1;
    g_ops[idx].T = T;
  }
  if (X.setup_fc(g_ops[idx].op, g_q, y, g_qp) != xnn_status_success) return -1;
  if (X.run(g_ops[idx].op, X.pool) != xnn_status_success) return -1;
  return 0;
}

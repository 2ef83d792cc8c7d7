/*
 * CPU ORACLE — test infrastructure, not product code.
 *
 * A plain-C restatement of the LiteRT-LM executor hot path (Prefill / Decode /
 * logits for a Gemma3-style int4 decoder).  Only the test-suite, the smoke
 * check and the benchmark's CPU-baseline leg may load this library; the CUDA
 * library never links or calls it.
 *
 * What follows the reference, and where:
 *   - executor state machine (held-back last token, step counter, Reset):
 *       runtime/executor/llm_litert_compiled_model_executor.cc:90-298,416-586
 *       runtime/executor/llm_litert_compiled_model_executor.h:95-97
 *   - prefill work-group (bucket) plan:
 *       runtime/executor/litert_compiled_model_executor_utils.cc:300-330
 *   - attention-mask rule:
 *       runtime/executor/litert_compiled_model_executor_utils.cc:332-397
 *   - greedy arg-max / soft-max of the CPU sampler:
 *       runtime/components/sampling_cpu_util.cc:21-134
 *
 * PARITY STATUS: the reference keeps the decoder arithmetic inside an opaque
 * third-party graph (LiteRT CompiledModel::Run -> TFLite -> XNNPACK; LiteRT @
 * c8f55dfbf3f9cefa93528f060e0982d5247d23ae, TensorFlow @
 * 734f70856ea65331526cecb608f9f14c76aee2f2, both absent from the reference
 * tree) and ships no golden logits or tokens.  The layer arithmetic below is
 * therefore a written specification ("parity unpinned" for logits); the state
 * machine, bucket plan, mask rule and sampler ARE pinned by the reference's
 * sources and test vectors (see tests/).
 *
 * Layer specification (frozen here; the CUDA kernels implement the same):
 *   x   = dequant(E[token]) * sqrt(d)
 *   per layer i (global iff i % period == period-1):
 *     h = rmsnorm(x, g_pre_attn);  [q|k|v] = Wqkv h
 *     q,k = rmsnorm per head over head_dim (g_q, g_k); RoPE half-split pairing
 *           (j, j+hd/2), theta = pos * base^(-2j/hd), base 1e4 local/1e6 global
 *     K[pos], V[pos] <- k, v     (paged cache, page = 256 positions)
 *     o = softmax(q.K^T / sqrt(hd) + mask) V ; mask open iff kpos <= qpos and
 *           (global or qpos - kpos < window)
 *     x = x + rmsnorm(Wo o, g_post_attn)
 *     h = rmsnorm(x, g_pre_ffn); f = Wdown( gelu_tanh(Wgate h) * (Wup h) )
 *     x = x + rmsnorm(f, g_post_ffn)
 *   logits = E rmsnorm(x, g_final)         (tied int4 table)
 *   rmsnorm(x, g) = x * rsqrt(mean(x^2) + eps) * g,  eps = 1e-6
 * int4: row-major [N][K/2] bytes, element 2j in the low nibble of byte j,
 * two's complement in [-7, 7], one fp32 scale per output row, zero-point 0.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#define ORC_PAGE 256
#define ORC_MAX_BUCKETS 8

/* ------------------------------------------------------------------ int4 */

/* Unpack canonical packed int4 rows into int8 values (bit-exact gate). */
void orc_unpack_int4(const uint8_t* packed, int64_t n, int64_t k, int8_t* out) {
  for (int64_t r = 0; r < n; ++r) {
    const uint8_t* p = packed + r * (k / 2);
    int8_t* o = out + r * k;
    for (int64_t j = 0; j < k / 2; ++j) {
      int lo = p[j] & 0xF, hi = p[j] >> 4;
      o[2 * j] = (int8_t)(lo >= 8 ? lo - 16 : lo);
      o[2 * j + 1] = (int8_t)(hi >= 8 ? hi - 16 : hi);
    }
  }
}

/* Symmetric per-row quantisation: scale = max|w| / 7, q = rint(w / scale). */
void orc_quantize_int4(const float* w, int64_t n, int64_t k, uint8_t* packed,
                       float* scale) {
  for (int64_t r = 0; r < n; ++r) {
    const float* row = w + r * k;
    float amax = 0.f;
    for (int64_t j = 0; j < k; ++j) {
      float a = fabsf(row[j]);
      if (a > amax) amax = a;
    }
    float s = amax > 0.f ? amax / 7.0f : 1.0f;
    scale[r] = s;
    for (int64_t j = 0; j < k; j += 2) {
      int q0 = (int)rintf(row[j] / s), q1 = (int)rintf(row[j + 1] / s);
      if (q0 > 7) q0 = 7;
      if (q0 < -7) q0 = -7;
      if (q1 > 7) q1 = 7;
      if (q1 < -7) q1 = -7;
      packed[r * (k / 2) + j / 2] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
    }
  }
}

/* KV index rule: position -> (logical page, slot); element offset inside the
 * pool for layout [physical_page][kv_head][slot][head_dim]. */
void orc_kv_index(int pos, int* page, int* slot) {
  *page = pos / ORC_PAGE;
  *slot = pos % ORC_PAGE;
}
int64_t orc_kv_offset(int phys_page, int kv_head, int slot, int n_kv_heads,
                      int head_dim) {
  return (((int64_t)phys_page * n_kv_heads + kv_head) * ORC_PAGE + slot) *
         head_dim;
}

/* ------------------------------------------------- sampler (greedy path) */

/* First (lowest-index) maximum per batch row: sampling_cpu_util.cc:32-41. */
int orc_greedy(const float* logits, int64_t total, int batch, int32_t* out) {
  if (batch <= 0 || total % batch != 0) return 3;
  int64_t v = total / batch;
  for (int b = 0; b < batch; ++b) {
    const float* row = logits + b * v;
    int64_t best = 0;
    for (int64_t i = 1; i < v; ++i)
      if (row[best] < row[i]) best = i; /* std::max_element semantics */
    out[b] = (int32_t)best;
  }
  return 0;
}

/* Soft-max over the selected indices: sampling_cpu_util.cc:66-134. */
int orc_softmax(const float* logits, int64_t total, const int32_t* topk,
                int64_t n_topk, float temperature, int batch, float* probs,
                float* max_vals) {
  if (total == 0) return 3;
  if (total % batch != 0) return 3;
  if (temperature <= 0.0f) return 3;
  int64_t v = total / batch, k = n_topk / batch;
  for (int b = 0; b < batch; ++b) {
    int64_t mi = 0;
    for (int64_t i = 1; i < k; ++i)
      if (logits[b * v + topk[b * k + mi]] < logits[b * v + topk[b * k + i]])
        mi = i;
    float mx = logits[b * v + topk[b * k + mi]];
    max_vals[b] = mx;
    float sum = 0.f;
    if (temperature < 1.1920929e-07f) temperature = 1.1920929e-07f;
    for (int64_t i = 0; i < k; ++i) {
      probs[b * k + i] = expf((logits[b * v + topk[b * k + i]] - mx) / temperature);
      sum += probs[b * k + i];
    }
    if (sum <= 1.1920929e-07f) {
      for (int64_t i = 0; i < k; ++i) probs[b * k + i] = 1.0f / (float)k;
    } else if (isinf(sum)) {
      for (int64_t i = 0; i < k; ++i) probs[b * k + i] = 0.f;
      probs[b * k + mi] = 1.f;
    } else {
      float inv = 1.0f / sum;
      for (int64_t i = 0; i < k; ++i) probs[b * k + i] *= inv;
    }
  }
  return 0;
}

/* --------------------------------------------- prefill work-group planner */

/* buckets must be sorted descending (SortedPrefillSignatureMap order).
 * Returns the number of groups; group g uses bucket out_bucket[g] for
 * out_len[g] ids.  utils.cc:300-330. */
int orc_plan_work_groups(const int* buckets, int n_buckets, int input_length,
                         int* out_bucket, int* out_len, int max_groups) {
  int n = 0;
  int max_len = buckets[0];
  while (input_length >= max_len) {
    if (n >= max_groups) return -1;
    out_bucket[n] = max_len;
    out_len[n] = max_len;
    ++n;
    input_length -= max_len;
  }
  if (input_length > 0) {
    for (int i = 0; i < n_buckets; ++i) {
      if (i + 1 < n_buckets && buckets[i + 1] >= input_length) continue;
      if (n >= max_groups) return -1;
      out_bucket[n] = buckets[i];
      out_len[n] = input_length;
      ++n;
      break;
    }
  }
  return n;
}

/* Dense float attention mask exactly as the reference builds it
 * (utils.cc:332-397): everything closed (-45824 for f16-safe calculation,
 * else -0.7*FLT_MAX), then row i open on [0, start+i]. */
void orc_fill_mask(float* mask, int rows, int ctx, int start, int steps,
                   int is_f16) {
  float closed = is_f16 ? -45824.0f : -0.7f * 3.402823466e+38f;
  for (int64_t i = 0; i < (int64_t)rows * ctx; ++i) mask[i] = closed;
  for (int i = 0; i < steps; ++i)
    for (int j = 0; j <= start + i && j < ctx; ++j) mask[(int64_t)i * ctx + j] = 0.0f;
}

/* ------------------------------------------------------------- the model */

typedef struct {
  char name[48];
  uint32_t dtype; /* 0 = packed int4 bytes, 1 = float32 */
  uint32_t rows, cols, pad;
  uint64_t offset, nbytes;
} OrcTensorEntry; /* 80 bytes */

typedef struct {
  int n_layers, d, hq, hkv, hd, ffn, vocab, max_ctx, window, period, kv_dtype;
  int n_buckets;
  int buckets[ORC_MAX_BUCKETS];
  float rope_local, rope_global, eps;
} OrcCfg;

typedef struct {
  int8_t* w; /* expanded [rows][cols] */
  const float* scale;
  int rows, cols;
} OrcMat;

typedef struct {
  OrcMat wqkv, wo, wgate, wup, wdown;
  const float *g_pre_attn, *g_post_attn, *g_pre_ffn, *g_post_ffn, *g_q, *g_k;
} OrcLayer;

typedef struct {
  OrcCfg cfg;
  const uint8_t* blob;
  OrcMat embed;
  const float* g_final;
  OrcLayer* layers;
  float *rope_cos[2], *rope_sin[2]; /* [max_ctx][hd/2], 0 = local 1 = global */
} OrcModel;

static const OrcTensorEntry* find_tensor(const uint8_t* blob, const char* name) {
  uint32_t n = *(const uint32_t*)(blob + 12);
  const OrcTensorEntry* e = (const OrcTensorEntry*)(blob + 256);
  for (uint32_t i = 0; i < n; ++i)
    if (strncmp(e[i].name, name, 48) == 0) return &e[i];
  return NULL;
}

static int load_mat(const uint8_t* blob, const char* base, OrcMat* m) {
  char nm[64];
  snprintf(nm, sizeof nm, "%s.q", base);
  const OrcTensorEntry* q = find_tensor(blob, nm);
  snprintf(nm, sizeof nm, "%s.scale", base);
  const OrcTensorEntry* s = find_tensor(blob, nm);
  if (!q || !s) return -1;
  m->rows = (int)q->rows;
  m->cols = (int)q->cols;
  m->scale = (const float*)(blob + s->offset);
  m->w = (int8_t*)malloc((size_t)m->rows * m->cols);
  if (!m->w) return -1;
  orc_unpack_int4(blob + q->offset, m->rows, m->cols, m->w);
  return 0;
}

static const float* load_vec(const uint8_t* blob, const char* name) {
  const OrcTensorEntry* e = find_tensor(blob, name);
  return e ? (const float*)(blob + e->offset) : NULL;
}

/* RoPE tables in double precision, rounded once to float.  The CUDA library
 * builds its tables with the same expressions on the host. */
void orc_rope_table(double base, int hd, int max_ctx, float* cos_t, float* sin_t) {
  int half = hd / 2;
  for (int p = 0; p < max_ctx; ++p)
    for (int j = 0; j < half; ++j) {
      double inv = pow(base, -2.0 * (double)j / (double)hd);
      double a = (double)p * inv;
      cos_t[(int64_t)p * half + j] = (float)cos(a);
      sin_t[(int64_t)p * half + j] = (float)sin(a);
    }
}

void orc_model_destroy(OrcModel* m);

/* blob: the weights record ("B2LMWT01"); must outlive the model. */
OrcModel* orc_model_create(const uint8_t* blob, uint64_t len) {
  if (len < 512 || memcmp(blob, "B2LMWT01", 8) != 0) return NULL;
  OrcModel* m = (OrcModel*)calloc(1, sizeof *m);
  const int32_t* ic = (const int32_t*)(blob + 16);
  const float* fc = (const float*)(blob + 80);
  OrcCfg* c = &m->cfg;
  c->n_layers = ic[0]; c->d = ic[1]; c->hq = ic[2]; c->hkv = ic[3]; c->hd = ic[4];
  c->ffn = ic[5]; c->vocab = ic[6]; c->max_ctx = ic[7]; c->window = ic[8];
  c->period = ic[9]; c->kv_dtype = ic[10]; c->n_buckets = ic[11];
  c->rope_local = fc[0]; c->rope_global = fc[1]; c->eps = fc[2];
  const int32_t* bk = (const int32_t*)(blob + 112);
  for (int i = 0; i < c->n_buckets && i < ORC_MAX_BUCKETS; ++i) c->buckets[i] = bk[i];
  m->blob = blob;
  m->layers = (OrcLayer*)calloc((size_t)c->n_layers, sizeof(OrcLayer));
  int bad = load_mat(blob, "embed", &m->embed);
  m->g_final = load_vec(blob, "final_norm");
  if (!m->g_final) bad = 1;
  for (int i = 0; i < c->n_layers && !bad; ++i) {
    char nm[64];
    OrcLayer* L = &m->layers[i];
#define LM(field, s) snprintf(nm, sizeof nm, "L%d." s, i); bad |= load_mat(blob, nm, &L->field) != 0;
#define LV(field, s) snprintf(nm, sizeof nm, "L%d." s, i); L->field = load_vec(blob, nm); bad |= L->field == NULL;
    LM(wqkv, "wqkv") LM(wo, "wo") LM(wgate, "wgate") LM(wup, "wup") LM(wdown, "wdown")
    LV(g_pre_attn, "pre_attn") LV(g_post_attn, "post_attn") LV(g_pre_ffn, "pre_ffn")
    LV(g_post_ffn, "post_ffn") LV(g_q, "q_norm") LV(g_k, "k_norm")
#undef LM
#undef LV
  }
  if (bad) { orc_model_destroy(m); return NULL; }
  int half = c->hd / 2;
  for (int t = 0; t < 2; ++t) {
    m->rope_cos[t] = (float*)malloc(sizeof(float) * (size_t)c->max_ctx * half);
    m->rope_sin[t] = (float*)malloc(sizeof(float) * (size_t)c->max_ctx * half);
    orc_rope_table(t ? c->rope_global : c->rope_local, c->hd, c->max_ctx,
                   m->rope_cos[t], m->rope_sin[t]);
  }
  return m;
}

void orc_model_destroy(OrcModel* m) {
  if (!m) return;
  free(m->embed.w);
  if (m->layers)
    for (int i = 0; i < m->cfg.n_layers; ++i) {
      free(m->layers[i].wqkv.w); free(m->layers[i].wo.w); free(m->layers[i].wgate.w);
      free(m->layers[i].wup.w); free(m->layers[i].wdown.w);
    }
  free(m->layers);
  for (int t = 0; t < 2; ++t) { free(m->rope_cos[t]); free(m->rope_sin[t]); }
  free(m);
}

void orc_model_cfg(const OrcModel* m, int32_t* out16) {
  const OrcCfg* c = &m->cfg;
  int32_t v[16] = {c->n_layers, c->d, c->hq, c->hkv, c->hd, c->ffn, c->vocab,
                   c->max_ctx, c->window, c->period, c->kv_dtype, c->n_buckets};
  memcpy(out16, v, sizeof v);
}

/* Optional replacement of the matrix product (the XNNPACK timing baseline of xnn_baseline.c installs one);
 * the parity oracle never sets it.  A non-zero return falls back to the loop below. */
typedef int (*OrcMatmulHook)(const void* key, const int8_t* w, const float* scale, int N, int K, const float* x, int T,
                             float* y, int ldy);
static OrcMatmulHook g_matmul_hook = NULL;
void orc_set_matmul_hook(void* fn) { g_matmul_hook = (OrcMatmulHook)fn; }
#ifdef _OPENMP
#include <omp.h>
void orc_set_threads(int n) { if (n > 0) omp_set_num_threads(n); }
#else
void orc_set_threads(int n) { (void)n; }
#endif

/* y[t][n] = scale[n] * sum_k W[n][k] x[t][k].  fp32 products are summed in
 * 32-element chunks in fp32 and the chunk totals in double. */
static void matmul_w4(const OrcMat* m, const float* x, int T, float* y, int ldy) {
  int N = m->rows, K = m->cols;
  if (g_matmul_hook && g_matmul_hook(m->w, m->w, m->scale, N, K, x, T, y, ldy) == 0) return;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const int8_t* w = m->w + (size_t)n * K;
    float s = m->scale[n];
    for (int t = 0; t < T; ++t) {
      const float* xr = x + (size_t)t * K;
      double tot = 0.0;
      for (int k0 = 0; k0 < K; k0 += 32) {
        float acc = 0.f;
        int k1 = k0 + 32 < K ? k0 + 32 : K;
#pragma omp simd reduction(+ : acc)
        for (int k = k0; k < k1; ++k) acc += (float)w[k] * xr[k];
        tot += (double)acc;
      }
      y[(size_t)t * ldy + n] = (float)tot * s;
    }
  }
}

static void rmsnorm(const float* x, const float* g, int n, float eps, float* y) {
  double ss = 0.0;
  for (int i = 0; i < n; ++i) ss += (double)x[i] * (double)x[i];
  float r = (float)(1.0 / sqrt(ss / (double)n + (double)eps));
  for (int i = 0; i < n; ++i) y[i] = x[i] * r * g[i];
}

/* Round-to-nearest-even to bfloat16 precision (what a bf16 KV cache stores). */
static float bf16_round(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7F800000u) == 0x7F800000u) return x;
  u += 0x7FFFu + ((u >> 16) & 1u);
  u &= 0xFFFF0000u;
  memcpy(&x, &u, 4);
  return x;
}

static float gelu_tanh(float x) {
  const float c = 0.7978845608028654f; /* sqrt(2/pi) */
  return 0.5f * x * (1.0f + tanhf(c * (x + 0.044715f * x * x * x)));
}

/* --------------------------------------------------------- the executor */

typedef struct {
  OrcModel* m;
  float** kcache; /* per layer: [n_pages][hkv][ORC_PAGE][hd] */
  float** vcache;
  int n_pages;
  int current_step;
  int next_input_token_id; /* -1 = none pending */
  int last_plan_n;
  int last_plan_bucket[64], last_plan_len[64];
  int n_layers; /* copy: the model may be released first */
} OrcExec;

OrcExec* orc_exec_create(OrcModel* m) {
  OrcExec* e = (OrcExec*)calloc(1, sizeof *e);
  const OrcCfg* c = &m->cfg;
  e->m = m;
  e->n_layers = c->n_layers;
  e->n_pages = (c->max_ctx + ORC_PAGE - 1) / ORC_PAGE;
  size_t per = (size_t)e->n_pages * c->hkv * ORC_PAGE * c->hd;
  e->kcache = (float**)calloc((size_t)c->n_layers, sizeof(float*));
  e->vcache = (float**)calloc((size_t)c->n_layers, sizeof(float*));
  for (int i = 0; i < c->n_layers; ++i) {
    e->kcache[i] = (float*)calloc(per, sizeof(float));
    e->vcache[i] = (float*)calloc(per, sizeof(float));
  }
  e->current_step = 0;
  e->next_input_token_id = -1;
  return e;
}

void orc_exec_destroy(OrcExec* e) {
  if (!e) return;
  for (int i = 0; i < e->n_layers; ++i) { free(e->kcache[i]); free(e->vcache[i]); }
  free(e->kcache); free(e->vcache); free(e);
}

/* Runs n tokens at consecutive positions start..start+n-1 through all layers.
 * logits (vocab floats) is filled for the LAST token when non-NULL.
 * hidden_out (n*d floats) receives the final residual stream when non-NULL. */
static int forward(OrcExec* e, const int32_t* tokens, int n, int start,
                   float* logits, float* hidden_out) {
  const OrcModel* m = e->m;
  const OrcCfg* c = &m->cfg;
  int d = c->d, hd = c->hd, hq = c->hq, hkv = c->hkv, ffn = c->ffn, half = hd / 2;
  int nq = hq * hd, nkv = hkv * hd, nqkv = nq + 2 * nkv, grp = hq / hkv;
  if (start + n > c->max_ctx) return 3;
  float* x = (float*)malloc(sizeof(float) * (size_t)n * d);
  float* h = (float*)malloc(sizeof(float) * (size_t)n * (d > ffn ? d : ffn));
  float* qkv = (float*)malloc(sizeof(float) * (size_t)n * nqkv);
  float* att = (float*)malloc(sizeof(float) * (size_t)n * nq);
  float* tmp = (float*)malloc(sizeof(float) * (size_t)n * d);
  float* gate = (float*)malloc(sizeof(float) * (size_t)n * ffn);
  float* up = (float*)malloc(sizeof(float) * (size_t)n * ffn);
  float emb_scale = sqrtf((float)d);
  for (int t = 0; t < n; ++t) {
    int tok = tokens[t];
    if (tok < 0 || tok >= c->vocab) { free(x); free(h); free(qkv); free(att); free(tmp); free(gate); free(up); return 3; }
    const int8_t* row = m->embed.w + (size_t)tok * d;
    float s = m->embed.scale[tok];
    for (int i = 0; i < d; ++i) x[(size_t)t * d + i] = (float)row[i] * s * emb_scale;
  }
  float att_scale = 1.0f / sqrtf((float)hd);
  for (int li = 0; li < c->n_layers; ++li) {
    const OrcLayer* L = &m->layers[li];
    int is_global = (li % c->period) == c->period - 1;
    const float* ct = m->rope_cos[is_global];
    const float* st = m->rope_sin[is_global];
    for (int t = 0; t < n; ++t) rmsnorm(x + (size_t)t * d, L->g_pre_attn, d, c->eps, h + (size_t)t * d);
    matmul_w4(&L->wqkv, h, n, qkv, nqkv);
    /* q/k norm, RoPE, KV append */
    for (int t = 0; t < n; ++t) {
      int pos = start + t;
      float* row = qkv + (size_t)t * nqkv;
      for (int hh = 0; hh < hq + hkv; ++hh) {
        float* v = row + (size_t)hh * hd;
        rmsnorm(v, hh < hq ? L->g_q : L->g_k, hd, c->eps, v);
        for (int j = 0; j < half; ++j) {
          float cs = ct[(size_t)pos * half + j], sn = st[(size_t)pos * half + j];
          float a = v[j], b = v[j + half];
          v[j] = a * cs - b * sn;
          v[j + half] = b * cs + a * sn;
        }
      }
      int page, slot;
      orc_kv_index(pos, &page, &slot);
      for (int kh = 0; kh < hkv; ++kh) {
        int64_t off = orc_kv_offset(page, kh, slot, hkv, hd);
        memcpy(e->kcache[li] + off, row + nq + (size_t)kh * hd, sizeof(float) * hd);
        memcpy(e->vcache[li] + off, row + nq + nkv + (size_t)kh * hd, sizeof(float) * hd);
        if (c->kv_dtype == 1)
          for (int j = 0; j < hd; ++j) {
            e->kcache[li][off + j] = bf16_round(e->kcache[li][off + j]);
            e->vcache[li][off + j] = bf16_round(e->vcache[li][off + j]);
          }
      }
    }
    /* attention */
#pragma omp parallel for schedule(dynamic, 4)
    for (int th = 0; th < n * hq; ++th) {
      int t = th / hq, qh = th % hq, kh = qh / grp;
      int pos = start + t;
      int lo = 0;
      if (!is_global && pos - c->window + 1 > 0) lo = pos - c->window + 1;
      const float* q = qkv + (size_t)t * nqkv + (size_t)qh * hd;
      int nk = pos - lo + 1;
      float* sc = (float*)malloc(sizeof(float) * (size_t)nk);
      float mx = -INFINITY;
      for (int kp = lo; kp <= pos; ++kp) {
        int page, slot;
        orc_kv_index(kp, &page, &slot);
        const float* kr = e->kcache[li] + orc_kv_offset(page, kh, slot, hkv, hd);
        double dot = 0.0;
        for (int j = 0; j < hd; ++j) dot += (double)q[j] * (double)kr[j];
        float s = (float)dot * att_scale;
        sc[kp - lo] = s;
        if (s > mx) mx = s;
      }
      double sum = 0.0;
      for (int i = 0; i < nk; ++i) { sc[i] = expf(sc[i] - mx); sum += sc[i]; }
      float* o = att + (size_t)t * nq + (size_t)qh * hd;
      double* acc = (double*)calloc((size_t)hd, sizeof(double));
      for (int kp = lo; kp <= pos; ++kp) {
        int page, slot;
        orc_kv_index(kp, &page, &slot);
        const float* vr = e->vcache[li] + orc_kv_offset(page, kh, slot, hkv, hd);
        double p = sc[kp - lo];
        for (int j = 0; j < hd; ++j) acc[j] += p * (double)vr[j];
      }
      for (int j = 0; j < hd; ++j) o[j] = (float)(acc[j] / sum);
      free(acc);
      free(sc);
    }
    matmul_w4(&L->wo, att, n, tmp, d);
    for (int t = 0; t < n; ++t) {
      float* a = tmp + (size_t)t * d;
      rmsnorm(a, L->g_post_attn, d, c->eps, a);
      float* xr = x + (size_t)t * d;
      for (int i = 0; i < d; ++i) xr[i] += a[i];
      rmsnorm(xr, L->g_pre_ffn, d, c->eps, h + (size_t)t * d);
    }
    matmul_w4(&L->wgate, h, n, gate, ffn);
    matmul_w4(&L->wup, h, n, up, ffn);
    for (size_t i = 0; i < (size_t)n * ffn; ++i) gate[i] = gelu_tanh(gate[i]) * up[i];
    matmul_w4(&L->wdown, gate, n, tmp, d);
    for (int t = 0; t < n; ++t) {
      float* a = tmp + (size_t)t * d;
      rmsnorm(a, L->g_post_ffn, d, c->eps, a);
      float* xr = x + (size_t)t * d;
      for (int i = 0; i < d; ++i) xr[i] += a[i];
    }
  }
  if (hidden_out) memcpy(hidden_out, x, sizeof(float) * (size_t)n * d);
  if (logits) {
    rmsnorm(x + (size_t)(n - 1) * d, m->g_final, d, c->eps, h);
    matmul_w4(&m->embed, h, 1, logits, c->vocab);
  }
  free(x); free(h); free(qkv); free(att); free(tmp); free(gate); free(up);
  return 0;
}

/* executor.cc:157-276 restated: a group of `len` ids runs the pending id (if
 * any) followed by ids[0..len-2]; ids[len-1] becomes the pending id.  A 1-id
 * group therefore runs nothing and REPLACES the pending id. */
static int prefill_group(OrcExec* e, const int32_t* ids, int len) {
  int32_t* run = (int32_t*)malloc(sizeof(int32_t) * (size_t)(len + 1));
  int n = 0, start = e->current_step;
  for (int i = 0; i < len - 1;) {
    if (e->next_input_token_id != -1) {
      run[n++] = e->next_input_token_id;
      e->next_input_token_id = -1;
    } else {
      run[n++] = ids[i++];
    }
    e->current_step++;
  }
  e->next_input_token_id = ids[len - 1];
  int rc = 0;
  if (n > 0) rc = forward(e, run, n, start, NULL, NULL);
  free(run);
  return rc;
}

/* executor.cc:90-155.  Returns an absl::StatusCode integer. */
int orc_exec_prefill(OrcExec* e, const int32_t* ids, int n) {
  if (n <= 0) return 13; /* RET_CHECK_GT -> Internal */
  const OrcCfg* c = &e->m->cfg;
  int ng = orc_plan_work_groups(c->buckets, c->n_buckets, n, e->last_plan_bucket,
                                e->last_plan_len, 64);
  if (ng < 0) return 13;
  e->last_plan_n = ng;
  int used = 0;
  for (int g = 0; g < ng; ++g) {
    int rc = prefill_group(e, ids + used, e->last_plan_len[g]);
    if (rc) return rc;
    used += e->last_plan_len[g];
  }
  if (used != n) return 13; /* "Work groups not covering the entire prefill input." */
  return 0;
}

/* executor.cc:416-534.  id_or_null: explicit token, else the pending one. */
int orc_exec_decode_logits(OrcExec* e, const int32_t* id_or_null, float* logits) {
  int id = e->next_input_token_id;
  if (id_or_null) id = *id_or_null;
  if (id == -1) return 3; /* "No id available to be decoded." */
  e->next_input_token_id = -1;
  int32_t tok = id;
  int rc = forward(e, &tok, 1, e->current_step, logits, NULL);
  if (rc) return rc;
  e->current_step++;
  return 0;
}

/* executor.cc:278-298: logits -> greedy id (negative -> 0) -> pending id. */
int orc_exec_decode_token(OrcExec* e, int32_t* out_id, float* logits_scratch) {
  int rc = orc_exec_decode_logits(e, NULL, logits_scratch);
  if (rc) return rc;
  int32_t id;
  orc_greedy(logits_scratch, e->m->cfg.vocab, 1, &id);
  if (id < 0) id = 0;
  *out_id = id;
  e->next_input_token_id = id;
  return 0;
}

/* executor.cc:568-574: counters only; cache contents stay. */
void orc_exec_reset(OrcExec* e) {
  e->current_step = 0;
  e->next_input_token_id = -1;
}

/* executor.h:95-97. */
int orc_exec_current_step(const OrcExec* e) {
  return e->current_step + (e->next_input_token_id == -1 ? 0 : 1);
}
int orc_exec_internal_step(const OrcExec* e) { return e->current_step; }
int orc_exec_pending_token(const OrcExec* e) { return e->next_input_token_id; }
int orc_exec_last_plan(const OrcExec* e, int* buckets, int* lens) {
  for (int i = 0; i < e->last_plan_n; ++i) { buckets[i] = e->last_plan_bucket[i]; lens[i] = e->last_plan_len[i]; }
  return e->last_plan_n;
}

/* Copies one cached K or V row (head_dim floats) for inspection. */
void orc_exec_read_kv(const OrcExec* e, int layer, int is_v, int kv_head, int pos,
                      float* out) {
  int page, slot;
  orc_kv_index(pos, &page, &slot);
  const float* base = is_v ? e->vcache[layer] : e->kcache[layer];
  memcpy(out, base + orc_kv_offset(page, kv_head, slot, e->m->cfg.hkv, e->m->cfg.hd),
         sizeof(float) * (size_t)e->m->cfg.hd);
}

/* ------------------------------------------- operator-level restatements */

/* y[t][n] for a canonical packed matrix; used to check the GEMV/GEMM kernels. */
void orc_matmul_w4(const uint8_t* packed, const float* scale, int N, int K,
                   const float* x, int T, float* y) {
  OrcMat m;
  m.rows = N; m.cols = K; m.scale = scale;
  m.w = (int8_t*)malloc((size_t)N * K);
  orc_unpack_int4(packed, N, K, m.w);
  matmul_w4(&m, x, T, y, N);
  free(m.w);
}

/* Attention over explicit tensors: q [T][hq][hd], k/v [S][hkv][hd] (fp32),
 * query t sits at position qpos0 + t, key s at position s.  window <= 0 means
 * global.  out [T][hq][hd]. */
void orc_attention(const float* q, const float* k, const float* v, int T, int S,
                   int hq, int hkv, int hd, int qpos0, int window, float* out) {
  int grp = hq / hkv;
  float scale = 1.0f / sqrtf((float)hd);
#pragma omp parallel for schedule(dynamic, 4)
  for (int th = 0; th < T * hq; ++th) {
    int t = th / hq, qh = th % hq, kh = qh / grp, pos = qpos0 + t;
    int hi = pos < S - 1 ? pos : S - 1, lo = 0;
    if (window > 0 && pos - window + 1 > 0) lo = pos - window + 1;
    float* o = out + ((size_t)t * hq + qh) * hd;
    if (hi < lo) { memset(o, 0, sizeof(float) * hd); continue; }
    int nk = hi - lo + 1;
    float* sc = (float*)malloc(sizeof(float) * (size_t)nk);
    const float* qr = q + ((size_t)t * hq + qh) * hd;
    float mx = -INFINITY;
    for (int s = lo; s <= hi; ++s) {
      const float* kr = k + ((size_t)s * hkv + kh) * hd;
      double dot = 0.0;
      for (int j = 0; j < hd; ++j) dot += (double)qr[j] * (double)kr[j];
      sc[s - lo] = (float)dot * scale;
      if (sc[s - lo] > mx) mx = sc[s - lo];
    }
    double sum = 0.0;
    for (int i = 0; i < nk; ++i) { sc[i] = expf(sc[i] - mx); sum += sc[i]; }
    double* acc = (double*)calloc((size_t)hd, sizeof(double));
    for (int s = lo; s <= hi; ++s) {
      const float* vr = v + ((size_t)s * hkv + kh) * hd;
      double p = sc[s - lo];
      for (int j = 0; j < hd; ++j) acc[j] += p * (double)vr[j];
    }
    for (int j = 0; j < hd; ++j) o[j] = (float)(acc[j] / sum);
    free(acc);
    free(sc);
  }
}

// Host-side classes of the B200 executor library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <map>
#include <memory>
#include <utility>
#include <vector>

#include "../../include/b200lm.h"
#include "common.cuh"
#include "decode_ops.cuh"
#include "decode_fused.cuh"
#include "decode_wide.cuh"
#include "tp_nccl.h"

namespace b200lm {

// Tensor-core GEMM copies of the layer matrices (128-row x 64-k blocks).
struct LayerGemmWeights {
  const uint8_t *wqkv, *wo, *wgu, *wdown;
  const float *sqkv, *so, *sgu, *sdown;
};

// Device-resident weights of one decoder; shared by every executor created
// over it.
struct Model {
  int device = 0;
  ModelDims dims{};
  bool has_tc = false;
  const uint8_t* embed_rows = nullptr;
  const float* embed_scale = nullptr;
  const uint4* head_w = nullptr;
  const uint8_t* head_g = nullptr;   // the head in the tensor-core GEMM's layout (wide decode), with has_tc
  const float* head_gs = nullptr;
  const float* g_final = nullptr;
  float gmax_final = 0.f;
  const float* rope_cos[2] = {nullptr, nullptr};
  const float* rope_sin[2] = {nullptr, nullptr};
  std::vector<LayerWeights> layers_host;
  std::vector<LayerGemmWeights> gemm_host;
  std::vector<float> attn_bound;     // per layer: sqrt(hd) max|g_q| max|g_k| >= any |q.k| / sqrt(hd)
  const LayerWeights* layers_dev = nullptr;
  // layouts of the chained decode kernel (see ChainedLayer)
  int o_slices = 1;                  // head slices of the o-proj (K split by whole heads, 64-wide at least)
  std::vector<ChainedLayer> chained_host;
  const ChainedLayer* chained_dev = nullptr;
  const unsigned char* head_ws = nullptr;
  const float* gH = nullptr;
  const float* rope_cs[2] = {nullptr, nullptr};
  std::vector<void*> allocations;

  ~Model();
  void* alloc(size_t bytes);
  static std::shared_ptr<Model> load(const uint8_t* image, size_t n, int device, bool want_tc);
};

// An activation matrix [rows][cols] bf16 as the GEMM's token operand: the same tensor with a 128-row and a
// 64-row copy box (the kernel's token tile is 256 / 128 or 64 wide).
struct ActMap {
  CUtensorMap box128;
  CUtensorMap box64;
};
// token width of the GEMM tile for T token rows
inline int ts_tile_tokens(int T) { return T <= 64 ? 64 : T <= 128 ? 128 : 256; }
CUtensorMap make_activation_map_box(const __nv_bfloat16* base, int rows, int cols, int box_rows);
ActMap make_activation_map(const __nv_bfloat16* base, int rows, int cols);
int pick_ksplit(int T, int n_tiles, int KB, int sms);
void launch_gemm(cudaStream_t st, int mode, const ActMap& a_map, const __nv_bfloat16* A, const uint4* w4t,
                 const float* s4t, const uint8_t* w4g, const float* s4g, int T, int N, int K, int ksplit, bool geglu,
                 float* outF, __nv_bfloat16* outB, int* err, int64_t* launches);

// One session: KV cache, step counter, pending token, scratch activations.
class Executor {
 public:
  static std::unique_ptr<Executor> create(std::shared_ptr<Model> model, const B200LmConfig& cfg);
  ~Executor();

  void prefill(const int* ids, int n, bool wait, const volatile int* cancel);
  void decode_logits(const int* id_or_null, float* host_logits);
  void decode_tokens(int nsteps, int* out_ids);
  void reset();
  // several sessions in one executor (own KV pages, step counter and pending id each; one weight copy)
  void select_session(int session);                 // the calls above then act on that session
  void decode_tokens_batch(int nsteps, int* out_ids /* [nsteps][n_sessions] */);
  void check_device_error(const char* where);
  void trace_decode_step(int* out_id, long long* stamps, long long capacity, int* n_barriers, int* n_cta, int* khz);
  void read_kv_row(int layer, int is_v, int kv_head, int pos, float* out, int* page, int* slot);
  void tp_allreduce(float* buf, size_t count);      // sum over the tensor-parallel ranks, in place, on `stream`

  std::shared_ptr<Model> model;
  int device = 0;
  int n_sms = 0;
  int tp_rank = 0, tp_world = 1;
  size_t smem_optin = 0;            // opt-in shared memory per block of the device
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int max_num_tokens = 0;
  int prefill_gemm = 0, decode_mode = 0;
  // reference state machine (llm_litert_compiled_model_executor.h: current_step_, next_input_token_id_)
  int current_step = 0;
  int next_input_token = -1;
  std::vector<std::pair<int, int>> last_plan;
  int n_sessions = 1;
  int active = 0;                                   // session the three fields above belong to
  struct SessionState {
    int current_step = 0;
    int next_input_token = -1;
    std::vector<std::pair<int, int>> last_plan;
  };
  std::vector<SessionState> parked;                 // state of the sessions that are not active
  int64_t launches = 0;
  size_t h2d_bytes = 0, d2h_bytes = 0;

 private:
  Executor() = default;
  void* alloc(size_t bytes, bool zero);
  void run_prefill_chunk(const int* tokens, int T, int start);
  void prefill_group(const int* ids, int len);
  void launch_decode_steps(int nsteps, int ncols = 1, int first_session = -1);
  void push_decode_state(const int* tokens, const int* pos, int ncols);
  int take_decode_id(const int* id_or_null);

  std::vector<void*> allocations;
  std::vector<LayerKv> kv_host;
  const LayerKv* kv_dev = nullptr;
  std::vector<int> page_table_host;
  const int* page_table_dev = nullptr;
  int pages_per_seq = 0;
  DecodeArgs dargs{};
  size_t dec_smem = 0;
  size_t stream_smem = 0;
  int stream_half = 0;
  // tensor parallelism: sum over the ranks of a buffer of partial projections, on the executor's stream
  NcclApi::Comm tp_comm = nullptr;
  unsigned barrier_epoch = 0;
  // chained decode kernel: exchange area (two parity copies of flag-carrying words) and the next free tag
  fu_u64* ll_dev = nullptr;
  size_t ll_bytes = 0;
  unsigned ll_tag = 0;
  FusedPlan last_plan_ll{};         // plan of the last chained launch (diagnostics of a wait that gave up)
  int last_ncols = 1;
  bool chained_ok = false;          // the model fits the chained kernel (with n_sessions columns)
  long long* trace_dev = nullptr;
  cudaGraphExec_t graph_exec = nullptr;
  // wide lockstep decode (B200LM_DECODE_WIDE)
  WideState wide{nullptr, nullptr, nullptr};
  float* wide_part = nullptr;       // key-split partial states of the wide attention
  int* pin_wide = nullptr;          // staging of the wide state words
  std::map<std::pair<int, int>, cudaGraphExec_t> wide_graphs;   // one step, keyed by (sessions, first session)
  int64_t wide_per_step = 0;        // kernel launches of one wide step
  void wide_step(int nb, int first);
  void launch_wide_steps(int nsteps, int nb, int first);
  // prefill scratch
  int t_max = 0, t_pad = 0;
  int* pf_tokens = nullptr;
  float* pf_xres = nullptr;
  __nv_bfloat16* pf_h = nullptr;
  float* pf_qkv = nullptr;
  __nv_bfloat16* pf_attn = nullptr;
  __nv_bfloat16* pf_act = nullptr;
  float* pf_parts = nullptr;
  ActMap tm_h{}, tm_attn{}, tm_act{};
  bool attn_tc = false;             // tensor-core prefill attention in use
  __nv_bfloat16* pf_q = nullptr;    // [t_pad][hq][hd] normalised, rotated, scaled queries
  CUtensorMap tm_q{};
  std::vector<CUtensorMap> tm_k, tm_vt;   // per layer
  // pinned staging
  static constexpr int kTokRing = 4;    // prompt-id slices that may be queued for upload at once
  void* pinned = nullptr;
  float* pin_logits = nullptr;
  int* pin_ints = nullptr;          // kTokRing slices of t_pad ids
  int* pin_steps = nullptr;         // ids sampled by a multi-step decode call
  cudaEvent_t tok_ring_done[kTokRing] = {nullptr, nullptr, nullptr, nullptr};
  bool tok_ring_used[kTokRing] = {false, false, false, false};
  int tok_ring_next = 0;
  DecodeState* pin_state = nullptr;
};

}  // namespace b200lm

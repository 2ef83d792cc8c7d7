// Drives B200LlmExecutor (the LlmExecutorBase adapter) the way
// runtime/core/pipeline.cc drives an executor: Prefill with an ExecutorInputs
// holding int32 ids [1, n], then Decode(output_tokens) in a loop, then
// DecodeLogits with an explicit id.  Prints what it saw as key=value lines for
// the Python test to compare with the C ABI driven directly.
//   adapter_driver <model.litertlm> <n_decode> <id0> <id1> ...
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "b200_llm_executor.h"

using namespace litert::lm;

int main(int argc, char** argv) {
  if (argc < 4) return 2;
  B200LmConfig cfg{};
  cfg.struct_size = sizeof(cfg);
  auto ex_or = B200LlmExecutor::Create(argv[1], cfg, LlmExecutorSettings());
  if (!ex_or.ok()) {
    std::printf("create_code=%d\ncreate_msg=%s\n", (int)ex_or.status().code(), ex_or.status().message().c_str());
    return 0;
  }
  auto& ex = *ex_or.value();
  int n_decode = std::atoi(argv[2]);
  std::vector<int32_t> ids;
  for (int i = 3; i < argc; ++i) ids.push_back(std::atoi(argv[i]));
  // ids as the caller loop hands them over: CopyToTensorBuffer<int>(ids, {1, n}) (runtime/core/pipeline.cc:257-262)
  auto buf = CopyToTensorBuffer<int32_t>(absl::MakeConstSpan(ids), {1, (int32_t)ids.size()});
  ExecutorInputs inputs{ExecutorTextData(std::move(*buf))};
  ExecutorPrefillParams params;
  params.SetWaitForCompletion(true);
  absl::Status st = ex.Prefill(inputs, params);
  std::printf("backend=%s\nprefill_code=%d\nstep_after_prefill=%d\nvocab=%d\n", std::string(ex.ExecutorBackendName()).c_str(),
              (int)st.code(), ex.GetCurrentStep().value(), ex.GetVocabSize().value());
  // what TryGetMaxNumTokens (runtime/core/pipeline.cc:51-62) would read
  auto settings = ex.GetExecutorSettings();
  std::printf("max_num_tokens=%d\n", settings.ok() ? (int)settings->GetMaxNumTokens() : -1);
  auto out_or = CreateTensorBuffer<int32_t>({1, 1});
  auto& out = *out_or;
  std::printf("tokens=");
  for (int i = 0; i < n_decode; ++i) {
    st = ex.Decode(out);
    if (!st.ok()) { std::printf("!%d", (int)st.code()); break; }
    std::printf("%d,", (*CopyFromTensorBuffer<int32_t>(out))[0]);
  }
  std::printf("\n");
  std::vector<int32_t> first{ids[0]};
  auto one = CopyToTensorBuffer<int32_t>(absl::MakeConstSpan(first), {1, 1});
  auto logits_or = ex.DecodeLogits(ExecutorInputs{ExecutorTextData(std::move(*one))});
  if (logits_or.ok()) {
    auto l = *CopyFromTensorBuffer<float>(*logits_or);
    int best = 0, v = ex.GetVocabSize().value();
    for (int i = 1; i < v; ++i) if (l[best] < l[i]) best = i;
    std::printf("logits_dims=%zu\nlogits_argmax=%d\nlive_locks=%d\n", logits_or->TensorType()->Layout().Dimensions().size(), best,
                logits_or->LiveLocks());
  }
  // a cancel flag that is already raised stops the call before any work group runs
  {
    std::atomic_bool cancel{true};
    ExecutorPrefillParams cp;
    cp.SetWaitForCompletion(true);
    cp.SetCancelFlag(&cancel);
    auto again = CopyToTensorBuffer<int32_t>(absl::MakeConstSpan(ids), {1, (int32_t)ids.size()});
    absl::Status cs = ex.Prefill(ExecutorInputs{ExecutorTextData(std::move(*again))}, cp);
    std::printf("cancelled_prefill_code=%d\n", (int)cs.code());
  }
  // ids that are not int32 are refused like ReferTensorBufferAsSpan refuses them
  {
    auto wrong = CreateTensorBuffer<float>({1, 4});
    absl::Status ws = ex.Prefill(ExecutorInputs{ExecutorTextData(std::move(*wrong))});
    std::printf("float_ids_code=%d\n", (int)ws.code());
  }
  std::printf("step_end=%d\n", ex.GetCurrentStep().value());
  st = ex.Decode(ExecutorInputs(), out);      // no pending id, none given -> must fail, wrong buffer size first
  std::printf("undersized_logits_code=%d\n", (int)st.code());
  st = ex.Reset();
  std::printf("reset_code=%d\nstep_after_reset=%d\n", (int)st.code(), ex.GetCurrentStep().value());
  auto l2 = ex.DecodeLogits(ExecutorInputs());
  std::printf("decode_without_id_code=%d\n", (int)l2.status().code());
  return 0;
}

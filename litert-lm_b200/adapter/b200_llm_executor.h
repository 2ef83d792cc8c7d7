// B200LlmExecutor — the C++ face of libb200lm.so inside LiteRT-LM.
//
// A header-only subclass of litert::lm::LlmExecutorBase
// (runtime/executor/llm_executor_base.h:33-121) that forwards every call to the
// C ABI in include/b200lm.h, so runtime/core/pipeline.cc and the Session code
// drive it exactly as they drive LlmLiteRtCompiledModelExecutor:
//   Prefill(inputs[, params])      -> B200Lm_Prefill
//   Decode(output_tokens)          -> B200Lm_DecodeToken
//   Decode(inputs, output_logits)  -> B200Lm_DecodeLogits
//   DecodeLogits(inputs)           -> B200Lm_DecodeLogits into a new [1,1,V] host buffer
//   GetVocabSize / GetCurrentStep / Reset / ExecutorBackendName
// Checks that the reference performs before touching the model are kept: batch
// must be 1 and the id tensor non-empty (llm_litert_compiled_model_executor.cc:92-97),
// an explicit decode id must be exactly one int32 (:303-315).
//
// ONE body for both builds: against the real headers when B200LM_WITH_LITERT_LM is
// defined, otherwise against litert_shim.h, which offers the same names and
// signatures for the subset used here (TensorType().Layout().Dimensions(),
// ReferTensorBufferAsSpan, TensorBufferScopedLock::Create, CreateTensorBuffer).
#pragma once
#include <atomic>
#include <chrono>
#include <cstdlib>
#include <memory>
#include <string>
#include <thread>
#include <utility>

#include "b200lm.h"

#ifdef B200LM_WITH_LITERT_LM
#include "runtime/executor/llm_executor_base.h"
#include "runtime/executor/llm_executor_settings.h"
#include "runtime/util/convert_tensor_buffer.h"
#else
#include "litert_shim.h"
#endif

namespace litert::lm {

class B200LlmExecutor : public LlmExecutorBase {
 public:
  // model_path: a `.litertlm` file holding an int4 decoder weights record.  `settings`
  // is what the engine built for this executor (LlmExecutorSettings::CreateDefault);
  // its max_num_tokens is overwritten with the capacity of the KV cache, which is
  // what GetExecutorSettings() must report (runtime/core/pipeline.cc:51-62).
  static absl::StatusOr<std::unique_ptr<B200LlmExecutor>> Create(const std::string& model_path, const B200LmConfig& config,
                                                                 LlmExecutorSettings settings) {
    B200LmExecutor* h = nullptr;
    char* err = nullptr;
    int rc = B200Lm_Create(&config, nullptr, 0, model_path.c_str(), &h, &err);
    if (rc != 0) return ToStatus(rc, err);
    return std::unique_ptr<B200LlmExecutor>(new B200LlmExecutor(h, std::move(settings)));
  }
  static absl::StatusOr<std::unique_ptr<B200LlmExecutor>> CreateFromBytes(const void* bytes, uint64_t n, const B200LmConfig& config,
                                                                          LlmExecutorSettings settings) {
    B200LmExecutor* h = nullptr;
    char* err = nullptr;
    int rc = B200Lm_Create(&config, bytes, n, nullptr, &h, &err);
    if (rc != 0) return ToStatus(rc, err);
    return std::unique_ptr<B200LlmExecutor>(new B200LlmExecutor(h, std::move(settings)));
  }
  ~B200LlmExecutor() override { B200Lm_Destroy(h_); }

  absl::Status Prefill(const ExecutorInputs& inputs) override { return Prefill(inputs, ExecutorPrefillParams()); }

  absl::Status Prefill(const ExecutorInputs& inputs, const ExecutorPrefillParams& params) override {
    auto ids_or = inputs.GetTextTokenIdsPtr();
    if (!ids_or.ok()) return ids_or.status();
    const ::litert::TensorBuffer& ids = **ids_or;
    auto type = ids.TensorType();
    if (!type) return absl::InternalError("token ids have no tensor type");
    auto dims = type->Layout().Dimensions();
    if (dims.size() != 2) return absl::InvalidArgumentError("token ids must be [batch, sequence_length]");
    auto span = ReferTensorBufferAsSpan<int32_t>(ids);
    if (!span) return absl::InvalidArgumentError("token ids must be int32 in host memory");
    if (dims[0] != 1) return absl::InternalError("Only batch size 1 is accepted.");
    if (dims[1] <= 0 || span->empty()) return absl::InternalError("Prefill token ids must be non-empty.");
    // The C ABI polls an int32 word between work groups; the caller's flag is a
    // std::atomic_bool.  While the call runs, a helper thread mirrors the flag into
    // the word, so a cancel raised in the middle of a long prompt is seen at the
    // next work group, not only one raised before the call.
    volatile int32_t cancel_word = 0;
    const std::atomic_bool* cancel = params.GetCancelFlag();
    std::atomic<bool> call_done{false};
    std::thread mirror;
    if (cancel != nullptr) {
      if (cancel->load()) cancel_word = 1;
      mirror = std::thread([&] {
        while (!call_done.load(std::memory_order_acquire)) {
          if (cancel->load()) cancel_word = 1;
          std::this_thread::sleep_for(std::chrono::microseconds(100));
        }
      });
    }
    char* err = nullptr;
    int rc = B200Lm_Prefill(h_, span->data(), (int32_t)dims[1], params.GetWaitForCompletion() ? 1 : 0,
                            cancel ? &cancel_word : nullptr, &err);
    if (mirror.joinable()) {
      call_done.store(true, std::memory_order_release);
      mirror.join();
    }
    return ToStatus(rc, err);
  }

  absl::Status Decode(::litert::TensorBuffer& output_tokens) override {
    auto size = output_tokens.Size();
    if (!size || *size < sizeof(int32_t)) return absl::InvalidArgumentError("output_tokens must hold one int32");
    char* err = nullptr;
    int32_t id = -1;
    int rc = B200Lm_DecodeToken(h_, &id, &err);
    if (rc != 0) return ToStatus(rc, err);
    // the lock lives until the id has been written
    auto lock_and_addr = ::litert::TensorBufferScopedLock::Create(output_tokens, ::litert::TensorBuffer::LockMode::kWrite);
    if (!lock_and_addr) return absl::InternalError("cannot map output_tokens");
    static_cast<int32_t*>(lock_and_addr->second)[0] = id;
    return absl::OkStatus();
  }

  absl::Status Decode(const ExecutorInputs& inputs, ::litert::TensorBuffer& output_logits) override {
    int vocab = 0;
    B200Lm_GetVocabSize(h_, &vocab, nullptr);
    auto size = output_logits.Size();
    if (!size || *size < sizeof(float) * (size_t)vocab)
      return absl::InvalidArgumentError("output_logits is smaller than [1, 1, vocab] float32");
    int32_t id = 0;
    bool has_id = false;
    absl::Status st = ExplicitId(inputs, &id, &has_id);
    if (!st.ok()) return st;
    // the lock lives across the call that writes the logits
    auto lock_and_addr = ::litert::TensorBufferScopedLock::Create(output_logits, ::litert::TensorBuffer::LockMode::kWrite);
    if (!lock_and_addr) return absl::InternalError("cannot map output_logits");
    char* err = nullptr;
    int rc = B200Lm_DecodeLogits(h_, has_id ? &id : nullptr, static_cast<float*>(lock_and_addr->second), &err);
    return ToStatus(rc, err);
  }

  absl::StatusOr<::litert::TensorBuffer> DecodeLogits(const ExecutorInputs& inputs) override {
    int vocab = 0;
    B200Lm_GetVocabSize(h_, &vocab, nullptr);
    auto logits = CreateTensorBuffer<float>({1, 1, vocab});       // as fake_llm_executor.cc:159-161 shapes them
    if (!logits) return absl::InternalError("cannot allocate the logits buffer");
    absl::Status st = Decode(inputs, *logits);
    if (!st.ok()) return st;
    return std::move(*logits);
  }

  absl::string_view ExecutorBackendName() const override { return B200Lm_BackendName(); }

  absl::StatusOr<int> GetVocabSize() override {
    int v = 0;
    char* err = nullptr;
    int rc = B200Lm_GetVocabSize(h_, &v, &err);
    if (rc != 0) return ToStatus(rc, err);
    return v;
  }

  absl::StatusOr<int> GetCurrentStep() const override {
    int v = 0;
    char* err = nullptr;
    int rc = B200Lm_GetCurrentStep(h_, &v, &err);
    if (rc != 0) return ToStatus(rc, err);
    return v;
  }

  // Settings whose GetMaxNumTokens() is the KV capacity: without this override the
  // caller loop assumes 4096 tokens (runtime/core/pipeline.cc:51-62).
  absl::StatusOr<LlmExecutorSettings> GetExecutorSettings() const override { return settings_; }

  absl::Status Reset() override {
    char* err = nullptr;
    return ToStatus(B200Lm_Reset(h_, &err), err);
  }

 private:
  B200LlmExecutor(B200LmExecutor* h, LlmExecutorSettings settings) : h_(h), settings_(std::move(settings)) {
    int v = 0;
    if (B200Lm_GetMaxNumTokens(h_, &v, nullptr) == 0 && v > 0) settings_.SetMaxNumTokens((uint64_t)v);
  }

  static absl::Status ToStatus(int rc, char* err) {
    if (rc == 0) return absl::OkStatus();
    std::string msg = err ? err : "";
    free(err);                                   // the library mallocs, the caller frees
    return absl::Status(static_cast<absl::StatusCode>(rc), msg);
  }

  // An explicit id wins over the pending one and must be exactly one int32
  // (llm_litert_compiled_model_executor.cc:303-315).
  static absl::Status ExplicitId(const ExecutorInputs& inputs, int32_t* id, bool* has_id) {
    *has_id = false;
    if (!inputs.GetTextDataPtr().ok()) return absl::OkStatus();
    auto ids_or = inputs.GetTextTokenIdsPtr();
    if (!ids_or.ok()) return absl::OkStatus();
    const ::litert::TensorBuffer& ids = **ids_or;
    auto bytes = ids.PackedSize();
    if (!bytes || *bytes == 0) return absl::OkStatus();
    if (*bytes != sizeof(int32_t)) return absl::InternalError("Decode accepts a single token id.");
    auto span = ReferTensorBufferAsSpan<int32_t>(ids);
    if (!span) return absl::InvalidArgumentError("token ids must be int32 in host memory");
    *id = (*span)[0];
    *has_id = true;
    return absl::OkStatus();
  }

  B200LmExecutor* h_;
  LlmExecutorSettings settings_;
};

}  // namespace litert::lm

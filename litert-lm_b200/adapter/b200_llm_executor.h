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
// Built against the real headers when B200LM_WITH_LITERT_LM is defined (the
// tensor-buffer accessors then go through runtime/util/convert_tensor_buffer.h),
// otherwise against litert_shim.h.
#pragma once
#include <cstdlib>
#include <memory>
#include <string>

#include "b200lm.h"

#ifdef B200LM_WITH_LITERT_LM
#include "runtime/executor/llm_executor_base.h"
#include "runtime/util/convert_tensor_buffer.h"
#else
#include "litert_shim.h"
#endif

namespace litert::lm {

class B200LlmExecutor : public LlmExecutorBase {
 public:
  // model_path: a `.litertlm` file holding an int4 decoder weights record.
  static absl::StatusOr<std::unique_ptr<B200LlmExecutor>> Create(const std::string& model_path,
                                                                 const B200LmConfig& config) {
    B200LmExecutor* h = nullptr;
    char* err = nullptr;
    int rc = B200Lm_Create(&config, nullptr, 0, model_path.c_str(), &h, &err);
    if (rc != 0) return ToStatus(rc, err);
    return std::unique_ptr<B200LlmExecutor>(new B200LlmExecutor(h));
  }
  static absl::StatusOr<std::unique_ptr<B200LlmExecutor>> CreateFromBytes(const void* bytes, uint64_t n,
                                                                          const B200LmConfig& config) {
    B200LmExecutor* h = nullptr;
    char* err = nullptr;
    int rc = B200Lm_Create(&config, bytes, n, nullptr, &h, &err);
    if (rc != 0) return ToStatus(rc, err);
    return std::unique_ptr<B200LlmExecutor>(new B200LlmExecutor(h));
  }
  ~B200LlmExecutor() override { B200Lm_Destroy(h_); }

  absl::Status Prefill(const ExecutorInputs& inputs) override { return Prefill(inputs, ExecutorPrefillParams()); }

  absl::Status Prefill(const ExecutorInputs& inputs, const ExecutorPrefillParams& params) override {
    auto ids_or = inputs.GetTextTokenIdsPtr();
    if (!ids_or.ok()) return ids_or.status();
    const ::litert::TensorBuffer& ids = **ids_or;
    const int32_t* data = nullptr;
    int batch = 0, len = 0;
    absl::Status st = ViewIds(ids, &data, &batch, &len);
    if (!st.ok()) return st;
    if (batch != 1) return absl::InternalError("Only batch size 1 is accepted.");
    if (len <= 0) return absl::InternalError("Prefill token ids must be non-empty.");
    // std::atomic_bool is lock-free and one byte wide here; the C ABI polls an int32 flag,
    // so the adapter mirrors the flag into one before the call.
    volatile int32_t cancel_word = 0;
    const std::atomic_bool* cancel = params.GetCancelFlag();
    if (cancel != nullptr && cancel->load()) cancel_word = 1;
    char* err = nullptr;
    int rc = B200Lm_Prefill(h_, data, len, params.GetWaitForCompletion() ? 1 : 0, cancel ? &cancel_word : nullptr, &err);
    return ToStatus(rc, err);
  }

  absl::Status Decode(::litert::TensorBuffer& output_tokens) override {
    if (output_tokens.Size() < sizeof(int32_t)) return absl::InvalidArgumentError("output_tokens must hold one int32");
    char* err = nullptr;
    int32_t id = -1;
    int rc = B200Lm_DecodeToken(h_, &id, &err);
    if (rc != 0) return ToStatus(rc, err);
    static_cast<int32_t*>(LockForWrite(output_tokens))[0] = id;
    return absl::OkStatus();
  }

  absl::Status Decode(const ExecutorInputs& inputs, ::litert::TensorBuffer& output_logits) override {
    int vocab = 0;
    B200Lm_GetVocabSize(h_, &vocab, nullptr);
    if (output_logits.Size() < sizeof(float) * (size_t)vocab)
      return absl::InvalidArgumentError("output_logits is smaller than [1, 1, vocab] float32");
    int32_t id = 0;
    bool has_id = false;
    absl::Status st = ExplicitId(inputs, &id, &has_id);
    if (!st.ok()) return st;
    char* err = nullptr;
    int rc = B200Lm_DecodeLogits(h_, has_id ? &id : nullptr, static_cast<float*>(LockForWrite(output_logits)), &err);
    return ToStatus(rc, err);
  }

  absl::StatusOr<::litert::TensorBuffer> DecodeLogits(const ExecutorInputs& inputs) override {
    int vocab = 0;
    B200Lm_GetVocabSize(h_, &vocab, nullptr);
    ::litert::TensorBuffer logits = NewHostBuffer(vocab);
    absl::Status st = Decode(inputs, logits);
    if (!st.ok()) return st;
    return logits;
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

  // The value LlmExecutorSettings::GetMaxNumTokens() must report for this executor,
  // otherwise the pipeline assumes 4096 (runtime/core/pipeline.cc:51-62).
  int GetMaxNumTokens() const {
    int v = 0;
    B200Lm_GetMaxNumTokens(h_, &v, nullptr);
    return v;
  }

  absl::Status Reset() override {
    char* err = nullptr;
    return ToStatus(B200Lm_Reset(h_, &err), err);
  }

 private:
  explicit B200LlmExecutor(B200LmExecutor* h) : h_(h) {}

  static absl::Status ToStatus(int rc, char* err) {
    if (rc == 0) return absl::OkStatus();
    std::string msg = err ? err : "";
    free(err);                                   // the library mallocs, the caller frees
    return absl::Status(static_cast<absl::StatusCode>(rc), msg);
  }

#ifdef B200LM_WITH_LITERT_LM
  static absl::Status ViewIds(const ::litert::TensorBuffer& ids, const int32_t** data, int* batch, int* len) {
    auto type = ids.TensorType();
    if (!type) return absl::InternalError("token ids have no tensor type");
    auto dims = type->Layout().Dimensions();
    if (dims.size() != 2) return absl::InvalidArgumentError("token ids must be [batch, sequence_length]");
    auto span = ReferTensorBufferAsSpan<int32_t>(ids);
    if (!span) return absl::InvalidArgumentError("token ids must be int32 in host memory");
    *data = span->data(); *batch = dims[0]; *len = dims[1];
    return absl::OkStatus();
  }
  static void* LockForWrite(::litert::TensorBuffer& b) {
    auto lock = ::litert::TensorBufferScopedLock::Create(b, ::litert::TensorBuffer::LockMode::kWrite);
    return lock ? lock->second : nullptr;
  }
  static ::litert::TensorBuffer NewHostBuffer(int vocab) { return std::move(*CreateTensorBuffer<float>({1, 1, vocab})); }
#else
  static absl::Status ViewIds(const ::litert::TensorBuffer& ids, const int32_t** data, int* batch, int* len) {
    if (ids.GetElementType() != ::litert::ElementType::Int32 || !ids.IsHostMemory())
      return absl::InvalidArgumentError("token ids must be int32 in host memory");
    const auto& dims = ids.GetDimensions();
    if (dims.size() != 2) return absl::InvalidArgumentError("token ids must be [batch, sequence_length]");
    *data = static_cast<const int32_t*>(ids.Lock()); *batch = dims[0]; *len = dims[1];
    return absl::OkStatus();
  }
  static void* LockForWrite(::litert::TensorBuffer& b) { return b.Lock(); }
  static ::litert::TensorBuffer NewHostBuffer(int vocab) {
    return ::litert::TensorBuffer::CreateManagedHost(::litert::ElementType::Float32, {1, 1, vocab});
  }
#endif

  // An explicit id wins over the pending one and must be exactly one int32
  // (llm_litert_compiled_model_executor.cc:303-315).
  static absl::Status ExplicitId(const ExecutorInputs& inputs, int32_t* id, bool* has_id) {
    *has_id = false;
    if (!inputs.GetTextDataPtr().ok()) return absl::OkStatus();
    auto ids_or = inputs.GetTextTokenIdsPtr();
    if (!ids_or.ok()) return absl::OkStatus();
    const ::litert::TensorBuffer& ids = **ids_or;
    size_t bytes = ids.PackedSize();
    if (bytes == 0) return absl::OkStatus();
    if (bytes != sizeof(int32_t)) return absl::InternalError("Decode accepts a single token id.");
    const int32_t* data = nullptr;
    int batch = 0, len = 0;
    absl::Status st = ViewIds(ids, &data, &batch, &len);
    if (!st.ok()) return st;
    *id = data[0];
    *has_id = true;
    return absl::OkStatus();
  }

  B200LmExecutor* h_;
};

}  // namespace litert::lm

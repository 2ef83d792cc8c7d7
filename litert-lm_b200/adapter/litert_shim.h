// Minimal stand-ins for the absl / LiteRT / LiteRT-LM types the executor
// interface is written against, so that the adapter in b200_llm_executor.h
// compiles and is tested where those projects' headers are absent.  Inside a
// LiteRT-LM checkout define B200LM_WITH_LITERT_LM and this file is not used.
//
// Only the subset the executor's callers touch is modelled (cf.
// runtime/util/convert_tensor_buffer.h:63-231, runtime/core/pipeline.cc:104-135):
// a host-memory TensorBuffer with dimensions, element type, Size(), Duplicate()
// (shared storage), Read/Write and a scoped lock that yields the host address.
#pragma once
#include <atomic>
#include <cstdint>
#include <cstring>
#include <memory>
#include <optional>
#include <string>
#include <string_view>
#include <utility>
#include <vector>

namespace absl {
enum class StatusCode : int {
  kOk = 0, kCancelled = 1, kUnknown = 2, kInvalidArgument = 3, kDeadlineExceeded = 4, kNotFound = 5,
  kFailedPrecondition = 9, kOutOfRange = 11, kUnimplemented = 12, kInternal = 13,
};
using string_view = std::string_view;
class Status {
 public:
  Status() = default;
  Status(StatusCode c, std::string m) : code_(c), msg_(std::move(m)) {}
  bool ok() const { return code_ == StatusCode::kOk; }
  StatusCode code() const { return code_; }
  const std::string& message() const { return msg_; }
 private:
  StatusCode code_ = StatusCode::kOk;
  std::string msg_;
};
inline Status OkStatus() { return Status(); }
inline Status InvalidArgumentError(std::string m) { return Status(StatusCode::kInvalidArgument, std::move(m)); }
inline Status UnimplementedError(std::string m) { return Status(StatusCode::kUnimplemented, std::move(m)); }
inline Status InternalError(std::string m) { return Status(StatusCode::kInternal, std::move(m)); }
inline Status FailedPreconditionError(std::string m) { return Status(StatusCode::kFailedPrecondition, std::move(m)); }
template <typename T>
class StatusOr {
 public:
  StatusOr(T v) : v_(std::move(v)) {}                       // NOLINT
  StatusOr(Status s) : s_(std::move(s)) {}                  // NOLINT
  bool ok() const { return v_.has_value(); }
  const Status& status() const { return s_; }
  T& value() { return *v_; }
  const T& value() const { return *v_; }
  T& operator*() { return *v_; }
  const T& operator*() const { return *v_; }
  T* operator->() { return &*v_; }
  const T* operator->() const { return &*v_; }
 private:
  std::optional<T> v_;
  Status s_;
};
}  // namespace absl

namespace litert {
enum class ElementType { None, Int32, Float32 };
using Dimensions = std::vector<int32_t>;

class TensorBuffer {
 public:
  enum class LockMode { kRead, kWrite, kReadWrite };
  TensorBuffer() = default;
  static TensorBuffer CreateManagedHost(ElementType type, Dimensions dims) {
    TensorBuffer b;
    b.type_ = type;
    b.dims_ = std::move(dims);
    size_t n = 1;
    for (int32_t d : b.dims_) n *= (size_t)d;
    b.bytes_ = n * 4;
    b.data_ = std::shared_ptr<uint8_t>(new uint8_t[b.bytes_ ? b.bytes_ : 1](), std::default_delete<uint8_t[]>());
    return b;
  }
  ElementType GetElementType() const { return type_; }
  const Dimensions& GetDimensions() const { return dims_; }
  size_t Size() const { return bytes_; }
  size_t PackedSize() const { return bytes_; }
  bool IsHostMemory() const { return true; }
  TensorBuffer Duplicate() const { return *this; }           // shares the storage, like a LiteRT handle
  void* Lock() const { return data_.get(); }
  bool HasStorage() const { return data_ != nullptr; }
 private:
  ElementType type_ = ElementType::None;
  Dimensions dims_;
  size_t bytes_ = 0;
  std::shared_ptr<uint8_t> data_;
};
}  // namespace litert

namespace litert::lm {

// runtime/executor/llm_executor_io_types.h:32-51
class ExecutorTextData {
 public:
  ExecutorTextData() = default;
  explicit ExecutorTextData(::litert::TensorBuffer&& token_ids) : token_ids_(std::move(token_ids)) {}
  const ::litert::TensorBuffer& GetTokenIds() const { return token_ids_; }
  ::litert::TensorBuffer& GetMutableTokenIds() { return token_ids_; }
 private:
  ::litert::TensorBuffer token_ids_;
};

// runtime/executor/llm_executor_io_types.h:172-214 (text part only)
class ExecutorInputs {
 public:
  ExecutorInputs() = default;
  explicit ExecutorInputs(ExecutorTextData&& text) : text_(std::move(text)) {}
  void SetTextData(ExecutorTextData&& text) { text_ = std::move(text); }
  absl::StatusOr<const ExecutorTextData*> GetTextDataPtr() const {
    if (!text_.has_value()) return absl::FailedPreconditionError("ExecutorInputs::text_data_ is not set.");
    return &*text_;
  }
  absl::StatusOr<const ::litert::TensorBuffer*> GetTextTokenIdsPtr() const {
    if (!text_.has_value()) return absl::FailedPreconditionError("ExecutorInputs::text_data_ is not set.");
    return &text_->GetTokenIds();
  }
 private:
  std::optional<ExecutorTextData> text_;
};

// runtime/executor/llm_executor_io_types.h:217-250
class ExecutorPrefillParams {
 public:
  int GetCurrentStep() const { return current_step_; }
  void SetCurrentStep(int s) { current_step_ = s; }
  bool GetWaitForCompletion() const { return wait_; }
  void SetWaitForCompletion(bool w) { wait_ = w; }
  const std::atomic_bool* GetCancelFlag() const { return cancel_; }
  void SetCancelFlag(const std::atomic_bool* c) { cancel_ = c; }
 private:
  int current_step_ = -1;
  bool wait_ = false;
  const std::atomic_bool* cancel_ = nullptr;
};

// The virtuals of runtime/executor/llm_executor_base.h:33-121 that text-only
// callers use.
class LlmExecutorBase {
 public:
  virtual ~LlmExecutorBase() = default;
  virtual absl::Status Prefill(const ExecutorInputs& inputs) = 0;
  virtual absl::Status Prefill(const ExecutorInputs& inputs, const ExecutorPrefillParams& params) = 0;
  virtual absl::Status Decode(::litert::TensorBuffer& output_tokens) = 0;
  virtual absl::Status Decode(const ExecutorInputs& inputs, ::litert::TensorBuffer& output_logits) = 0;
  virtual absl::StatusOr<::litert::TensorBuffer> DecodeLogits(const ExecutorInputs& inputs) = 0;
  virtual absl::string_view ExecutorBackendName() const = 0;
  virtual absl::StatusOr<int> GetVocabSize() = 0;
  virtual absl::StatusOr<int> GetCurrentStep() const = 0;
  virtual absl::Status Reset() = 0;
};
using LlmExecutor = LlmExecutorBase;

}  // namespace litert::lm

// Stand-ins for the absl / LiteRT / LiteRT-LM types the executor interface is
// written against, so that the adapter in b200_llm_executor.h compiles and is
// tested where those projects' headers are absent.  Inside a LiteRT-LM checkout
// define B200LM_WITH_LITERT_LM and this file is not used: the adapter body is
// the same either way, so everything here has the NAME, SIGNATURE and result
// convention of the real thing.
//
// Only the subset that the executor's callers touch is modelled
// (runtime/util/convert_tensor_buffer.h:63-231, runtime/core/pipeline.cc:51-62,104-135,
// runtime/components/top_p_cpu_sampler.cc:61-110):
//   litert::Expected / Unexpected, litert::Layout, RankedTensorType,
//   litert::TensorBuffer {CreateManaged, TensorType, BufferType, Size, PackedSize,
//   Duplicate, Read, Write}, TensorBufferScopedLock::Create(buffer, mode),
//   litert::lm::{ElementTypeFor, CreateTensorBuffer, CopyFromTensorBuffer,
//   CopyToTensorBuffer, ReferTensorBufferAsSpan}, LlmExecutorSettings
//   {Get/SetMaxNumTokens} and the LlmExecutorBase virtuals.
// Behaviour pinned by runtime/util/convert_tensor_buffer_test.cc:44-266: spans are
// only handed out for host memory, an element-type mismatch is
// kLiteRtStatusErrorInvalidArgument, Duplicate() shares the storage.
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

// ---------------------------------------------------------------- absl subset
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
inline std::string StrCat(std::string_view a, std::string_view b) { return std::string(a) + std::string(b); }
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
template <typename T>
class Span {
 public:
  Span() = default;
  Span(T* p, size_t n) : p_(p), n_(n) {}
  template <typename U>
  Span(std::vector<U>& v) : p_(v.data()), n_(v.size()) {}   // NOLINT
  template <typename U>
  Span(const std::vector<U>& v) : p_(v.data()), n_(v.size()) {}   // NOLINT
  T* data() const { return p_; }
  size_t size() const { return n_; }
  bool empty() const { return n_ == 0; }
  T& operator[](size_t i) const { return p_[i]; }
  T* begin() const { return p_; }
  T* end() const { return p_ + n_; }
 private:
  T* p_ = nullptr;
  size_t n_ = 0;
};
template <typename T>
Span<T> MakeSpan(T* p, size_t n) { return Span<T>(p, n); }
template <typename T>
Span<T> MakeSpan(std::vector<T>& v) { return Span<T>(v.data(), v.size()); }
template <typename T>
Span<const T> MakeConstSpan(const T* p, size_t n) { return Span<const T>(p, n); }
template <typename T>
Span<const T> MakeConstSpan(const std::vector<T>& v) { return Span<const T>(v.data(), v.size()); }
}  // namespace absl

// ---------------------------------------------------------------- LiteRT subset
enum LiteRtStatus : int {
  kLiteRtStatusOk = 0,
  kLiteRtStatusErrorInvalidArgument = 1,
  kLiteRtStatusErrorRuntimeFailure = 500,
};
enum LiteRtTensorBufferType : int {
  kLiteRtTensorBufferTypeUnknown = 0,
  kLiteRtTensorBufferTypeHostMemory = 1,
  kLiteRtTensorBufferTypeOpenClBuffer = 10,       // stands for every buffer that is not host memory
};

namespace litert {

class Error {
 public:
  Error(LiteRtStatus s, std::string m) : status_(s), msg_(std::move(m)) {}
  LiteRtStatus Status() const { return status_; }
  const std::string& Message() const { return msg_; }
 private:
  LiteRtStatus status_;
  std::string msg_;
};
class Unexpected {
 public:
  Unexpected(LiteRtStatus s, std::string m = "") : err_(s, std::move(m)) {}      // NOLINT
  explicit Unexpected(class Error e) : err_(std::move(e)) {}
  const class Error& Error() const { return err_; }
 private:
  class Error err_;
};
template <typename T>
class Expected {
 public:
  Expected(T v) : v_(std::move(v)) {}                       // NOLINT
  Expected(const Unexpected& u) : e_(u.Error()) {}          // NOLINT
  Expected(class Error e) : e_(std::move(e)) {}             // NOLINT
  bool HasValue() const { return v_.has_value(); }
  explicit operator bool() const { return HasValue(); }
  T& Value() { return *v_; }
  const T& Value() const { return *v_; }
  T& operator*() { return *v_; }
  const T& operator*() const { return *v_; }
  T* operator->() { return &*v_; }
  const T* operator->() const { return &*v_; }
  const class Error& Error() const { return *e_; }
 private:
  std::optional<T> v_;
  std::optional<class Error> e_;
};
template <>
class Expected<void> {
 public:
  Expected() = default;
  Expected(const Unexpected& u) : e_(u.Error()) {}          // NOLINT
  bool HasValue() const { return !e_.has_value(); }
  explicit operator bool() const { return HasValue(); }
  const class Error& Error() const { return *e_; }
 private:
  std::optional<class Error> e_;
};

enum class ElementType { None, Int32, Float32 };
using Dimensions = std::vector<int32_t>;

class Layout {
 public:
  Layout() = default;
  explicit Layout(litert::Dimensions&& dims) : dims_(std::move(dims)) {}
  absl::Span<const int32_t> Dimensions() const { return absl::Span<const int32_t>(dims_.data(), dims_.size()); }
  size_t Rank() const { return dims_.size(); }
 private:
  litert::Dimensions dims_;
};
class RankedTensorType {
 public:
  RankedTensorType() = default;
  RankedTensorType(enum ElementType t, class Layout l) : type_(t), layout_(std::move(l)) {}
  enum ElementType ElementType() const { return type_; }
  const class Layout& Layout() const { return layout_; }
 private:
  enum ElementType type_ = ElementType::None;
  class Layout layout_;
};

class TensorBuffer {
 public:
  enum class LockMode { kRead, kWrite, kReadWrite };
  TensorBuffer() = default;
  static Expected<TensorBuffer> CreateManaged(LiteRtTensorBufferType buffer_type, const RankedTensorType& type, size_t bytes) {
    TensorBuffer b;
    b.buffer_type_ = buffer_type;
    b.type_ = type;
    b.bytes_ = bytes;
    b.data_ = std::shared_ptr<uint8_t>(new uint8_t[bytes ? bytes : 1](), std::default_delete<uint8_t[]>());
    b.locks_ = std::make_shared<std::atomic<int>>(0);
    return b;
  }
  Expected<RankedTensorType> TensorType() const {
    if (!data_) return Unexpected(kLiteRtStatusErrorRuntimeFailure, "empty tensor buffer");
    return type_;
  }
  Expected<LiteRtTensorBufferType> BufferType() const {
    if (!data_) return Unexpected(kLiteRtStatusErrorRuntimeFailure, "empty tensor buffer");
    return buffer_type_;
  }
  Expected<size_t> Size() const { return bytes_; }
  Expected<size_t> PackedSize() const { return bytes_; }
  Expected<TensorBuffer> Duplicate() const {      // another handle on the same storage
    if (!data_) return Unexpected(kLiteRtStatusErrorRuntimeFailure, "empty tensor buffer");
    return *this;
  }
  template <typename T>
  Expected<void> Write(absl::Span<const T> data) {
    if (data.size() * sizeof(T) > bytes_) return Unexpected(kLiteRtStatusErrorRuntimeFailure, "TensorBuffer size is smaller than the given data");
    std::memcpy(data_.get(), data.data(), data.size() * sizeof(T));
    return {};
  }
  template <typename T>
  Expected<void> Read(absl::Span<T> data) {
    if (data.size() * sizeof(T) > bytes_) return Unexpected(kLiteRtStatusErrorRuntimeFailure, "TensorBuffer size is smaller than the given data");
    std::memcpy(data.data(), data_.get(), data.size() * sizeof(T));
    return {};
  }
  // number of scoped locks alive on this storage (test aid: a span must not outlive its lock unnoticed)
  int LiveLocks() const { return locks_ ? locks_->load() : 0; }

 private:
  friend class TensorBufferScopedLock;
  LiteRtTensorBufferType buffer_type_ = kLiteRtTensorBufferTypeUnknown;
  RankedTensorType type_;
  size_t bytes_ = 0;
  std::shared_ptr<uint8_t> data_;
  std::shared_ptr<std::atomic<int>> locks_;
};

class TensorBufferScopedLock {
 public:
  TensorBufferScopedLock(TensorBufferScopedLock&& o) noexcept : locks_(std::move(o.locks_)) { o.locks_.reset(); }
  TensorBufferScopedLock& operator=(TensorBufferScopedLock&& o) noexcept {
    Release();
    locks_ = std::move(o.locks_);
    o.locks_.reset();
    return *this;
  }
  TensorBufferScopedLock(const TensorBufferScopedLock&) = delete;
  TensorBufferScopedLock& operator=(const TensorBufferScopedLock&) = delete;
  ~TensorBufferScopedLock() { Release(); }
  static Expected<std::pair<TensorBufferScopedLock, void*>> Create(TensorBuffer& buffer,
                                                                  TensorBuffer::LockMode mode = TensorBuffer::LockMode::kReadWrite) {
    (void)mode;
    if (!buffer.data_) return Unexpected(kLiteRtStatusErrorRuntimeFailure, "empty tensor buffer");
    if (buffer.buffer_type_ != kLiteRtTensorBufferTypeHostMemory)
      return Unexpected(kLiteRtStatusErrorRuntimeFailure, "this stand-in only maps host memory");
    return std::make_pair(TensorBufferScopedLock(buffer.locks_), static_cast<void*>(buffer.data_.get()));
  }
 private:
  explicit TensorBufferScopedLock(std::shared_ptr<std::atomic<int>> l) : locks_(std::move(l)) {
    if (locks_) locks_->fetch_add(1);
  }
  void Release() {
    if (locks_) locks_->fetch_sub(1);
    locks_.reset();
  }
  std::shared_ptr<std::atomic<int>> locks_;
};

}  // namespace litert

// ---------------------------------------------------------------- LiteRT-LM subset
namespace litert::lm {

// runtime/util/convert_tensor_buffer.h:40-58
template <typename T>
struct ElementTypeFor;
template <>
struct ElementTypeFor<int32_t> { static constexpr ::litert::ElementType kType = ::litert::ElementType::Int32; };
template <>
struct ElementTypeFor<float> { static constexpr ::litert::ElementType kType = ::litert::ElementType::Float32; };

// runtime/util/convert_tensor_buffer.h:60-75
template <typename T>
::litert::Expected<::litert::TensorBuffer> CreateTensorBuffer(::litert::Dimensions&& dimensions,
                                                              LiteRtTensorBufferType buffer_type = kLiteRtTensorBufferTypeHostMemory) {
  int size = 1;
  for (int dim : dimensions) size *= dim;
  return ::litert::TensorBuffer::CreateManaged(
      buffer_type, ::litert::RankedTensorType(ElementTypeFor<T>::kType, ::litert::Layout(std::move(dimensions))), size * sizeof(T));
}

// runtime/util/convert_tensor_buffer.h:148-163
template <typename T>
::litert::Expected<::litert::TensorBuffer> CopyToTensorBuffer(absl::Span<const T> data, ::litert::Dimensions&& dimensions,
                                                              LiteRtTensorBufferType buffer_type = kLiteRtTensorBufferTypeHostMemory) {
  auto out = ::litert::TensorBuffer::CreateManaged(
      buffer_type, ::litert::RankedTensorType(ElementTypeFor<T>::kType, ::litert::Layout(std::move(dimensions))), data.size() * sizeof(T));
  if (!out.HasValue()) return out.Error();
  out->Write(data);
  return std::move(*out);
}

// runtime/util/convert_tensor_buffer.h:77-104
template <typename T>
::litert::Expected<std::vector<T>> CopyFromTensorBuffer(::litert::TensorBuffer& tensor_buffer) {
  if (auto type = tensor_buffer.TensorType(); !type.HasValue() || type->ElementType() != ElementTypeFor<T>::kType)
    return ::litert::Unexpected(kLiteRtStatusErrorInvalidArgument, "Element type is not compatible to the target type.");
  auto size = tensor_buffer.Size();
  std::vector<T> copied(*size / sizeof(T));
  tensor_buffer.Read(absl::MakeSpan(copied));
  return copied;
}

// runtime/util/convert_tensor_buffer.h:192-229: no copy, host memory only.
template <typename T>
::litert::Expected<absl::Span<T>> ReferTensorBufferAsSpan(::litert::TensorBuffer& tensor_buffer) {
  if (auto buffer_type = tensor_buffer.BufferType(); !buffer_type.HasValue() || *buffer_type != kLiteRtTensorBufferTypeHostMemory)
    return ::litert::Unexpected(kLiteRtStatusErrorInvalidArgument, "Tensor buffer is not in the host memory.");
  if (auto type = tensor_buffer.TensorType(); !type.HasValue() || type->ElementType() != ElementTypeFor<T>::kType)
    return ::litert::Unexpected(kLiteRtStatusErrorInvalidArgument, "Element type is not compatible to the target type.");
  auto size = tensor_buffer.Size();
  auto lock_and_addr = ::litert::TensorBufferScopedLock::Create(tensor_buffer, ::litert::TensorBuffer::LockMode::kRead);
  if (!lock_and_addr.HasValue()) return lock_and_addr.Error();
  return absl::MakeSpan(static_cast<T*>(lock_and_addr->second), *size / sizeof(T));
}
template <typename T>
::litert::Expected<absl::Span<T>> ReferTensorBufferAsSpan(const ::litert::TensorBuffer& tensor_buffer) {
  auto mutable_tensor_buffer = tensor_buffer.Duplicate();
  if (!mutable_tensor_buffer) return mutable_tensor_buffer.Error();
  return ReferTensorBufferAsSpan<T>(*mutable_tensor_buffer);
}

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

// runtime/executor/llm_executor_settings.h:95-154: the part the caller loop reads.
class LlmExecutorSettings {
 public:
  uint32_t GetMaxNumTokens() const { return max_num_tokens_; }
  void SetMaxNumTokens(uint64_t max_num_tokens) { max_num_tokens_ = (uint32_t)max_num_tokens; }
 private:
  uint32_t max_num_tokens_ = 0;
};

// The virtuals of runtime/executor/llm_executor_base.h:33-121 that text-only
// callers use; the ones with a base-class default keep it.
class LlmExecutorBase {
 public:
  virtual ~LlmExecutorBase() = default;
  virtual absl::string_view ExecutorBackendName() const = 0;
  virtual absl::Status Prefill(const ExecutorInputs& inputs) = 0;
  virtual absl::Status Prefill(const ExecutorInputs& inputs, const ExecutorPrefillParams& params) {
    return absl::UnimplementedError(absl::StrCat("Prefill with prefill query params not implemented for backend: ", ExecutorBackendName()));
  }
  virtual absl::Status Decode(::litert::TensorBuffer& output_tokens) = 0;
  virtual absl::Status Decode(const ExecutorInputs& inputs, ::litert::TensorBuffer& output_logits) = 0;
  virtual absl::StatusOr<::litert::TensorBuffer> DecodeLogits(const ExecutorInputs& inputs) {
    return absl::UnimplementedError(absl::StrCat("DecodeLogits not implemented for backend: ", ExecutorBackendName()));
  }
  virtual absl::StatusOr<int> GetVocabSize() = 0;
  virtual absl::StatusOr<int> GetCurrentStep() const {
    return absl::UnimplementedError(absl::StrCat("GetCurrentStep not implemented for backend: ", ExecutorBackendName()));
  }
  virtual absl::StatusOr<LlmExecutorSettings> GetExecutorSettings() const {
    return absl::UnimplementedError(absl::StrCat("GetExecutorSettings not implemented for backend: ", ExecutorBackendName()));
  }
  virtual absl::Status Reset() {
    return absl::UnimplementedError(absl::StrCat("Reset not implemented for backend: ", ExecutorBackendName()));
  }
};
using LlmExecutor = LlmExecutorBase;

}  // namespace litert::lm

// C++ surface of the sm100 loader for callers written against the reference's public API: the classes and
// structs a program gets from the reference's include/aginfer/runtime.h (Status, StatusOr, TensorView,
// RuntimeOptions, Runtime, Model, Session ... with the same member names, field order and enumerator values),
// implemented header-only over the C ABI of aginfer_b200.h.  A program that includes this file under the
// name "aginfer/runtime.h" and links libaginfer_b200.so instead of the reference's static library compiles
// unchanged; the reference's own tests/runtime_test.cc and tests/cuda_runtime_test.cc are built that way by
// oracle/Makefile (target sm100) and run by tests/test_reference_boundary.py.
//
// What differs from the reference behind the same calls is the loader's (graph replay, pinned upload, the
// run options that select work); see aginfer_b200.h.  Objects are move-only and a Session borrows its
// Runtime and Model, which must outlive it, exactly as in the reference (cpp/runtime.cc:217).
#pragma once

#include "aginfer_b200.h"

#include <cstddef>
#include <cstdint>
#include <memory>
#include <optional>
#include <string>
#include <utility>
#include <vector>

namespace aginfer {

inline constexpr std::uint32_t kRuntimeAbi = AGI_RUNTIME_ABI;

// Enumerator order and values are those of agi_status (and of the reference's StatusCode).
enum class StatusCode {
  kOk = AGI_OK,
  kInvalidArgument = AGI_INVALID_ARGUMENT,
  kNotFound = AGI_NOT_FOUND,
  kIoError = AGI_IO_ERROR,
  kCorruptPackage = AGI_CORRUPT_PACKAGE,
  kIncompatiblePlatform = AGI_INCOMPATIBLE_PLATFORM,
  kIncompatibleArchitecture = AGI_INCOMPATIBLE_ARCHITECTURE,
  kIncompatibleAbi = AGI_INCOMPATIBLE_ABI,
  kCudaError = AGI_CUDA_ERROR,
  kOutOfMemory = AGI_OUT_OF_MEMORY,
};

inline const char* StatusCodeName(StatusCode code) noexcept { return agi_status_name(static_cast<int>(code)); }

class Status {
 public:
  Status() = default;
  Status(StatusCode code, std::string message) : code_(code), message_(std::move(message)) {}
  static Status Ok() { return Status(); }
  bool ok() const noexcept { return code_ == StatusCode::kOk; }
  StatusCode code() const noexcept { return code_; }
  const std::string& message() const noexcept { return message_; }

 private:
  StatusCode code_ = StatusCode::kOk;
  std::string message_;
};

template <typename T>
class StatusOr {
 public:
  StatusOr(Status status) : status_(std::move(status)) {}
  StatusOr(T value) : held_(std::move(value)) {}
  bool ok() const noexcept { return status_.ok(); }
  const Status& status() const noexcept { return status_; }
  T& value() & { return *held_; }
  const T& value() const& { return *held_; }
  T&& value() && { return std::move(*held_); }

 private:
  Status status_;
  std::optional<T> held_;
};

enum class DType { kFp32 = AGI_F32, kFp16 = AGI_F16, kBf16 = AGI_BF16, kFp8E4M3 = AGI_F8_E4M3, kInt32 = AGI_I32 };
enum class MemoryLocation { kHost = AGI_HOST, kDevice = AGI_DEVICE };
enum class MathMode { kStrict, kTf32 };

struct TensorView {
  std::string name;
  DType dtype = DType::kFp32;
  std::vector<std::int64_t> shape;
  std::vector<std::int64_t> stride;   // in elements
  void* data = nullptr;
  std::size_t byte_size = 0;
  MemoryLocation location = MemoryLocation::kDevice;
  bool caller_owned = true;
};

struct TensorInfo {
  std::string name;
  DType dtype = DType::kFp32;
  std::vector<std::int64_t> shape;
  std::vector<std::int64_t> stride;
  std::size_t byte_size = 0;
  MemoryLocation location = MemoryLocation::kDevice;
};

struct RunOptions {
  std::uint32_t denoising_steps = 0;   // zero: the session's profile as packaged; n: its sibling for n steps
  std::uint64_t seed = 0;
  bool deterministic = true;
  MathMode math_mode = MathMode::kStrict;
  const TensorView* initial_noise_override = nullptr;
};

struct RuntimeOptions {
  std::uint32_t required_runtime_abi = kRuntimeAbi;
  std::uint32_t cuda_arch_override = 0;              // non-zero fields replace the probe of the machine
  std::uint32_t cuda_driver_version_override = 0;
  std::uint32_t cuda_runtime_version_override = 0;
  std::uint32_t cublaslt_abi_override = 0;
  std::uint32_t cudnn_abi_override = 0;
};

struct SessionOptions {
  std::string profile;
};

struct TargetInfo {
  std::string platform;
  std::string cuda_arch;
  std::uint32_t runtime_abi = 0;
};

struct WorkspaceInfo {
  std::uint64_t arena_bytes = 0;
  std::uint64_t workspace_bytes = 0;
};

using CudaStream = void*;

namespace detail {
inline Status Failure(agi_status code) { return Status(static_cast<StatusCode>(code), agi_last_error()); }
struct Release {
  void operator()(agi_runtime* p) const { agi_runtime_destroy(p); }
  void operator()(agi_model* p) const { agi_model_destroy(p); }
  void operator()(agi_session* p) const { agi_session_destroy(p); }
};
inline agi_tensor_view Raw(const TensorView& v) {
  agi_tensor_view raw{};
  raw.name = v.name.c_str();
  raw.dtype = static_cast<std::uint32_t>(v.dtype);
  raw.location = static_cast<std::uint32_t>(v.location);
  // a view whose stride list does not match its shape list can never match a profile: the rank is then one
  // that no plan tensor has, and the loader answers with the reference's message for a rank mismatch
  raw.rank = v.shape.size() == v.stride.size() ? static_cast<std::uint32_t>(v.shape.size()) : 0xffffffffu;
  raw.shape = v.shape.data();
  raw.stride = v.stride.data();
  raw.data = v.data;
  raw.byte_size = v.byte_size;
  return raw;
}
}  // namespace detail

class Session;

class Runtime {
 public:
  Runtime(Runtime&&) noexcept = default;
  Runtime& operator=(Runtime&&) noexcept = default;
  static StatusOr<Runtime> Create(const RuntimeOptions& options = {}) {
    const agi_runtime_options raw{options.required_runtime_abi, options.cuda_arch_override,
                                  options.cuda_driver_version_override, options.cuda_runtime_version_override,
                                  options.cublaslt_abi_override, options.cudnn_abi_override};
    agi_runtime* handle = nullptr;
    if (const agi_status code = agi_runtime_create(&raw, &handle)) return detail::Failure(code);
    return Runtime(handle);
  }

 private:
  explicit Runtime(agi_runtime* handle) : handle_(handle) {}
  std::unique_ptr<agi_runtime, detail::Release> handle_;
  friend class Session;
};

class Model {
 public:
  Model(Model&&) noexcept = default;
  Model& operator=(Model&&) noexcept = default;
  static StatusOr<Model> Load(const std::string& aim_path) {
    agi_model* handle = nullptr;
    if (const agi_status code = agi_model_load(aim_path.c_str(), &handle)) return detail::Failure(code);
    return Model(handle);
  }

 private:
  explicit Model(agi_model* handle) : handle_(handle) {}
  std::unique_ptr<agi_model, detail::Release> handle_;
  friend class Session;
};

class Session {
 public:
  Session(Session&&) noexcept = default;
  Session& operator=(Session&&) noexcept = default;

  // `flags`: AGI_SESSION_* switches of this loader (no counterpart in the reference); zero = defaults.
  static StatusOr<Session> Create(Runtime& runtime, Model& model, const SessionOptions& options = {},
                                  std::uint32_t flags = 0) {
    agi_session* handle = nullptr;
    if (const agi_status code =
            agi_session_create(runtime.handle_.get(), model.handle_.get(), options.profile.c_str(), flags, &handle))
      return detail::Failure(code);
    return Session(handle);
  }

  TargetInfo GetTargetInfo() const {
    const char* platform = "";
    const char* arch = "";
    TargetInfo info;
    if (agi_session_get_target_info(handle_.get(), &platform, &arch, &info.runtime_abi) == AGI_OK) {
      info.platform = platform;
      info.cuda_arch = arch;
    }
    return info;
  }
  std::vector<TensorInfo> GetInputInfo() const { return Infos(agi_session_get_input_count, agi_session_get_input_info); }
  std::vector<TensorInfo> GetOutputInfo() const { return Infos(agi_session_get_output_count, agi_session_get_output_info); }

  StatusOr<WorkspaceInfo> GetRequiredWorkspace(const std::string& profile) const {
    WorkspaceInfo info;
    if (const agi_status code =
            agi_session_get_required_workspace(handle_.get(), profile.c_str(), &info.arena_bytes, &info.workspace_bytes))
      return detail::Failure(code);
    return info;
  }

  Status Enqueue(const std::vector<TensorView>& inputs, const std::vector<TensorView>& outputs, const RunOptions& options,
                 CudaStream stream) {
    std::vector<agi_tensor_view> raw_in, raw_out;
    for (const TensorView& v : inputs) raw_in.push_back(detail::Raw(v));
    for (const TensorView& v : outputs) raw_out.push_back(detail::Raw(v));
    agi_run_options raw{};
    raw.denoising_steps = options.denoising_steps;
    raw.deterministic = options.deterministic ? 1u : 0u;
    raw.seed = options.seed;
    raw.math_mode = static_cast<std::uint32_t>(options.math_mode);
    agi_tensor_view noise{};
    if (options.initial_noise_override != nullptr) {
      noise = detail::Raw(*options.initial_noise_override);
      raw.initial_noise_override = &noise;
    }
    if (const agi_status code = agi_session_enqueue(handle_.get(), raw_in.data(), raw_in.size(), raw_out.data(),
                                                    raw_out.size(), &raw, stream))
      return detail::Failure(code);
    return Status::Ok();
  }

 private:
  explicit Session(agi_session* handle) : handle_(handle) {}
  template <typename Count, typename Info>
  std::vector<TensorInfo> Infos(Count count_of, Info info_of) const {
    std::vector<TensorInfo> found;
    std::uint32_t count = 0;
    if (count_of(handle_.get(), &count) != AGI_OK) return found;
    for (std::uint32_t i = 0; i < count; ++i) {
      agi_tensor_info raw{};
      if (info_of(handle_.get(), i, &raw) != AGI_OK) break;
      TensorInfo t;
      t.name = raw.name;
      t.dtype = static_cast<DType>(raw.dtype);
      t.shape.assign(raw.shape, raw.shape + raw.rank);
      t.stride.assign(raw.stride, raw.stride + raw.rank);
      t.byte_size = static_cast<std::size_t>(raw.byte_size);
      t.location = static_cast<MemoryLocation>(raw.location);
      found.push_back(std::move(t));
    }
    return found;
  }
  std::unique_ptr<agi_session, detail::Release> handle_;
};

}  // namespace aginfer

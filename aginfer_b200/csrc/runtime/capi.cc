#include "aginfer_b200.h"

#include "digest.h"
#include "error_slot.h"
#include "session.h"

#include <cstring>
#include <memory>
#include <string>

struct agi_runtime {
  agi::RuntimeOptions options;
};
struct agi_model {
  std::unique_ptr<agi::Package> package;
};
struct agi_session {
  std::unique_ptr<agi::Session> impl;
  std::string arch_name;
  std::uint32_t runtime_abi = 0;
};

namespace {

thread_local std::string g_last_error;

agi_status Fail(agi::Code code, std::string message) {
  g_last_error = std::move(message);
  return static_cast<agi_status>(code);
}
agi_status Done(const agi::Status& status) {
  if (status.ok()) return AGI_OK;
  return Fail(status.code, status.message);
}
agi_status Null(const char* what) { return Fail(agi::kInvalidArgument, std::string(what) + " must not be NULL"); }

// index-th tensor of `kind` in the session's profile, or nullptr
const agi::wire::Tensor* NthTensor(const agi::Session& s, std::uint32_t kind, std::uint32_t index) {
  const auto& profile = s.profile();
  for (std::uint32_t i = 0; i < profile.tensor_count; ++i) {
    const auto& t = s.plan().tensors[profile.first_tensor + i];
    if (t.io_kind == kind && index-- == 0) return &t;
  }
  return nullptr;
}

std::uint32_t CountTensors(const agi::Session& s, std::uint32_t kind) {
  std::uint32_t n = 0;
  for (std::uint32_t i = 0; i < s.profile().tensor_count; ++i)
    n += s.plan().tensors[s.profile().first_tensor + i].io_kind == kind;
  return n;
}

agi_status FillInfo(const agi_session* session, std::uint32_t kind, std::uint32_t index, agi_tensor_info* out) {
  if (session == nullptr) return Null("session");
  if (out == nullptr) return Null("out");
  const agi::wire::Tensor* t = NthTensor(*session->impl, kind, index);
  if (t == nullptr) return Fail(agi::kInvalidArgument, "tensor index is out of range for the selected profile");
  std::memset(out, 0, sizeof *out);
  out->name = session->impl->plan().Text(t->name).data();  // NUL-terminated inside the mapped plan
  switch (t->dtype) {
    case agi::wire::kF16: out->dtype = AGI_F16; break;
    case agi::wire::kBF16: out->dtype = AGI_BF16; break;
    case agi::wire::kF8E4M3: out->dtype = AGI_F8_E4M3; break;
    case agi::wire::kI32: out->dtype = AGI_I32; break;
    default: out->dtype = AGI_F32; break;
  }
  out->location = t->location == agi::wire::kDevice ? AGI_DEVICE : AGI_HOST;
  out->rank = t->rank;
  for (std::uint32_t d = 0; d < t->rank; ++d) {
    out->shape[d] = t->shape[d];
    out->stride[d] = t->stride[d];
  }
  out->byte_size = t->byte_size;
  return AGI_OK;
}

}  // namespace

namespace agi {
agi_status RecordFailure(int code, const std::string& message) { return Fail(static_cast<Code>(code), message); }
}  // namespace agi

extern "C" {

const char* agi_status_name(int status) { return agi::CodeName(status); }
const char* agi_last_error(void) { return g_last_error.c_str(); }
const char* agi_version(void) {
  static const std::string text = std::string("aginfer-b200 0.1.0 abi 1 sha256=") + agi::Sha256::Backend();
  return text.c_str();
}

agi_status agi_runtime_create(const agi_runtime_options* options, agi_runtime** out) {
  if (out == nullptr) return Null("out");
  *out = nullptr;
  agi::RuntimeOptions o;
  if (options != nullptr) {
    o.required_runtime_abi = options->required_runtime_abi;
    o.cuda_arch = options->cuda_arch_override;
    o.cuda_driver_version = options->cuda_driver_version_override;
    o.cuda_runtime_version = options->cuda_runtime_version_override;
    o.cublaslt_abi = options->cublaslt_abi_override;
    o.cudnn_abi = options->cudnn_abi_override;
  }
  if (o.required_runtime_abi != agi::kRuntimeAbi)
    return Fail(agi::kIncompatibleAbi, "requested Runtime ABI does not match this library");
  const agi::Status probed = agi::ProbeSystem(&o);
  if (!probed.ok()) return Done(probed);
  *out = new agi_runtime{o};
  return AGI_OK;
}
void agi_runtime_destroy(agi_runtime* runtime) { delete runtime; }

agi_status agi_runtime_get_options(const agi_runtime* runtime, agi_runtime_options* out) {
  if (runtime == nullptr) return Null("runtime");
  if (out == nullptr) return Null("out");
  const agi::RuntimeOptions& o = runtime->options;
  *out = agi_runtime_options{o.required_runtime_abi, o.cuda_arch, o.cuda_driver_version, o.cuda_runtime_version,
                             o.cublaslt_abi, o.cudnn_abi};
  return AGI_OK;
}

agi_status agi_model_load(const char* aim_path, agi_model** out) {
  if (out == nullptr) return Null("out");
  *out = nullptr;
  if (aim_path == nullptr) return Null("aim_path");
  auto model = std::make_unique<agi_model>();
  const agi::Status opened = agi::Package::Open(aim_path, &model->package);
  if (!opened.ok()) return Done(opened);
  *out = model.release();
  return AGI_OK;
}
void agi_model_destroy(agi_model* model) { delete model; }

agi_status agi_model_variant_count(const agi_model* model, uint32_t* out) {
  if (model == nullptr) return Null("model");
  if (out == nullptr) return Null("out");
  *out = model->package->header().variant_count;
  return AGI_OK;
}
agi_status agi_model_variant_arch(const agi_model* model, uint32_t index, uint32_t* out) {
  if (model == nullptr) return Null("model");
  if (out == nullptr) return Null("out");
  if (index >= model->package->header().variant_count) return Fail(agi::kInvalidArgument, "variant index is out of range");
  *out = model->package->variants()[index].arch;
  return AGI_OK;
}

agi_status agi_session_create(agi_runtime* runtime, agi_model* model, const char* profile, uint32_t flags,
                              agi_session** out) {
  if (out == nullptr) return Null("out");
  *out = nullptr;
  if (runtime == nullptr) return Null("runtime");
  if (model == nullptr) return Null("model");
  auto session = std::make_unique<agi_session>();
  const agi::Status made =
      agi::Session::Create(runtime->options, *model->package, profile != nullptr ? profile : "", flags, &session->impl);
  if (!made.ok()) return Done(made);
  session->arch_name = "sm" + std::to_string(session->impl->arch());
  session->runtime_abi = model->package->header().runtime_abi;
  *out = session.release();
  return AGI_OK;
}
void agi_session_destroy(agi_session* session) { delete session; }

agi_status agi_session_get_target_info(const agi_session* session, const char** platform, const char** cuda_arch,
                                       uint32_t* runtime_abi) {
  if (session == nullptr) return Null("session");
  if (platform != nullptr) *platform = agi::HostPlatformName();
  if (cuda_arch != nullptr) *cuda_arch = session->arch_name.c_str();
  if (runtime_abi != nullptr) *runtime_abi = session->runtime_abi;
  return AGI_OK;
}

agi_status agi_session_get_input_count(const agi_session* session, uint32_t* out) {
  if (session == nullptr) return Null("session");
  if (out == nullptr) return Null("out");
  *out = CountTensors(*session->impl, agi::wire::kInput);
  return AGI_OK;
}
agi_status agi_session_get_output_count(const agi_session* session, uint32_t* out) {
  if (session == nullptr) return Null("session");
  if (out == nullptr) return Null("out");
  *out = CountTensors(*session->impl, agi::wire::kOutput);
  return AGI_OK;
}
agi_status agi_session_get_input_info(const agi_session* session, uint32_t index, agi_tensor_info* out) {
  return FillInfo(session, agi::wire::kInput, index, out);
}
agi_status agi_session_get_output_info(const agi_session* session, uint32_t index, agi_tensor_info* out) {
  return FillInfo(session, agi::wire::kOutput, index, out);
}

agi_status agi_session_get_required_workspace(const agi_session* session, const char* profile,
                                              uint64_t* arena_bytes, uint64_t* workspace_bytes) {
  if (session == nullptr) return Null("session");
  if (profile != nullptr && profile[0] != '\0' && !session->impl->HasProfile(profile))
    return Fail(agi::kInvalidArgument, std::string("profile is not present in the static execution plan: ") + profile);
  if (arena_bytes != nullptr) *arena_bytes = session->impl->plan().header->arena_bytes;
  if (workspace_bytes != nullptr) *workspace_bytes = session->impl->plan().header->workspace_bytes;
  return AGI_OK;
}

agi_status agi_session_enqueue(agi_session* session, const agi_tensor_view* inputs, size_t input_count,
                               const agi_tensor_view* outputs, size_t output_count, const agi_run_options* options,
                               void* stream) {
  if (session == nullptr) return Null("session");
  if ((inputs == nullptr && input_count != 0) || (outputs == nullptr && output_count != 0)) return Null("views");
  std::vector<agi::TensorArg> args(input_count + output_count);
  for (size_t i = 0; i < args.size(); ++i) {
    const agi_tensor_view& v = i < input_count ? inputs[i] : outputs[i - input_count];
    args[i] = agi::TensorArg{v.name, v.dtype, v.location, v.rank, v.shape, v.stride, v.data, v.byte_size};
  }
  agi::RunSelect select;
  agi::TensorArg noise;
  if (options != nullptr) {
    select.denoising_steps = options->denoising_steps;
    if (const agi_tensor_view* v = options->initial_noise_override) {
      noise = agi::TensorArg{v->name, v->dtype, v->location, v->rank, v->shape, v->stride, v->data, v->byte_size};
      select.noise_override = &noise;
    }
  }
  return Done(session->impl->Enqueue(args.data(), input_count, args.data() + input_count, output_count,
                                     static_cast<CUstream>(stream), select));
}

agi_status agi_session_get_stats(const agi_session* session, agi_session_stats* out) {
  if (session == nullptr) return Null("session");
  if (out == nullptr) return Null("out");
  const agi::SessionStats& s = session->impl->stats();
  *out = agi_session_stats{s.enqueues, s.kernel_launches, s.graph_launches, s.graphs_built,
                           session->impl->active_profile().launch_count, s.upload_seconds};
  return AGI_OK;
}

agi_status agi_sha256(const void* data, size_t size, int portable, uint8_t out[32]) {
  if ((data == nullptr && size != 0) || out == nullptr) return Null("buffer");
  const agi::Digest d = portable ? agi::Sha256::PortableOf(data, size) : agi::Sha256::Of(data, size);
  std::memcpy(out, d.data(), 32);
  return AGI_OK;
}

}  // extern "C"

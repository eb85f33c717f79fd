#include "session.h"

#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cstring>

namespace agi {
namespace {

constexpr std::size_t kStageBytes = 32u << 20;
constexpr std::size_t kMaxCachedGraphs = 8;
constexpr std::uint32_t kStaticSharedLimit = 48u * 1024;

void* OpenAny(std::initializer_list<const char*> names) {
  for (const char* name : names)
    if (void* lib = dlopen(name, RTLD_NOW | RTLD_LOCAL)) return lib;
  return nullptr;
}

std::uint32_t ToPublicDType(std::uint32_t wire_dtype) {
  switch (wire_dtype) {
    case wire::kF16: return kPubF16;
    case wire::kBF16: return kPubBF16;
    case wire::kF8E4M3: return kPubF8E4M3;
    case wire::kI32: return kPubI32;
    default: return kPubF32;
  }
}

}  // namespace

Status ProbeSystem(RuntimeOptions* o) {
  if (o->cuda_arch == 0 || o->cuda_driver_version == 0) {
    std::string why;
    const CudaApi* cu = CudaApi::Get(&why);
    if (cu == nullptr) return Status(kCudaError, why);
    CUdevice device = 0;
    int major = 0, minor = 0, version = 0;
    const bool ok = cu->cuInit(0) == CUDA_SUCCESS && cu->cuDeviceGet(&device, 0) == CUDA_SUCCESS &&
                    cu->cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, device) == CUDA_SUCCESS &&
                    cu->cuDeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, device) == CUDA_SUCCESS &&
                    cu->cuDriverGetVersion(&version) == CUDA_SUCCESS;
    if (!ok) return Status(kCudaError, "cannot query CUDA device 0 and Driver version");
    if (o->cuda_arch == 0) o->cuda_arch = static_cast<std::uint32_t>(major * 10 + minor);
    if (o->cuda_driver_version == 0) o->cuda_driver_version = static_cast<std::uint32_t>(version);
  }
  if (o->cuda_runtime_version == 0) {
    void* rt = OpenAny({"libcudart.so.12", "libcudart.so"});
    if (rt == nullptr) return Status(kCudaError, "cannot load CUDA Runtime");
    auto get = reinterpret_cast<int (*)(int*)>(dlsym(rt, "cudaRuntimeGetVersion"));
    int version = 0;
    const bool ok = get != nullptr && get(&version) == 0;
    dlclose(rt);
    if (!ok) return Status(kCudaError, "cannot query CUDA Runtime version");
    o->cuda_runtime_version = static_cast<std::uint32_t>(version);
  }
  if (o->cublaslt_abi == 0) {
    for (std::uint32_t abi : {12u, 11u}) {
      const std::string name = "libcublasLt.so." + std::to_string(abi);
      if (void* lib = OpenAny({name.c_str()})) {
        dlclose(lib);
        o->cublaslt_abi = abi;
        break;
      }
    }
    if (o->cublaslt_abi == 0) return Status(kCudaError, "cannot load a supported cuBLASLt ABI");
  }
  if (o->cudnn_abi == 0) {
    for (std::uint32_t abi : {9u, 8u}) {
      const std::string name = "libcudnn.so." + std::to_string(abi);
      if (void* lib = OpenAny({name.c_str()})) {
        dlclose(lib);
        o->cudnn_abi = abi;
        break;
      }
    }
    if (o->cudnn_abi == 0) return Status(kCudaError, "cannot load a supported cuDNN ABI");
  }
  return {};
}

Status Session::Create(const RuntimeOptions& rt, const Package& package, const std::string& profile,
                       std::uint32_t flags, std::unique_ptr<Session>* out) {
  const wire::VariantEntry* variant = package.FindVariant(rt.cuda_arch);
  if (variant == nullptr)
    return Status(kIncompatibleArchitecture, "AIM has no exact sm" + std::to_string(rt.cuda_arch) +
                                                 " variant; fallback and PTX JIT are forbidden");
  std::uint64_t driver_min = 0, runtime_min = 0, runtime_max = 0, cublaslt = 0, cudnn = 0;
  AGI_RETURN_IF_ERROR(ManifestUnsigned(package.manifest(), "cuda_driver_min", &driver_min));
  AGI_RETURN_IF_ERROR(ManifestUnsigned(package.manifest(), "cuda_runtime_min", &runtime_min));
  AGI_RETURN_IF_ERROR(ManifestUnsigned(package.manifest(), "cuda_runtime_max", &runtime_max));
  AGI_RETURN_IF_ERROR(ManifestUnsigned(package.manifest(), "cublaslt_abi", &cublaslt));
  AGI_RETURN_IF_ERROR(ManifestUnsigned(package.manifest(), "cudnn_abi", &cudnn));
  if (rt.cuda_driver_version < driver_min || rt.cuda_runtime_version < runtime_min ||
      rt.cuda_runtime_version > runtime_max || rt.cublaslt_abi != cublaslt || rt.cudnn_abi != cudnn)
    return Status(kIncompatibleAbi, "CUDA/cuBLASLt/cuDNN compatibility check failed");

  std::unique_ptr<Session> s(new Session);
  s->package_ = &package;
  s->variant_ = variant;
  s->flags_ = flags;
  AGI_RETURN_IF_ERROR(OpenPlan(package.data() + variant->plan_offset, static_cast<std::size_t>(variant->plan_size),
                               variant->arch, variant->weight_size, &s->plan_));
  s->profile_ = profile.empty() ? &s->plan_.profiles[0] : s->plan_.Find(profile);
  if (s->profile_ == nullptr)
    return Status(kInvalidArgument, "profile is not present in the static execution plan: " + profile);
  s->bound_.assign(s->profile_->tensor_count, nullptr);
  s->states_.push_back(std::make_unique<ProfileState>());
  s->states_[0]->profile = s->profile_;
  s->active_ = s->states_[0].get();
  *out = std::move(s);
  return {};
}

Session::~Session() {
  if (cu_ == nullptr || context_ == nullptr) return;
  cu_->cuCtxSetCurrent(context_);
  for (auto& state : states_)
    for (CachedGraph& g : state->graphs)
      if (g.exec != nullptr) cu_->cuGraphExecDestroy(g.exec);
  if (workspace_ != 0) cu_->cuMemFree(workspace_);
  if (arena_ != 0) cu_->cuMemFree(arena_);
  if (weights_ != 0) cu_->cuMemFree(weights_);
  if (module_ != nullptr) cu_->cuModuleUnload(module_);
  if (retained_primary_) cu_->cuDevicePrimaryCtxRelease(device_);
}

Status Session::Bind(const TensorArg* views, std::size_t count, std::uint32_t io_kind) {
  for (std::size_t v = 0; v < count; ++v) {
    const TensorArg& view = views[v];
    const std::string name = view.name != nullptr ? view.name : "";
    const wire::Tensor* want = nullptr;
    std::uint32_t slot = 0;
    for (std::uint32_t i = 0; i < profile_->tensor_count && want == nullptr; ++i) {
      const wire::Tensor& t = plan_.tensors[profile_->first_tensor + i];
      if (t.io_kind == io_kind && plan_.Text(t.name) == name) {
        want = &t;
        slot = i;
      }
    }
    if (want == nullptr) return Status(kInvalidArgument, "unexpected tensor for selected profile: " + name);
    if (bound_[slot] != nullptr) return Status(kInvalidArgument, "duplicate TensorView: " + name);
    const std::uint32_t want_location = want->location == wire::kDevice ? kPubDevice : kPubHost;
    if (view.dtype != ToPublicDType(want->dtype) || view.location != want_location)
      return Status(kInvalidArgument, "dtype or memory location mismatch for tensor: " + name);
    if (view.data == nullptr || view.byte_size < want->byte_size || view.rank != want->rank ||
        (view.rank != 0 && (view.shape == nullptr || view.stride == nullptr)))
      return Status(kInvalidArgument, "buffer, byte size, or rank mismatch for tensor: " + name);
    for (std::uint32_t d = 0; d < want->rank; ++d)
      if (view.shape[d] != want->shape[d] || view.stride[d] != want->stride[d])
        return Status(kInvalidArgument, "shape or stride is outside the selected profile: " + name);
    bound_[slot] = view.data;
  }
  return {};
}

Status Session::Upload(const std::uint8_t* src, std::uint64_t bytes) {
  const auto t0 = std::chrono::steady_clock::now();
  Status result;
  if ((flags_ & kBlockingUpload) != 0 || bytes <= kStageBytes) {
    result = cu_->Check(cu_->cuMemcpyHtoD(weights_, src, static_cast<std::size_t>(bytes)), "cuMemcpyHtoD");
  } else {
    // Two pinned buffers: the CPU fills one from the file mapping while the copy engine drains the other.
    void* stage[2] = {nullptr, nullptr};
    CUevent drained[2] = {nullptr, nullptr};
    CUstream stream = nullptr;
    result = cu_->Check(cu_->cuStreamCreate(&stream, CU_STREAM_NON_BLOCKING), "cuStreamCreate");
    for (int i = 0; i < 2 && result.ok(); ++i) {
      result = cu_->Check(cu_->cuMemHostAlloc(&stage[i], kStageBytes, 0), "cuMemHostAlloc", kOutOfMemory);
      if (result.ok()) result = cu_->Check(cu_->cuEventCreate(&drained[i], CU_EVENT_DISABLE_TIMING), "cuEventCreate");
    }
    std::uint64_t done = 0;
    for (int turn = 0; result.ok() && done < bytes; turn ^= 1) {
      const std::size_t chunk = static_cast<std::size_t>(std::min<std::uint64_t>(kStageBytes, bytes - done));
      if (done >= 2 * kStageBytes) result = cu_->Check(cu_->cuEventSynchronize(drained[turn]), "cuEventSynchronize");
      if (!result.ok()) break;
      std::memcpy(stage[turn], src + done, chunk);
      result = cu_->Check(cu_->cuMemcpyHtoDAsync(weights_ + done, stage[turn], chunk, stream), "cuMemcpyHtoDAsync");
      if (result.ok()) result = cu_->Check(cu_->cuEventRecord(drained[turn], stream), "cuEventRecord");
      done += chunk;
    }
    if (stream != nullptr) {
      const Status drained_all = cu_->Check(cu_->cuStreamSynchronize(stream), "cuStreamSynchronize");
      if (result.ok()) result = drained_all;
    }
    for (int i = 0; i < 2; ++i) {
      if (drained[i] != nullptr) cu_->cuEventDestroy(drained[i]);
      if (stage[i] != nullptr) cu_->cuMemFreeHost(stage[i]);
    }
    if (stream != nullptr) cu_->cuStreamDestroy(stream);
  }
  stats_.upload_seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
  return result;
}

Status Session::Prepare() {
  if (prepared_) return cu_->Check(cu_->cuCtxSetCurrent(context_), "cuCtxSetCurrent");
  std::string why;
  cu_ = CudaApi::Get(&why);
  if (cu_ == nullptr) return Status(kCudaError, why);
  AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuInit(0), "cuInit"));
  if (context_ == nullptr) {
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuCtxGetCurrent(&context_), "cuCtxGetCurrent"));
    if (context_ != nullptr) {
      AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuCtxGetDevice(&device_), "cuCtxGetDevice"));
    } else {
      AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuDeviceGet(&device_, 0), "cuDeviceGet"));
    }
    int major = 0, minor = 0;
    CUresult r = cu_->cuDeviceGetAttribute(&major, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MAJOR, device_);
    if (r == CUDA_SUCCESS) r = cu_->cuDeviceGetAttribute(&minor, CU_DEVICE_ATTRIBUTE_COMPUTE_CAPABILITY_MINOR, device_);
    if (r != CUDA_SUCCESS) {
      context_ = nullptr;
      return cu_->Check(r, "cuDeviceGetAttribute");
    }
    if (static_cast<std::uint32_t>(major * 10 + minor) != variant_->arch) {
      context_ = nullptr;
      return Status(kIncompatibleArchitecture, "active CUDA device does not match the selected AIM architecture");
    }
    if (context_ == nullptr) {
      AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuDevicePrimaryCtxRetain(&context_, device_), "cuDevicePrimaryCtxRetain"));
      retained_primary_ = true;
      AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuCtxSetCurrent(context_), "cuCtxSetCurrent"));
    }
  }
  // From here on a failure leaves the partially built state in place; the destructor frees it
  // and the next Enqueue starts over at the step that failed.
  if (module_ == nullptr)
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuModuleLoadData(&module_, package_->data() + variant_->kernel_offset),
                                   "cuModuleLoadData"));
  if (weights_ == 0) {
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuMemAlloc(&weights_, static_cast<std::size_t>(variant_->weight_size)),
                                   "cuMemAlloc", kOutOfMemory));
    const Status uploaded = Upload(package_->data() + variant_->weight_offset, variant_->weight_size);
    if (!uploaded.ok()) {
      cu_->cuMemFree(weights_);
      weights_ = 0;
      return uploaded;
    }
  }
  const std::uint64_t arena_bytes = plan_.header->arena_bytes, workspace_bytes = plan_.header->workspace_bytes;
  if (arena_ == 0 && arena_bytes != 0) {
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuMemAlloc(&arena_, static_cast<std::size_t>(arena_bytes)), "cuMemAlloc", kOutOfMemory));
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuMemsetD8Async(arena_, 0, static_cast<std::size_t>(arena_bytes), nullptr), "cuMemsetD8Async"));
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuStreamSynchronize(nullptr), "cuStreamSynchronize"));
  }
  if (workspace_ == 0 && workspace_bytes != 0)
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuMemAlloc(&workspace_, static_cast<std::size_t>(workspace_bytes)), "cuMemAlloc", kOutOfMemory));

  prepared_ = true;
  return {};
}

// Select the profile an Enqueue runs: the session's own, or its sibling for another number of denoising steps.
// A sibling must take and return exactly the tensors of the session's profile.
Status Session::Select(std::uint32_t denoising_steps) {
  if (denoising_steps == 0) {
    active_ = states_[0].get();
    return {};
  }
  const std::string name = std::string(plan_.Text(profile_->name)) + "/steps=" + std::to_string(denoising_steps);
  for (auto& state : states_)
    if (plan_.Text(state->profile->name) == name) {
      active_ = state.get();
      return {};
    }
  const wire::Profile* found = plan_.Find(name);
  if (found == nullptr)
    return Status(kInvalidArgument, "no recipe for " + std::to_string(denoising_steps) +
                                        " denoising steps in the static execution plan (profile " + name + ")");
  bool same = found->tensor_count == profile_->tensor_count;
  for (std::uint32_t i = 0; same && i < found->tensor_count; ++i) {
    const wire::Tensor& a = plan_.tensors[found->first_tensor + i];
    const wire::Tensor& b = plan_.tensors[profile_->first_tensor + i];
    same = plan_.Text(a.name) == plan_.Text(b.name) && a.dtype == b.dtype && a.location == b.location &&
           a.io_kind == b.io_kind && a.rank == b.rank && a.byte_size == b.byte_size &&
           std::memcmp(a.shape, b.shape, sizeof(a.shape)) == 0 && std::memcmp(a.stride, b.stride, sizeof(a.stride)) == 0;
  }
  if (!same) return Status(kCorruptPackage, "profile " + name + " does not have the tensors of the session's profile");
  states_.push_back(std::make_unique<ProfileState>());
  states_.back()->profile = found;
  active_ = states_.back().get();
  return {};
}

Status Session::Resolve() {
  ProfileState& state = *active_;
  if (state.resolved) return {};
  const wire::Profile* profile = state.profile;
  std::uint32_t widest = 0;
  for (std::uint32_t l = 0; l < profile->launch_count; ++l)
    widest = std::max(widest, plan_.launches[profile->first_launch + l].argument_count);
  if (slots_.size() < widest) {
    slots_.resize(widest);
    params_.resize(widest);
  }
  // Resolve each distinct kernel once; a function's dynamic shared-memory limit is a property of the
  // function, so it is raised to the largest request any launch of the profile makes.
  state.functions.clear();
  state.functions.reserve(profile->launch_count);
  state.cooperative.clear();
  std::vector<std::pair<std::uint32_t, CUfunction>> resolved;      // name offset -> function
  std::vector<std::uint32_t> shared_need;
  for (std::uint32_t l = 0; l < profile->launch_count; ++l) {
    const wire::Launch& launch = plan_.launches[profile->first_launch + l];
    std::size_t slot = 0;
    while (slot < resolved.size() && resolved[slot].first != launch.kernel) ++slot;
    if (slot == resolved.size()) {
      const std::string name(plan_.Text(launch.kernel));
      CUfunction fn = nullptr;
      AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuModuleGetFunction(&fn, module_, name.c_str()), "cuModuleGetFunction(" + name + ")"));
      resolved.emplace_back(launch.kernel, fn);
      shared_need.push_back(0);
    }
    shared_need[slot] = std::max(shared_need[slot], launch.shared_bytes);
    state.functions.push_back(resolved[slot].second);
    state.cooperative.push_back(plan_.Text(launch.kernel).rfind("agi_coop_", 0) == 0);
  }
  for (std::size_t slot = 0; slot < resolved.size(); ++slot) {
    // Ask for the same (largest) shared-memory carve-out for every kernel of the recipe: consecutive launches
    // then never make an SM wait to be re-partitioned between L1 and shared memory.  A hint; failure is ignored.
    cu_->cuFuncSetAttribute(resolved[slot].second, CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT,
                            CU_SHAREDMEM_CARVEOUT_MAX_SHARED);
    // Static and dynamic shared memory together may not pass 48 KB without the opt-in attribute.
    int static_bytes = 0;
    cu_->cuFuncGetAttribute(&static_bytes, CU_FUNC_ATTRIBUTE_SHARED_SIZE_BYTES, resolved[slot].second);
    if (shared_need[slot] + static_cast<std::uint32_t>(static_bytes) <= kStaticSharedLimit) continue;
    int granted = 0;   // another profile of this session may already have raised the limit further
    cu_->cuFuncGetAttribute(&granted, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, resolved[slot].second);
    if (granted >= static_cast<int>(shared_need[slot])) continue;
    const std::string name(plan_.Text(resolved[slot].first));
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuFuncSetAttribute(resolved[slot].second, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES,
                                                           static_cast<int>(shared_need[slot])),
                                   "cuFuncSetAttribute(" + name + ")"));
  }
  state.resolved = true;
  return {};
}

Status Session::Issue(CUstream stream) {
  for (std::uint32_t l = 0; l < active_->profile->launch_count; ++l) {
    const wire::Launch& launch = plan_.launches[active_->profile->first_launch + l];
    for (std::uint32_t a = 0; a < launch.argument_count; ++a) {
      const wire::Argument& arg = plan_.arguments[launch.first_argument + a];
      switch (arg.kind) {
        case wire::kTensor:
          slots_[a] = reinterpret_cast<std::uintptr_t>(bound_[arg.index - active_->profile->first_tensor]);
          break;
        case wire::kArenaOffset: slots_[a] = arena_ + arg.offset; break;
        case wire::kWeightsOffset: slots_[a] = weights_ + arg.offset; break;
        default: slots_[a] = arg.value; break;  // scalars: low four bytes are the kernel parameter
      }
      params_[a] = &slots_[a];
    }
    CUresult r;
    const bool cooperative = active_->cooperative[l] && (flags_ & kNoCooperativeLaunch) == 0;
    if (cooperative || ((flags_ & kProgrammaticLaunch) != 0 && l != 0)) {
      CUlaunchAttribute attr{};
      if (cooperative) {   // ordinary stream order in front of it: it starts when its predecessor has finished
        attr.id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE;
        attr.value.cooperative = 1;
      } else {
        attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attr.value.programmaticStreamSerializationAllowed = 1;
      }
      CUlaunchConfig cfg{};
      cfg.gridDimX = launch.grid[0]; cfg.gridDimY = launch.grid[1]; cfg.gridDimZ = launch.grid[2];
      cfg.blockDimX = launch.block[0]; cfg.blockDimY = launch.block[1]; cfg.blockDimZ = launch.block[2];
      cfg.sharedMemBytes = launch.shared_bytes;
      cfg.hStream = stream;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      r = cu_->cuLaunchKernelEx(&cfg, active_->functions[l], params_.data(), nullptr);
    } else {
      r = cu_->cuLaunchKernel(active_->functions[l], launch.grid[0], launch.grid[1], launch.grid[2], launch.block[0],
                              launch.block[1], launch.block[2], launch.shared_bytes, stream, params_.data(), nullptr);
    }
    ++stats_.kernel_launches;
    if (r != CUDA_SUCCESS) return cu_->Check(r, "cuLaunchKernel");
  }
  return {};
}

Status Session::Replay(CUstream stream) {
  const bool graph_safe = (active_->profile->flags & 1u) != 0 && (flags_ & kNoGraphReplay) == 0 && stream != nullptr;
  if (!graph_safe) return Issue(stream);
  CUstreamCaptureStatus capturing = CU_STREAM_CAPTURE_STATUS_NONE;
  if (cu_->cuStreamIsCapturing(stream, &capturing) != CUDA_SUCCESS || capturing != CU_STREAM_CAPTURE_STATUS_NONE)
    return Issue(stream);  // the caller is building its own graph: contribute plain launches

  CachedGraph* hit = nullptr;
  std::vector<CachedGraph>& graphs_ = active_->graphs;
  for (CachedGraph& g : graphs_)
    if (g.key == bound_) hit = &g;
  if (hit == nullptr) {
    AGI_RETURN_IF_ERROR(cu_->Check(cu_->cuStreamBeginCapture(stream, CU_STREAM_CAPTURE_MODE_THREAD_LOCAL), "cuStreamBeginCapture"));
    const Status issued = Issue(stream);
    CUgraph graph = nullptr;
    const CUresult ended = cu_->cuStreamEndCapture(stream, &graph);
    if (!issued.ok()) {
      if (graph != nullptr) cu_->cuGraphDestroy(graph);
      return issued;
    }
    AGI_RETURN_IF_ERROR(cu_->Check(ended, "cuStreamEndCapture"));
    CUgraphExec exec = nullptr;
    const CUresult built = cu_->cuGraphInstantiateWithFlags(&exec, graph, 0);
    cu_->cuGraphDestroy(graph);
    AGI_RETURN_IF_ERROR(cu_->Check(built, "cuGraphInstantiate"));
    ++stats_.graphs_built;
    if (graphs_.size() >= kMaxCachedGraphs) {
      auto oldest = std::min_element(graphs_.begin(), graphs_.end(),
                                     [](const CachedGraph& a, const CachedGraph& b) { return a.last_use < b.last_use; });
      cu_->cuGraphExecDestroy(oldest->exec);
      graphs_.erase(oldest);
    }
    graphs_.push_back(CachedGraph{bound_, exec, 0});
    hit = &graphs_.back();
  }
  hit->last_use = stats_.enqueues;
  ++stats_.graph_launches;
  return cu_->Check(cu_->cuGraphLaunch(hit->exec, stream), "cuGraphLaunch");
}

Status Session::Enqueue(const TensorArg* inputs, std::size_t input_count, const TensorArg* outputs,
                        std::size_t output_count, CUstream stream, const RunSelect& select) {
  AGI_RETURN_IF_ERROR(Select(select.denoising_steps));
  const wire::Profile* profile = active_->profile;
  std::vector<TensorArg> replaced;
  if (select.noise_override != nullptr) {
    // The override stands in for the input named "noise", whether or not the caller also passed one.
    bool has_noise = false;
    for (std::uint32_t i = 0; i < profile->tensor_count; ++i) {
      const wire::Tensor& t = plan_.tensors[profile->first_tensor + i];
      has_noise = has_noise || (t.io_kind == wire::kInput && plan_.Text(t.name) == "noise");
    }
    if (!has_noise) return Status(kInvalidArgument, "initial_noise_override: the selected profile has no input named noise");
    for (std::size_t i = 0; i < input_count; ++i)
      if (inputs[i].name == nullptr || std::string(inputs[i].name) != "noise") replaced.push_back(inputs[i]);
    TensorArg noise = *select.noise_override;
    noise.name = "noise";
    replaced.push_back(noise);
    inputs = replaced.data();
    input_count = replaced.size();
  }
  std::fill(bound_.begin(), bound_.end(), nullptr);
  std::size_t want_inputs = 0;
  for (std::uint32_t i = 0; i < profile->tensor_count; ++i)
    want_inputs += plan_.tensors[profile->first_tensor + i].io_kind == wire::kInput;
  if (input_count != want_inputs || output_count != profile->tensor_count - want_inputs)
    return Status(kInvalidArgument, "input or output tensor count does not match the selected profile");
  AGI_RETURN_IF_ERROR(Bind(inputs, input_count, wire::kInput));
  AGI_RETURN_IF_ERROR(Bind(outputs, output_count, wire::kOutput));
  AGI_RETURN_IF_ERROR(Prepare());
  AGI_RETURN_IF_ERROR(Resolve());
  ++stats_.enqueues;
  return Replay(stream);
}

}  // namespace agi

// Runtime options, and the Session that binds caller tensors and enqueues a profile's
// launch recipe.  Behaviour follows the reference's Runtime::Create, Session::Create and
// Session::Enqueue (cpp/runtime.cc:121-160, 245-355, 357-371, 427-506); the differences,
// all inside "how the same launches reach the GPU", are:
//   * weights are uploaded through two pinned staging buffers with asynchronous copies;
//   * the arena is zero-filled once after allocation;
//   * a launch that asks for more than 48 KB of dynamic shared memory gets the function
//     attribute that permits it;
//   * for a profile the package marks as graph-safe, the recipe is stream-captured on the
//     caller's stream at the first Enqueue for a given set of tensor addresses and replayed
//     with one graph launch afterwards (unless the caller is itself capturing, or passed the
//     legacy null stream, in which case launches are issued one by one as in the reference);
//   * the device is the current context's when there is one, else ordinal 0;
//   * kernels whose name starts with "agi_coop_" keep one CTA per SM resident and meet at grid-wide
//     counters: they are launched with the cooperative attribute, so that the driver refuses a grid that
//     cannot be resident at once instead of letting it wait for itself.
#pragma once

#include "cuda_api.h"
#include "package.h"
#include "plan_view.h"

#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace agi {

struct RuntimeOptions {
  std::uint32_t required_runtime_abi = kRuntimeAbi;
  std::uint32_t cuda_arch = 0;             // zero = probe
  std::uint32_t cuda_driver_version = 0;
  std::uint32_t cuda_runtime_version = 0;
  std::uint32_t cublaslt_abi = 0;
  std::uint32_t cudnn_abi = 0;
};

// Fills every zero field of `options` by inspecting the machine.
Status ProbeSystem(RuntimeOptions* options);

enum SessionFlags : std::uint32_t {
  kNoGraphReplay = 1u << 0,      // always issue launches one by one
  kProgrammaticLaunch = 1u << 1, // launch every kernel but the first with programmatic stream serialization
  kBlockingUpload = 1u << 2,     // upload weights with one blocking copy from the mapping, as the reference does
  kNoCooperativeLaunch = 1u << 3, // launch agi_coop_* kernels like any other (no co-residency guarantee from the driver)
};

// Public numbering of include/aginfer/runtime.h:61-62 in the reference.
enum PublicDType : std::uint32_t { kPubF32 = 0, kPubF16 = 1, kPubBF16 = 2, kPubF8E4M3 = 3, kPubI32 = 4 };
enum PublicLocation : std::uint32_t { kPubHost = 0, kPubDevice = 1 };

struct TensorArg {
  const char* name = nullptr;
  std::uint32_t dtype = 0;
  std::uint32_t location = kPubDevice;
  std::uint32_t rank = 0;
  const std::int64_t* shape = nullptr;
  const std::int64_t* stride = nullptr;
  void* data = nullptr;
  std::uint64_t byte_size = 0;
};

// What of the reference's RunOptions (include/aginfer/runtime.h:84-90) selects work: the number of denoising
// steps picks a sibling profile "<profile>/steps=<n>" of the session's profile (0 = the session's profile as
// packaged), and a noise override stands in for the input tensor named "noise".
struct RunSelect {
  std::uint32_t denoising_steps = 0;
  const TensorArg* noise_override = nullptr;
};

struct SessionStats {
  std::uint64_t enqueues = 0;
  std::uint64_t kernel_launches = 0;   // cuLaunchKernel(Ex) calls issued, captured ones included
  std::uint64_t graph_launches = 0;
  std::uint64_t graphs_built = 0;
  double upload_seconds = 0;
};

class Session {
 public:
  ~Session();
  Session(const Session&) = delete;
  Session& operator=(const Session&) = delete;

  static Status Create(const RuntimeOptions& runtime, const Package& package, const std::string& profile,
                       std::uint32_t flags, std::unique_ptr<Session>* out);

  std::uint32_t arch() const { return variant_->arch; }
  const PlanView& plan() const { return plan_; }
  const wire::Profile& profile() const { return *profile_; }
  // The profile the last Enqueue ran (the session's own, or a step-count sibling of it).
  const wire::Profile& active_profile() const { return *active_->profile; }
  const SessionStats& stats() const { return stats_; }
  bool HasProfile(const std::string& name) const { return plan_.Find(name) != nullptr; }

  Status Enqueue(const TensorArg* inputs, std::size_t input_count, const TensorArg* outputs,
                 std::size_t output_count, CUstream stream, const RunSelect& select = RunSelect());

 private:
  Session() = default;
  Status Bind(const TensorArg* views, std::size_t count, std::uint32_t io_kind);
  Status Prepare();                       // one-time CUDA set-up
  Status Upload(const std::uint8_t* src, std::uint64_t bytes);
  Status Issue(CUstream stream);          // the launch loop
  Status Replay(CUstream stream);         // graph path; falls back to Issue
  Status Select(std::uint32_t denoising_steps);   // points active_ at the profile to run
  Status Resolve();                       // functions and attributes of the active profile, once per profile

  const Package* package_ = nullptr;
  const wire::VariantEntry* variant_ = nullptr;
  PlanView plan_;
  const wire::Profile* profile_ = nullptr;
  std::uint32_t flags_ = 0;

  const CudaApi* cu_ = nullptr;
  bool prepared_ = false;
  CUdevice device_ = 0;
  CUcontext context_ = nullptr;
  bool retained_primary_ = false;
  CUmodule module_ = nullptr;
  CUdeviceptr weights_ = 0, arena_ = 0, workspace_ = 0;
  std::vector<void*> bound_;              // device address per profile tensor
  std::vector<std::uint64_t> slots_;
  std::vector<void*> params_;

  struct CachedGraph {
    std::vector<void*> key;
    CUgraphExec exec = nullptr;
    std::uint64_t last_use = 0;
  };
  // Per profile the session has run: the session's own first, step-count siblings as they are asked for.
  struct ProfileState {
    const wire::Profile* profile = nullptr;
    bool resolved = false;
    std::vector<CUfunction> functions;    // one per launch of the profile
    std::vector<bool> cooperative;        // per launch: kernel name starts with "agi_coop_"
    std::vector<CachedGraph> graphs;
  };
  std::vector<std::unique_ptr<ProfileState>> states_;
  ProfileState* active_ = nullptr;
  SessionStats stats_;
};

}  // namespace agi

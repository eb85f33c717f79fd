/* C ABI of the B200 loader for AIM packages.
 *
 * Every entry point stands for one member of the reference's C++ API
 * (include/aginfer/runtime.h in wenhuiNi/AgInfer, cited per function as runtime.h:LINE,
 * implemented there in cpp/runtime.cc).  Argument meaning, status codes and error
 * conditions are the reference's; objects are opaque handles, vectors become
 * pointer + count, strings are NUL-terminated UTF-8.
 *
 * Each function returns an agi_status (0 = OK).  The text of the most recent failure on
 * the calling thread is available from agi_last_error().  Handles are not thread-safe:
 * use one session per thread / GPU, as with the reference (runtime.cc:226-228).
 * A session borrows its runtime and model; destroy the session first.
 */
#ifndef AGINFER_B200_H_
#define AGINFER_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define AGI_API __attribute__((visibility("default")))
#else
#define AGI_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* runtime.h:14-25 StatusCode, same numbering. */
typedef enum agi_status {
  AGI_OK = 0,
  AGI_INVALID_ARGUMENT = 1,
  AGI_NOT_FOUND = 2,
  AGI_IO_ERROR = 3,
  AGI_CORRUPT_PACKAGE = 4,
  AGI_INCOMPATIBLE_PLATFORM = 5,
  AGI_INCOMPATIBLE_ARCHITECTURE = 6,
  AGI_INCOMPATIBLE_ABI = 7,
  AGI_CUDA_ERROR = 8,
  AGI_OUT_OF_MEMORY = 9
} agi_status;

/* runtime.h:61-62 DType / MemoryLocation, same numbering. */
typedef enum agi_dtype { AGI_F32 = 0, AGI_F16 = 1, AGI_BF16 = 2, AGI_F8_E4M3 = 3, AGI_I32 = 4 } agi_dtype;
typedef enum agi_location { AGI_HOST = 0, AGI_DEVICE = 1 } agi_location;

#define AGI_RUNTIME_ABI 1u   /* runtime.h:12 kRuntimeAbi */
#define AGI_MAX_RANK 8

/* runtime.h:92-101 RuntimeOptions.  Zero in an override field means "probe the machine". */
typedef struct agi_runtime_options {
  uint32_t required_runtime_abi;
  uint32_t cuda_arch_override;
  uint32_t cuda_driver_version_override;
  uint32_t cuda_runtime_version_override;
  uint32_t cublaslt_abi_override;
  uint32_t cudnn_abi_override;
} agi_runtime_options;

/* runtime.h:64-73 TensorView (caller-owned buffer handed to Enqueue). */
typedef struct agi_tensor_view {
  const char* name;
  uint32_t dtype;      /* agi_dtype */
  uint32_t location;   /* agi_location */
  uint32_t rank;
  uint32_t reserved;   /* must be 0 */
  const int64_t* shape;   /* rank entries */
  const int64_t* stride;  /* rank entries, in elements */
  void* data;
  uint64_t byte_size;
} agi_tensor_view;

/* runtime.h:75-82 TensorInfo (what a profile expects). `name` stays valid while the model lives. */
typedef struct agi_tensor_info {
  const char* name;
  uint32_t dtype;
  uint32_t location;
  uint32_t rank;
  uint32_t reserved;
  int64_t shape[AGI_MAX_RANK];
  int64_t stride[AGI_MAX_RANK];
  uint64_t byte_size;
} agi_tensor_info;

/* runtime.h:84-90 RunOptions.  The reference accepts and ignores them (runtime.cc:499-500); here the two
 * that can select work in a static plan do:
 *   denoising_steps: 0 runs the session's profile as packaged; n > 0 runs its sibling profile
 *     "<profile>/steps=<n>" (a recipe unrolled for n Euler steps, same tensors), AGI_INVALID_ARGUMENT when
 *     the package carries none for n;
 *   initial_noise_override: when not NULL, stands in for the input tensor named "noise" (its own `name`
 *     is not looked at; validated against the profile like any other view; AGI_INVALID_ARGUMENT when the
 *     profile has no such input).  The caller may then leave "noise" out of `inputs`.
 * seed, deterministic and math_mode stay without effect: noise is an explicit input, every kernel of the
 * bundle is deterministic, and the arithmetic of a recipe is fixed when it is packaged. */
typedef struct agi_run_options {
  uint32_t denoising_steps;
  uint32_t deterministic;
  uint64_t seed;
  uint32_t math_mode;
  uint32_t reserved;
  const agi_tensor_view* initial_noise_override;
} agi_run_options;

/* Session behaviour switches (no counterpart in the reference; all default to off = 0). */
#define AGI_SESSION_NO_GRAPH_REPLAY   (1u << 0) /* issue every launch with cuLaunchKernel, as the reference does */
#define AGI_SESSION_PROGRAMMATIC_LAUNCH (1u << 1) /* programmatic stream serialization between consecutive launches */
#define AGI_SESSION_BLOCKING_UPLOAD   (1u << 2) /* one blocking cuMemcpyHtoD of the weights, as the reference does */
#define AGI_SESSION_NO_COOPERATIVE_LAUNCH (1u << 3) /* launch agi_coop_* kernels without the cooperative attribute */

typedef struct agi_runtime agi_runtime;
typedef struct agi_model agi_model;
typedef struct agi_session agi_session;

/* runtime.h:178 StatusCodeName. */
AGI_API const char* agi_status_name(int status);
/* Message of the last failing call on this thread ("" if none). */
AGI_API const char* agi_last_error(void);
/* Library identification: "aginfer-b200 <version> abi <n> sha256=<backend>". */
AGI_API const char* agi_version(void);

/* runtime.h:129 Runtime::Create.  `options` may be NULL (all defaults, probe everything). */
AGI_API agi_status agi_runtime_create(const agi_runtime_options* options, agi_runtime** out);
AGI_API void agi_runtime_destroy(agi_runtime* runtime);
/* The options after probing (what Session::Create compares the manifest against). */
AGI_API agi_status agi_runtime_get_options(const agi_runtime* runtime, agi_runtime_options* out);

/* runtime.h:146 Model::Load: mmap, integrity and target checks of an .aim file. */
AGI_API agi_status agi_model_load(const char* aim_path, agi_model** out);
AGI_API void agi_model_destroy(agi_model* model);
/* Number of variants and the numeric architecture of variant `index`. */
AGI_API agi_status agi_model_variant_count(const agi_model* model, uint32_t* out);
AGI_API agi_status agi_model_variant_arch(const agi_model* model, uint32_t index, uint32_t* out);

/* runtime.h:162-163 Session::Create.  `profile` NULL or "" selects the plan's first profile.
 * `flags` is a mask of AGI_SESSION_*. */
AGI_API agi_status agi_session_create(agi_runtime* runtime, agi_model* model, const char* profile, uint32_t flags,
                              agi_session** out);
AGI_API void agi_session_destroy(agi_session* session);

/* runtime.h:164 Session::GetTargetInfo.  Strings stay valid while the session lives. */
AGI_API agi_status agi_session_get_target_info(const agi_session* session, const char** platform, const char** cuda_arch,
                                       uint32_t* runtime_abi);
/* runtime.h:165-166 Session::GetInputInfo / GetOutputInfo: count, then one record per index. */
AGI_API agi_status agi_session_get_input_count(const agi_session* session, uint32_t* out);
AGI_API agi_status agi_session_get_output_count(const agi_session* session, uint32_t* out);
AGI_API agi_status agi_session_get_input_info(const agi_session* session, uint32_t index, agi_tensor_info* out);
AGI_API agi_status agi_session_get_output_info(const agi_session* session, uint32_t index, agi_tensor_info* out);
/* runtime.h:167 Session::GetRequiredWorkspace. `profile` NULL or "" skips the name check. */
AGI_API agi_status agi_session_get_required_workspace(const agi_session* session, const char* profile,
                                              uint64_t* arena_bytes, uint64_t* workspace_bytes);
/* runtime.h:168-170 Session::Enqueue: validate the views against the profile, initialise CUDA
 * resources on the first call (synchronous), then submit the recipe on `stream` (a CUstream /
 * cudaStream_t, or NULL for the legacy default stream) and return without waiting. */
AGI_API agi_status agi_session_enqueue(agi_session* session, const agi_tensor_view* inputs, size_t input_count,
                               const agi_tensor_view* outputs, size_t output_count, const agi_run_options* options,
                               void* stream);

/* Counters since session creation (no counterpart in the reference). */
typedef struct agi_session_stats {
  uint64_t enqueues;
  uint64_t kernel_launches;   /* cuLaunchKernel calls issued, including those recorded into a graph */
  uint64_t graph_launches;    /* Enqueue calls served by replaying a captured graph */
  uint64_t graphs_built;
  uint64_t launches_per_enqueue; /* launch records in the profile the last Enqueue ran */
  double upload_seconds;      /* wall time of the one-time weight upload */
} agi_session_stats;
AGI_API agi_status agi_session_get_stats(const agi_session* session, agi_session_stats* out);

/* No counterpart in the reference.  Y[M,N] (bf16) = X[M,K] . W[N,K]^T (+ bias[N]) with the split-K
 * tensor-core kernel of the sm100 bundle, for callers that may not allocate device memory (real-time
 * loops with a frozen memory map, plug-in hooks and callbacks of other frameworks, processes whose
 * memory budget is already spent): the split-K scratch is a fixed array inside the library image, so
 * the call makes no cudaMalloc / cudaFree and no allocating library call.  All pointers are device
 * pointers on the current device; `bias` may be NULL; K must be a multiple of 64; `splits` (1..16) is the
 * number of K slices.  Limit: splits * M * roundup(N, 128) * 4 bytes <= 8 MiB and at most 1024 output
 * tiles, otherwise AGI_INVALID_ARGUMENT.  The array is shared by every call on a device and keeps the
 * last call's contents (what must be zero is cleared on `stream` first); calls that overlap on one GPU
 * race.  `x` and `w` must be 16-byte aligned (the kernel fetches them with 16-byte copies), `y` and `bias`
 * 2-byte aligned; anything else is refused with AGI_INVALID_ARGUMENT before a launch.  The first call on
 * each device performs one-time synchronous set-up (symbol address lookup, kernel attribute): make it
 * during start-up, before any stream capture; the looked-up address is cached for the life of the
 * process, so do not use the entry point on a device after cudaDeviceReset. */
AGI_API agi_status agi_gemm_bf16_static_scratch(const void* x, const void* w, void* y, const void* bias, uint32_t M,
                                                uint32_t N, uint32_t K, uint32_t splits, void* stream);
/* No counterpart in the reference.  Copies the wait-status word of the static-scratch GEMM (first word of
 * the built-in array; 0 = every bounded wait inside the kernel was satisfied, anything else = the output
 * of the last call on this device is not to be trusted) into `out`, a 4-byte aligned device or pinned
 * host word, with one cudaMemcpyAsync on `stream`: enqueue it behind the GEMM it reports on.  Allocates
 * nothing. */
AGI_API agi_status agi_gemm_bf16_static_scratch_status(uint32_t* out, void* stream);

/* SHA-256 of a buffer with the library's hasher (test hook; `portable` != 0 forces the
 * non-accelerated block function). Role of cpp/sha256.cc:58-103. */
AGI_API agi_status agi_sha256(const void* data, size_t size, int portable, uint8_t out[32]);

#ifdef __cplusplus
}
#endif
#endif /* AGINFER_B200_H_ */

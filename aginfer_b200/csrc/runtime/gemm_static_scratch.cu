// agi_gemm_bf16_static_scratch: the split-K tensor-core GEMM for callers that must not allocate.
//
// Who needs this.  Some hosts of this library run where device allocation is off limits: inside a
// real-time control loop that has frozen its memory map after start-up, inside another framework's
// stream callback or plug-in hook where calling cudaMalloc would deadlock or is simply forbidden by
// the host's rules, or in a process whose memory budget was handed out in full before this library
// was loaded.  The packaged path (Session::Enqueue) gets its split-K scratch from the session arena,
// which the loader allocates; this entry point instead keeps the scratch in a fixed array that is part
// of the library image itself, so a call performs no cudaMalloc, no cudaFree and no allocating library
// call of any kind.
//
// What it costs.  Every GPU that loads the library carries the array (kScratchBytes, a little over
// 8 MiB) until the process exits, whether or not the entry point is ever called.  Shapes whose partial
// tiles do not fit are refused with AGI_INVALID_ARGUMENT; nothing falls back to allocating.
//
// Sharing.  There is one array per device and every call on that device uses it.  It keeps whatever the
// last call left; the parts that must start at zero (the per-tile arrival counters and the status word)
// are cleared on the caller's stream at the start of each call.  Two calls that overlap on one GPU
// (different streams, or different host threads) race on the array and give wrong results: serialise
// them on one stream.
//
// Set-up.  The first call on each device looks up the array's device address and raises the kernel's
// dynamic shared-memory limit; both are one-time, per-device, synchronous host calls.  Make that first
// call during start-up, outside any stream capture.  The looked-up address is cached per device for the
// life of the process: after cudaDeviceReset the cache is stale, so a process that resets a device must
// not use this entry point on it again.
//
// Waits.  Every wait inside the kernel is bounded; one that runs out records a code in the first word of the
// array and the kernel carries on, so the output is then wrong while the launch still succeeds.
// agi_gemm_bf16_static_scratch_status copies that word to the caller (0 = every wait was satisfied).
#include "aginfer_b200.h"

#include "../kernels/gemm_tc.cuh"
#include "error_slot.h"

#include <cuda_runtime.h>

#include <cstdint>
#include <mutex>
#include <string>

namespace {

constexpr unsigned kMaxTiles = 1024;                   // per-tile arrival counters
constexpr size_t kPartialBytes = size_t(8) << 20;      // fp32 partial tiles, [slice][M][N rounded up to 128]
constexpr size_t kStatusBytes = 256;
constexpr size_t kCounterBytes = kMaxTiles * sizeof(unsigned);
constexpr size_t kScratchBytes = kStatusBytes + kCounterBytes + kPartialBytes;
constexpr int kMaxDevices = 64;
constexpr unsigned kSmemBudget = 200 * 1024;

// Lives in the library image on every device that loads it.  In host code this name is only a handle
// for cudaGetSymbolAddress: it is not a device address and must never be passed to a kernel as one.
static __device__ __align__(256) unsigned char g_static_scratch[kScratchBytes];

std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};

agi_status Cuda(cudaError_t result, const char* what) {
  if (result == cudaSuccess) return AGI_OK;
  return agi::RecordFailure(AGI_CUDA_ERROR, std::string(what) + " failed: " + cudaGetErrorName(result) + " (" +
                                                cudaGetErrorString(result) + ")");
}

// Device address of the scratch array on the current device; resolved once per device.
agi_status ScratchOnCurrentDevice(unsigned char** out) {
  int device = 0;
  if (agi_status s = Cuda(cudaGetDevice(&device), "cudaGetDevice")) return s;
  if (device < 0 || device >= kMaxDevices)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "device ordinal is outside the supported range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* address = nullptr;
    if (agi_status s = Cuda(cudaGetSymbolAddress(&address, g_static_scratch), "cudaGetSymbolAddress")) return s;
    if (agi_status s = Cuda(cudaFuncSetAttribute(agi_gemm_tc_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 int(kSmemBudget + 1024)),
                            "cudaFuncSetAttribute"))
      return s;
    g_scratch_address[device] = static_cast<unsigned char*>(address);
  }
  *out = g_scratch_address[device];
  return AGI_OK;
}

std::uint64_t CeilDiv(std::uint64_t a, std::uint64_t b) { return (a + b - 1) / b; }

bool Aligned(const void* p, std::uintptr_t to) { return (reinterpret_cast<std::uintptr_t>(p) & (to - 1)) == 0; }

}  // namespace

extern "C" agi_status agi_gemm_bf16_static_scratch(const void* x, const void* w, void* y, const void* bias, uint32_t M,
                                                   uint32_t N, uint32_t K, uint32_t splits, void* stream) {
  if (x == nullptr || w == nullptr || y == nullptr)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "x, w and y must not be NULL");
  // The kernel fetches X and W with 16-byte asynchronous copies: a base address off that boundary would be a
  // misaligned-address fault on the GPU, so it is refused here, on the host.
  if (!Aligned(x, 16) || !Aligned(w, 16))
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "x and w must be 16-byte aligned device pointers");
  if (!Aligned(y, 2) || !Aligned(bias, 2))
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "y and bias must be 2-byte aligned (bf16) device pointers");
  if (M == 0 || N == 0 || K == 0 || K % 64u != 0)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "M, N, K must be positive and K a multiple of 64 elements");
  // Grid limits of the launch: blockIdx.y walks token tiles of up to 256, blockIdx.x feature tiles of 128.
  if (M > 256u * 65535u || K > 0x7fffffc0u)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "M or K is beyond what one launch can cover");
  // Same geometry rules as the packaged recipe: token tile a multiple of 16 up to 256, 128 rows of W per CTA.
  const std::uint64_t m_tiles = CeilDiv(M, 256), TN = CeilDiv(CeilDiv(M, m_tiles), 16) * 16;
  const std::uint64_t n_tiles = CeilDiv(N, 128), tiles = n_tiles * m_tiles, k_blocks = std::uint64_t(K) * 2 / 128;
  if (splits == 0) splits = 1;
  if (splits > 16 || splits > k_blocks)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "splits must be between 1 and min(16, K / 64)");
  const std::uint64_t per = CeilDiv(k_blocks, splits);
  splits = static_cast<uint32_t>(CeilDiv(k_blocks, per));
  // One K slice needs neither partial tiles nor arrival counters.
  const std::uint64_t need = splits > 1 ? std::uint64_t(splits) * M * n_tiles * 128 * sizeof(float) : 0;
  if (splits > 1 && (tiles > kMaxTiles || need > kPartialBytes))
    return agi::RecordFailure(
        AGI_INVALID_ARGUMENT,
        "shape needs " + std::to_string(need) + " bytes of split-K scratch and " + std::to_string(tiles) +
            " tile counters; the built-in array holds " + std::to_string(kPartialBytes) + " bytes and " +
            std::to_string(kMaxTiles) + " counters (use fewer splits, or the session path)");
  const unsigned stage_bytes = 16384 + unsigned(TN) * 128;
  const unsigned depth = per < 3 ? 3u : unsigned(per > 12 ? 12 : per);
  unsigned stages = kSmemBudget / stage_bytes;
  if (stages > 12) stages = 12;
  if (stages > depth) stages = depth;
  if (stages < 3) stages = 3;
  const unsigned shared_bytes = stages * stage_bytes + 1024;

  unsigned char* scratch = nullptr;
  if (agi_status s = ScratchOnCurrentDevice(&scratch)) return s;
  cudaStream_t cu_stream = static_cast<cudaStream_t>(stream);
  unsigned* status = reinterpret_cast<unsigned*>(scratch);
  unsigned* counters = reinterpret_cast<unsigned*>(scratch + kStatusBytes);
  float* partial = reinterpret_cast<float*>(scratch + kStatusBytes + kCounterBytes);
  // The array keeps the previous call's contents: counters and status must start at zero.
  if (agi_status s = Cuda(cudaMemsetAsync(scratch, 0, kStatusBytes + kCounterBytes, cu_stream), "cudaMemsetAsync"))
    return s;
  const unsigned flags = bias != nullptr ? kFlagBias : 0u;
  const bf16* dummy = static_cast<const bf16*>(y);  // never dereferenced when its flag is off
  agi_gemm_tc_bf16<<<dim3(unsigned(n_tiles), unsigned(m_tiles), splits), tc::kThreads, shared_bytes, cu_stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(w), y, bias != nullptr ? static_cast<const bf16*>(bias) : dummy,
      dummy, reinterpret_cast<const float*>(status), reinterpret_cast<const float*>(status), partial, counters, status,
      M, N, K, K, N, flags, unsigned(TN), stages);
  return Cuda(cudaGetLastError(), "agi_gemm_tc_bf16 launch");
}

extern "C" agi_status agi_gemm_bf16_static_scratch_status(uint32_t* out, void* stream) {
  if (out == nullptr || !Aligned(out, 4))
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "out must be a 4-byte aligned device or pinned host word");
  unsigned char* scratch = nullptr;
  if (agi_status s = ScratchOnCurrentDevice(&scratch)) return s;
  // Ordered on `stream` behind the GEMM whose waits it reports; copies four bytes, allocates nothing.
  return Cuda(cudaMemcpyAsync(out, scratch, sizeof(uint32_t), cudaMemcpyDefault, static_cast<cudaStream_t>(stream)),
              "cudaMemcpyAsync");
}

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
// call during start-up, outside any stream capture.
#include "aginfer_b200.h"

#include "../kernels/gemm_tc.cuh"
#include "error_slot.h"

#include <cuda_runtime.h>

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

unsigned CeilDiv(unsigned a, unsigned b) { return (a + b - 1) / b; }

}  // namespace

extern "C" agi_status agi_gemm_bf16_static_scratch(const void* x, const void* w, void* y, const void* bias, uint32_t M,
                                                   uint32_t N, uint32_t K, uint32_t splits, void* stream) {
  if (x == nullptr || w == nullptr || y == nullptr)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "x, w and y must not be NULL");
  if (M == 0 || N == 0 || K == 0 || (K * 2u) % 128u != 0)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "M, N, K must be positive and K a multiple of 64 elements");
  // Same geometry rules as the packaged recipe: token tile a multiple of 16 up to 256, 128 rows of W per CTA.
  const unsigned m_tiles = CeilDiv(M, 256), TN = CeilDiv(CeilDiv(M, m_tiles), 16) * 16;
  const unsigned n_tiles = CeilDiv(N, 128), tiles = n_tiles * m_tiles, k_blocks = K * 2u / 128u;
  if (splits == 0) splits = 1;
  if (splits > 16 || splits > k_blocks)
    return agi::RecordFailure(AGI_INVALID_ARGUMENT, "splits must be between 1 and min(16, K / 64)");
  const unsigned per = CeilDiv(k_blocks, splits);
  splits = CeilDiv(k_blocks, per);
  const size_t need = splits > 1 ? size_t(splits) * M * n_tiles * 128 * sizeof(float) : 0;
  if (tiles > kMaxTiles || need > kPartialBytes)
    return agi::RecordFailure(
        AGI_INVALID_ARGUMENT,
        "shape needs " + std::to_string(need) + " bytes of split-K scratch and " + std::to_string(tiles) +
            " tile counters; the built-in array holds " + std::to_string(kPartialBytes) + " bytes and " +
            std::to_string(kMaxTiles) + " counters (use fewer splits, or the session path)");
  const unsigned stage_bytes = 16384 + TN * 128;
  unsigned stages = kSmemBudget / stage_bytes;
  if (stages > 12) stages = 12;
  if (stages > (per < 3 ? 3u : per)) stages = per < 3 ? 3u : per;
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
  agi_gemm_tc_bf16<<<dim3(n_tiles, m_tiles, splits), tc::kThreads, shared_bytes, cu_stream>>>(
      static_cast<const bf16*>(x), static_cast<const bf16*>(w), y, bias != nullptr ? static_cast<const bf16*>(bias) : dummy,
      dummy, reinterpret_cast<const float*>(status), reinterpret_cast<const float*>(status), partial, counters, status,
      M, N, K, K, N, flags, TN, stages);
  return Cuda(cudaGetLastError(), "agi_gemm_tc_bf16 launch");
}

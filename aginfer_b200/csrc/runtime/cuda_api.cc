#include "cuda_api.h"

#include <dlfcn.h>

#include <mutex>

namespace agi {
namespace {

template <typename Fn>
bool Bind(void* lib, const char* symbol, Fn* slot) {
  *slot = reinterpret_cast<Fn>(dlsym(lib, symbol));
  return *slot != nullptr;
}

}  // namespace

std::string CudaApi::Explain(CUresult result, const std::string& what) const {
  const char* name = nullptr;
  const char* text = nullptr;
  if (cuGetErrorName != nullptr) cuGetErrorName(result, &name);
  if (cuGetErrorString != nullptr) cuGetErrorString(result, &text);
  std::string message = what + " failed";
  if (name != nullptr) message += ": " + std::string(name);
  if (text != nullptr) message += " (" + std::string(text) + ")";
  return message;
}

const CudaApi* CudaApi::Get(std::string* why) {
  static std::mutex mutex;
  static CudaApi table;
  static int state = 0;  // 0 = untried, 1 = ready, -1 = unusable
  static std::string failure;
  std::lock_guard<std::mutex> lock(mutex);
  if (state == 0) {
    void* lib = dlopen("libcuda.so.1", RTLD_NOW | RTLD_LOCAL);
    if (lib == nullptr) lib = dlopen("libcuda.so", RTLD_NOW | RTLD_LOCAL);
    if (lib == nullptr) {
      failure = "cannot load the CUDA Driver library";
      state = -1;
    } else {
      bool ok = true;
#define AGI_BIND(field, symbol) ok = Bind(lib, symbol, &table.field) && ok
      AGI_BIND(cuInit, "cuInit");
      AGI_BIND(cuDriverGetVersion, "cuDriverGetVersion");
      AGI_BIND(cuDeviceGet, "cuDeviceGet");
      AGI_BIND(cuDeviceGetAttribute, "cuDeviceGetAttribute");
      AGI_BIND(cuGetErrorName, "cuGetErrorName");
      AGI_BIND(cuGetErrorString, "cuGetErrorString");
      AGI_BIND(cuCtxGetCurrent, "cuCtxGetCurrent");
      AGI_BIND(cuCtxSetCurrent, "cuCtxSetCurrent");
      AGI_BIND(cuCtxGetDevice, "cuCtxGetDevice");
      AGI_BIND(cuDevicePrimaryCtxRetain, "cuDevicePrimaryCtxRetain");
      AGI_BIND(cuDevicePrimaryCtxRelease, "cuDevicePrimaryCtxRelease_v2");
      AGI_BIND(cuModuleLoadData, "cuModuleLoadData");
      AGI_BIND(cuModuleGetFunction, "cuModuleGetFunction");
      AGI_BIND(cuModuleUnload, "cuModuleUnload");
      AGI_BIND(cuFuncSetAttribute, "cuFuncSetAttribute");
      AGI_BIND(cuFuncGetAttribute, "cuFuncGetAttribute");
      AGI_BIND(cuMemAlloc, "cuMemAlloc_v2");
      AGI_BIND(cuMemFree, "cuMemFree_v2");
      AGI_BIND(cuMemHostAlloc, "cuMemHostAlloc");
      AGI_BIND(cuMemFreeHost, "cuMemFreeHost");
      AGI_BIND(cuMemcpyHtoD, "cuMemcpyHtoD_v2");
      AGI_BIND(cuMemcpyHtoDAsync, "cuMemcpyHtoDAsync_v2");
      AGI_BIND(cuMemsetD8Async, "cuMemsetD8Async");
      AGI_BIND(cuStreamCreate, "cuStreamCreate");
      AGI_BIND(cuStreamDestroy, "cuStreamDestroy_v2");
      AGI_BIND(cuStreamSynchronize, "cuStreamSynchronize");
      AGI_BIND(cuEventCreate, "cuEventCreate");
      AGI_BIND(cuEventDestroy, "cuEventDestroy_v2");
      AGI_BIND(cuEventRecord, "cuEventRecord");
      AGI_BIND(cuEventSynchronize, "cuEventSynchronize");
      AGI_BIND(cuLaunchKernel, "cuLaunchKernel");
      AGI_BIND(cuLaunchKernelEx, "cuLaunchKernelEx");
      AGI_BIND(cuStreamIsCapturing, "cuStreamIsCapturing");
      AGI_BIND(cuStreamBeginCapture, "cuStreamBeginCapture_v2");
      AGI_BIND(cuStreamEndCapture, "cuStreamEndCapture");
      AGI_BIND(cuGraphInstantiateWithFlags, "cuGraphInstantiateWithFlags");
      AGI_BIND(cuGraphLaunch, "cuGraphLaunch");
      AGI_BIND(cuGraphExecDestroy, "cuGraphExecDestroy");
      AGI_BIND(cuGraphDestroy, "cuGraphDestroy");
#undef AGI_BIND
      if (!ok) {
        failure = "CUDA Driver library is missing required symbols";
        state = -1;
      } else {
        state = 1;  // the library stays loaded for the life of the process
      }
    }
  }
  if (state < 0) {
    if (why != nullptr) *why = failure;
    return nullptr;
  }
  return &table;
}

}  // namespace agi

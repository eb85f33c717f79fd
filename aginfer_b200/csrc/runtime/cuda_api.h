// The CUDA Driver API, resolved at run time from libcuda.so.1 (role of the reference's
// cpp/cuda_driver.{h,cc}).  Nothing here links against CUDA: <cuda.h> supplies types only,
// so the library loads on machines without a driver and fails with CUDA_ERROR when asked
// to run.  Beyond the calls the reference uses, the table holds what the B200 session
// needs: async copies from pinned staging, function attributes for > 48 KB of dynamic
// shared memory, stream capture / graph replay and attribute-carrying launches.
#pragma once

#include "status.h"

#include <cuda.h>

#include <string>

namespace agi {

struct CudaApi {
  // Process-wide table; `Get` returns nullptr and fills `why` when the driver is unusable.
  static const CudaApi* Get(std::string* why);

  std::string Explain(CUresult result, const std::string& what) const;
  Status Check(CUresult result, const std::string& what, Code code = kCudaError) const {
    return result == CUDA_SUCCESS ? Status() : Status(code, Explain(result, what));
  }

#define AGI_CUDA_FN(name) decltype(&::name) name = nullptr
  AGI_CUDA_FN(cuInit);
  AGI_CUDA_FN(cuDriverGetVersion);
  AGI_CUDA_FN(cuDeviceGet);
  AGI_CUDA_FN(cuDeviceGetAttribute);
  AGI_CUDA_FN(cuGetErrorName);
  AGI_CUDA_FN(cuGetErrorString);
  AGI_CUDA_FN(cuCtxGetCurrent);
  AGI_CUDA_FN(cuCtxSetCurrent);
  AGI_CUDA_FN(cuCtxGetDevice);
  AGI_CUDA_FN(cuDevicePrimaryCtxRetain);
  AGI_CUDA_FN(cuDevicePrimaryCtxRelease);
  AGI_CUDA_FN(cuModuleLoadData);
  AGI_CUDA_FN(cuModuleGetFunction);
  AGI_CUDA_FN(cuModuleUnload);
  AGI_CUDA_FN(cuFuncSetAttribute);
  AGI_CUDA_FN(cuFuncGetAttribute);
  AGI_CUDA_FN(cuMemAlloc);
  AGI_CUDA_FN(cuMemFree);
  AGI_CUDA_FN(cuMemHostAlloc);
  AGI_CUDA_FN(cuMemFreeHost);
  AGI_CUDA_FN(cuMemcpyHtoD);
  AGI_CUDA_FN(cuMemcpyHtoDAsync);
  AGI_CUDA_FN(cuMemsetD8Async);
  AGI_CUDA_FN(cuStreamCreate);
  AGI_CUDA_FN(cuStreamDestroy);
  AGI_CUDA_FN(cuStreamSynchronize);
  AGI_CUDA_FN(cuEventCreate);
  AGI_CUDA_FN(cuEventDestroy);
  AGI_CUDA_FN(cuEventRecord);
  AGI_CUDA_FN(cuEventSynchronize);
  AGI_CUDA_FN(cuLaunchKernel);
  AGI_CUDA_FN(cuLaunchKernelEx);
  AGI_CUDA_FN(cuStreamIsCapturing);
  AGI_CUDA_FN(cuStreamBeginCapture);
  AGI_CUDA_FN(cuStreamEndCapture);
  AGI_CUDA_FN(cuGraphInstantiateWithFlags);
  AGI_CUDA_FN(cuGraphLaunch);
  AGI_CUDA_FN(cuGraphExecDestroy);
  AGI_CUDA_FN(cuGraphDestroy);
#undef AGI_CUDA_FN
};

}  // namespace agi

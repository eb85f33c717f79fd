// Shared device helpers for the sm_100a kernel bundle.
//
// Calling convention of every kernel in the bundle (AgInfer Kernel ABI 1.0,
// docs/kernel-abi-v1.md:39-53 in the reference): `extern "C" __global__`, parameters are
// device pointers, `unsigned` and `float` only, in plan-argument order; nothing is
// allocated, discovered or tuned on the device.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

// Epilogue / behaviour flags shared by the GEMM kernels (one `unsigned flags` parameter).
enum : unsigned {
  kFlagBias = 1u << 0,       // add bias[n]
  kFlagResidual = 1u << 1,   // add residual[m, n] (bf16, same leading dimension as the output)
  kFlagActMask = 0xFu << 4,  // activation applied after bias: 0 none, 1 GELU(tanh), 2 SiLU, 3 ReLU
  kActGeluTanh = 1u << 4,
  kActSilu = 2u << 4,
  kActRelu = 3u << 4,
  kFlagOutF32 = 1u << 8,     // write fp32 instead of bf16
  kFlagScaled = 1u << 9,     // multiply the accumulator by *scale_a * *scale_w (FP8 path)
  kFlagLayerNorm = 1u << 10, // fused prologue: LayerNorm (no affine) over each activation row before the GEMM
  kFlagLnModulate = 1u << 11, // ... followed by y * (1 + scale[k]) + shift[k] (AdaLN)
  kFlagSlab = 1u << 12,       // bulk-stream GEMM: whole K in one slot, rows unpadded, one copy per operand
};

// Programmatic dependent launch: when the loader launches with programmatic stream
// serialization, a kernel may start while its predecessor drains; `grid_dependency_wait`
// blocks until the predecessor's writes are visible.  Without that launch attribute both
// instructions do nothing.
// `grid_dependency_release` lets the successor's blocks be scheduled (they run their own prologue - barrier
// set-up, weight prefetch - and then block in their own wait until this grid has completed and flushed).
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// Wait first, release afterwards: the successor (and, transitively, everything after it) cannot start before this
// grid's predecessors have all completed.  Kernels that release before they wait let later grids cascade into
// their prologues while much earlier grids are still running, which is harmless for weights but not for data a
// prologue wants to read that an earlier grid of the same replay wrote; one launch of this kind between the
// writer and the readers restores the guarantee.
__device__ __forceinline__ void grid_dependency_wait_then_release() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // release as early as possible, then wait
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a thread block of up to 1024 threads; every thread receives the result.
__device__ __forceinline__ float block_sum(float v, float* scratch32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch32[warp] = v;
  __syncthreads();
  float total = lane < warps ? scratch32[lane] : 0.f;
  return warp_sum(total);
}
__device__ __forceinline__ float block_max(float v, float* scratch32) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch32[warp] = v;
  __syncthreads();
  float total = lane < warps ? scratch32[lane] : -3.0e38f;
  return warp_max(total);
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}
// Round-to-nearest-even, saturating to +-448 (never NaN for finite input).
__device__ __forceinline__ uint8_t float_to_e4m3(float x) { return __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3); }

__device__ __forceinline__ float gelu_tanh(float x) {
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(inner));
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }

__device__ __forceinline__ float apply_activation(float x, unsigned flags) {
  const unsigned act = flags & kFlagActMask;
  if (act == kActGeluTanh) return gelu_tanh(x);
  if (act == kActSilu) return silu(x);
  if (act == kActRelu) return fmaxf(x, 0.f);
  return x;
}

// 8 bf16 values <-> one 16-byte vector
struct alignas(16) Bf16x8 {
  bf162 v[4];
};
__device__ __forceinline__ void unpack8(const Bf16x8& p, float out[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p.v[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ Bf16x8 pack8(const float in[8]) {
  Bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
  return p;
}

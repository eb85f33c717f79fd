// Reference-quality GEMM on CUDA cores: Y[M, N] = epilogue(X[M, K] * W[N, K]^T).
// Shared-memory tiled, fp32 accumulation.  It is the "simt" tactic of the artifact set: a
// plain, easily audited implementation that the recipes can select per GEMM, used to
// cross-check the tcgen05 kernels and as the fallback tactic for shapes those do not cover.
#pragma once

#include "common.cuh"

template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float load_as_float<uint8_t>(const uint8_t* p) { return e4m3_to_float(*p); }

// Shared epilogue: acc -> (scale) -> (+bias) -> activation -> (+residual) -> store.
__device__ __forceinline__ void gemm_store(float acc, unsigned m, unsigned n, void* y, unsigned ldy, const bf16* bias,
                                           const bf16* residual, float alpha, unsigned flags) {
  float r = acc * alpha;
  if (flags & kFlagBias) r += __bfloat162float(bias[n]);
  r = apply_activation(r, flags);
  if (flags & kFlagResidual) r += __bfloat162float(residual[size_t(m) * ldy + n]);
  if (flags & kFlagOutF32) static_cast<float*>(y)[size_t(m) * ldy + n] = r;
  else static_cast<bf16*>(y)[size_t(m) * ldy + n] = __float2bfloat16_rn(r);
}

template <typename TX, typename TW>
__device__ __forceinline__ void gemm_simt_body(const TX* x, const TW* w, void* y, const bf16* bias,
                                               const bf16* residual, const float* scale_a, const float* scale_w,
                                               unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy,
                                               unsigned flags) {
  constexpr int TM = 64, TN = 64, TK = 16;
  __shared__ float xs[TK][TM + 1];
  __shared__ float ws[TK][TN + 1];
  grid_dependency_wait();
  const unsigned tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // 16 x 16 threads, 4 x 4 outputs each
  const unsigned m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
  float acc[4][4] = {};
  for (unsigned k0 = 0; k0 < K; k0 += TK) {
    for (unsigned i = threadIdx.x; i < TM * TK; i += 256) {
      const unsigned r = i / TK, c = i % TK;
      xs[c][r] = (m0 + r < M && k0 + c < K) ? load_as_float<TX>(x + size_t(m0 + r) * ldx + k0 + c) : 0.f;
      ws[c][r] = (n0 + r < N && k0 + c < K) ? load_as_float<TW>(w + size_t(n0 + r) * K + k0 + c) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = xs[kk][ty * 4 + i];
        b[i] = ws[kk][tx * 4 + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
  const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const unsigned m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) gemm_store(acc[i][j], m, n, y, ldy, bias, residual, alpha, flags);
    }
}

// grid = (ceil(N / 64), ceil(M / 64)), block = 256.
extern "C" __global__ void __launch_bounds__(256)
agi_gemm_simt_bf16(const bf16* x, const bf16* w, void* y, const bf16* bias, const bf16* residual,
                   const float* scale_a, const float* scale_w, unsigned M, unsigned N, unsigned K, unsigned ldx,
                   unsigned ldy, unsigned flags) {
  gemm_simt_body<bf16, bf16>(x, w, y, bias, residual, scale_a, scale_w, M, N, K, ldx, ldy, flags);
}
extern "C" __global__ void __launch_bounds__(256)
agi_gemm_simt_e4m3(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias, const bf16* residual,
                   const float* scale_a, const float* scale_w, unsigned M, unsigned N, unsigned K, unsigned ldx,
                   unsigned ldy, unsigned flags) {
  gemm_simt_body<uint8_t, uint8_t>(x, w, y, bias, residual, scale_a, scale_w, M, N, K, ldx, ldy, flags);
}

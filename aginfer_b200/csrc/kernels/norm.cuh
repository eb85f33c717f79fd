// Row normalisations as warp-shuffle reductions: RMSNorm with gain, LayerNorm (no affine)
// with optional AdaLN modulation y = LN(x) * (1 + scale) + shift.
#pragma once

#include "common.cuh"

// One block per row, `cols` a multiple of 8.  y = bf16(x * rsqrt(mean(x^2) + eps) * gain).  With kAmax the
// kernel also folds max |y| (of the rounded outputs) into *amax_bits, which saves the separate pass of the
// dynamic quantisation that follows (rounding is monotonic, so the rounded maximum is the maximum of the
// rounded values).
template <bool kAmax>
__device__ __forceinline__ void rmsnorm_body(const bf16* x, const bf16* gain, bf16* y, unsigned rows, unsigned cols,
                                             unsigned x_stride, unsigned y_stride, float eps, unsigned* amax_bits) {
  __shared__ float scratch[32];
  grid_dependency_wait();
  const unsigned row = blockIdx.x;
  if (row >= rows) return;
  const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + size_t(row) * x_stride);
  const Bf16x8* gr = reinterpret_cast<const Bf16x8*>(gain);
  Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + size_t(row) * y_stride);
  const unsigned vectors = cols / 8;
  float sumsq = 0.f;
  for (unsigned i = threadIdx.x; i < vectors; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) sumsq += f[j] * f[j];
  }
  const float rstd = rsqrtf(block_sum(sumsq, scratch) / float(cols) + eps);
  float best = 0.f;
  for (unsigned i = threadIdx.x; i < vectors; i += blockDim.x) {
    float f[8], g[8];
    unpack8(xr[i], f);
    unpack8(gr[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] = f[j] * rstd * g[j];
      if (kAmax) best = fmaxf(best, fabsf(f[j]));
    }
    yr[i] = pack8(f);
  }
  if (kAmax) {
    __syncthreads();  // scratch is reused
    best = block_max(best, scratch);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(__bfloat162float(__float2bfloat16_rn(best))));
  }
}

extern "C" __global__ void agi_rmsnorm_bf16(const bf16* x, const bf16* gain, bf16* y, unsigned rows, unsigned cols,
                                             unsigned x_stride, unsigned y_stride, float eps) {
  rmsnorm_body<false>(x, gain, y, rows, cols, x_stride, y_stride, eps, nullptr);
}

extern "C" __global__ void agi_rmsnorm_amax_bf16(const bf16* x, const bf16* gain, bf16* y, unsigned rows, unsigned cols,
                                                  unsigned x_stride, unsigned y_stride, float eps, unsigned* amax_bits) {
  rmsnorm_body<true>(x, gain, y, rows, cols, x_stride, y_stride, eps, amax_bits);
}

// One block per row.  y = bf16(((x - mean) * rstd) * (1 + scale[c]) + shift[c]) when
// `modulated` != 0 (scale / shift are bf16 vectors of `cols` entries), else plain LayerNorm
// without affine parameters.  Variance is the biased one, computed as mean((x - mean)^2).
extern "C" __global__ void agi_layernorm_bf16(const bf16* x, const bf16* scale, const bf16* shift, bf16* y,
                                               unsigned rows, unsigned cols, unsigned x_stride, unsigned y_stride,
                                               float eps, unsigned modulated) {
  __shared__ float scratch[32];
  grid_dependency_wait();
  const unsigned row = blockIdx.x;
  if (row >= rows) return;
  const Bf16x8* xr = reinterpret_cast<const Bf16x8*>(x + size_t(row) * x_stride);
  Bf16x8* yr = reinterpret_cast<Bf16x8*>(y + size_t(row) * y_stride);
  const unsigned vectors = cols / 8;
  float sum = 0.f;
  for (unsigned i = threadIdx.x; i < vectors; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) sum += f[j];
  }
  const float mean = block_sum(sum, scratch) / float(cols);
  float var = 0.f;
  for (unsigned i = threadIdx.x; i < vectors; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) var += (f[j] - mean) * (f[j] - mean);
  }
  const float rstd = rsqrtf(block_sum(var, scratch) / float(cols) + eps);
  for (unsigned i = threadIdx.x; i < vectors; i += blockDim.x) {
    float f[8];
    unpack8(xr[i], f);
    if (modulated) {
      float sc[8], sh[8];
      unpack8(reinterpret_cast<const Bf16x8*>(scale)[i], sc);
      unpack8(reinterpret_cast<const Bf16x8*>(shift)[i], sh);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * (1.f + sc[j]) + sh[j];
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd;
    }
    yr[i] = pack8(f);
  }
}

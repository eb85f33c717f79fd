// Small memory-bound kernels: test kernel, arena prologue, amax + E4M3 quantisation,
// SwiGLU, Euler update, type conversion, gathers.
#pragma once

#include "common.cuh"

// Same signature as the reference's only kernel (tests/vector_add.cu:1-7): out = left + right.
extern "C" __global__ void vector_add_f32(const float* left, const float* right, float* out, unsigned count) {
  grid_dependency_wait();
  const unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < count) out[i] = left[i] + right[i];
}

// Recipe prologue: set `count` 32-bit words to `value` (the arena is only zeroed once, at
// session set-up; amax accumulators and status words must restart at zero on every run).
extern "C" __global__ void agi_fill_u32(unsigned* words, unsigned value, unsigned count) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) words[i] = value;
}

// Copy 32-bit words (e.g. the arena's status word into a caller-visible tensor).
extern "C" __global__ void agi_copy_u32(const unsigned* in, unsigned* out, unsigned count) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) out[i] = in[i];
}

// amax_bits = max(amax_bits, bits(max |x|)).  Non-negative floats order like their bit
// patterns, so an integer atomicMax on a zero-initialised word accumulates the maximum.
extern "C" __global__ void agi_absmax_bf16(const bf16* x, unsigned count, unsigned* amax_bits) {
  __shared__ float scratch[32];
  grid_dependency_wait();
  float best = 0.f;
  const unsigned vectors = count / 8;
  const Bf16x8* xv = reinterpret_cast<const Bf16x8*>(x);
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += gridDim.x * blockDim.x) {
    float f[8];
    unpack8(xv[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) best = fmaxf(best, fabsf(f[j]));
  }
  for (unsigned i = vectors * 8 + blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
    best = fmaxf(best, fabsf(__bfloat162float(x[i])));
  best = block_max(best, scratch);
  if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(best));
}

// Per-tensor dynamic quantisation: scale = amax / 448 (1 when amax is 0), q = e4m3(x / scale)
// with IEEE division and round-to-nearest-even, saturating.  Block 0 publishes `scale`.
extern "C" __global__ void agi_quantize_e4m3_bf16(const bf16* x, uint8_t* q, const unsigned* amax_bits,
                                                   float* scale_out, unsigned count) {
  grid_dependency_wait();
  const float amax = __uint_as_float(*amax_bits);
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const unsigned vectors = count / 8;
  const Bf16x8* xv = reinterpret_cast<const Bf16x8*>(x);
  uint2* qv = reinterpret_cast<uint2*>(q);
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < vectors; i += gridDim.x * blockDim.x) {
    float f[8];
    unpack8(xv[i], f);
    unsigned lo = 0, hi = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo |= unsigned(float_to_e4m3(__fdiv_rn(f[j], scale))) << (8 * j);
      hi |= unsigned(float_to_e4m3(__fdiv_rn(f[4 + j], scale))) << (8 * j);
    }
    qv[i] = make_uint2(lo, hi);
  }
  for (unsigned i = vectors * 8 + blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
    q[i] = float_to_e4m3(__fdiv_rn(__bfloat162float(x[i]), scale));
}

// The same quantisation, written in the packed operand layout of the bulk-copy tensor-core GEMM
// ("K-block-major, swizzled"): the 128-byte K block kb of row r goes to ((kb * rows_padded + r) * 128), its
// 16-byte chunk c to position c ^ (r & 7).  One thread converts 16 consecutive values = one chunk.
// cols % 16 == 0; rows past `rows` (up to rows_padded) are left as they are: the GEMM never stores them.
extern "C" __global__ void agi_quantize_e4m3_packed_bf16(const bf16* x, uint8_t* q, const unsigned* amax_bits,
                                                          float* scale_out, unsigned rows, unsigned cols,
                                                          unsigned rows_padded) {
  grid_dependency_wait();
  const float amax = __uint_as_float(*amax_bits);
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.f) : 1.f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = scale;
  const unsigned chunks_per_row = cols / 16;
  const unsigned total = rows * chunks_per_row;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned r = i / chunks_per_row, chunk = i % chunks_per_row;
    const unsigned kb = chunk / 8, c = chunk % 8;
    float f[16];
    unpack8(*reinterpret_cast<const Bf16x8*>(x + size_t(r) * cols + chunk * 16), f);
    unpack8(*reinterpret_cast<const Bf16x8*>(x + size_t(r) * cols + chunk * 16 + 8), f + 8);
    unsigned words[4];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
      unsigned word = 0;
#pragma unroll
      for (int b = 0; b < 4; ++b) word |= unsigned(float_to_e4m3(__fdiv_rn(f[wd * 4 + b], scale))) << (8 * b);
      words[wd] = word;
    }
    uint8_t* dst = q + (size_t(kb) * rows_padded + r) * 128 + ((c ^ (r & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

// out[r, c] = silu(gate[r, c]) * up[r, c]; gate/up may be column blocks of one wider buffer.  With kAmax the
// maximum |out| (of the rounded values) is folded into *amax_bits for the dynamic quantisation that follows.
template <bool kAmax>
__device__ __forceinline__ void swiglu_body(const bf16* gate, const bf16* up, bf16* out, unsigned rows, unsigned cols,
                                            unsigned in_stride, unsigned out_stride, unsigned* amax_bits) {
  __shared__ float scratch[32];
  grid_dependency_wait();
  const unsigned per_row = cols / 8;
  float best = 0.f;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row; i += gridDim.x * blockDim.x) {
    const unsigned r = i / per_row, c = (i % per_row) * 8;
    float g[8], u[8];
    unpack8(*reinterpret_cast<const Bf16x8*>(gate + size_t(r) * in_stride + c), g);
    unpack8(*reinterpret_cast<const Bf16x8*>(up + size_t(r) * in_stride + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      g[j] = silu(g[j]) * u[j];
      if (kAmax) best = fmaxf(best, fabsf(g[j]));
    }
    *reinterpret_cast<Bf16x8*>(out + size_t(r) * out_stride + c) = pack8(g);
  }
  if (kAmax) {
    best = block_max(best, scratch);
    if (threadIdx.x == 0) atomicMax(amax_bits, __float_as_uint(__bfloat162float(__float2bfloat16_rn(best))));
  }
}

extern "C" __global__ void agi_swiglu_bf16(const bf16* gate, const bf16* up, bf16* out, unsigned rows, unsigned cols,
                                            unsigned in_stride, unsigned out_stride) {
  swiglu_body<false>(gate, up, out, rows, cols, in_stride, out_stride, nullptr);
}

extern "C" __global__ void agi_swiglu_amax_bf16(const bf16* gate, const bf16* up, bf16* out, unsigned rows,
                                                 unsigned cols, unsigned in_stride, unsigned out_stride,
                                                 unsigned* amax_bits) {
  swiglu_body<true>(gate, up, out, rows, cols, in_stride, out_stride, amax_bits);
}

// Flow-matching Euler update on the fp32 action latent: x += dt * v (v is the bf16 velocity);
// also refreshes the bf16 copy the next step's encoder reads.
extern "C" __global__ void agi_euler_step(float* x, const bf16* velocity, bf16* x_bf16, float dt, unsigned count) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
    const float next = x[i] + dt * __bfloat162float(velocity[i]);
    x[i] = next;
    x_bf16[i] = __float2bfloat16_rn(next);
  }
}

extern "C" __global__ void agi_bf16_to_f32(const bf16* in, float* out, unsigned count) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}
extern "C" __global__ void agi_f32_to_bf16(const float* in, bf16* out, unsigned count) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}

// Copy `rows` x `cols` bf16 with independent row strides (concatenation, slicing).
extern "C" __global__ void agi_copy_rows_bf16(const bf16* in, bf16* out, unsigned rows, unsigned cols,
                                               unsigned in_stride, unsigned out_stride) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * cols; i += gridDim.x * blockDim.x) {
    const unsigned r = i / cols, c = i % cols;
    out[size_t(r) * out_stride + c] = in[size_t(r) * in_stride + c];
  }
}

// out[r, :] = table[ids[r], :]  (embedding lookup; `cols` a multiple of 8).
extern "C" __global__ void agi_gather_rows_bf16(const bf16* table, const int* ids, bf16* out, unsigned rows,
                                                 unsigned cols, unsigned table_rows, unsigned out_stride) {
  grid_dependency_wait();
  const unsigned per_row = cols / 8;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * per_row; i += gridDim.x * blockDim.x) {
    const unsigned r = i / per_row, c = (i % per_row) * 8;
    unsigned id = static_cast<unsigned>(ids[r]);
    if (id >= table_rows) id = table_rows - 1;  // ids are validated offline; clamp instead of faulting
    *reinterpret_cast<Bf16x8*>(out + size_t(r) * out_stride + c) =
        *reinterpret_cast<const Bf16x8*>(table + size_t(id) * cols + c);
  }
}

// Strided row copy of 32-bit words: out[r, c] = in[r, c] for c < cols (e.g. the first 14 of 32 latent columns).
extern "C" __global__ void agi_copy_rows_u32(const unsigned* in, unsigned* out, unsigned rows, unsigned cols,
                                              unsigned in_stride, unsigned out_stride) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * cols; i += gridDim.x * blockDim.x) {
    const unsigned r = i / cols, c = i % cols;
    out[size_t(r) * out_stride + c] = in[size_t(r) * in_stride + c];
  }
}

// out[r, :] += addend[r % addend_rows, :]  (positional embeddings, broadcast rows).
// Releases its successor only after its own wait: recipes run it once per denoising step, after the per-chunk
// projections and before the blocks, so that a block kernel's prologue may read what those projections wrote.
extern "C" __global__ void agi_add_rows_bf16(bf16* out, const bf16* addend, unsigned rows, unsigned cols,
                                              unsigned out_stride, unsigned addend_rows) {
  grid_dependency_wait_then_release();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * cols; i += gridDim.x * blockDim.x) {
    const unsigned r = i / cols, c = i % cols;
    const float sum = __bfloat162float(out[size_t(r) * out_stride + c]) +
                      __bfloat162float(addend[size_t(r % addend_rows) * cols + c]);
    out[size_t(r) * out_stride + c] = __float2bfloat16_rn(sum);
  }
}

// Sinusoidal embedding of a scalar time: out[r, :] = [cos(t_r * f_i) | sin(t_r * f_i)], i < dim / 2,
// f_i = exp(-ln(10000) * i / (dim / 2)), t_r = t0 + r * dt.  Used for the flow-matching timestep
// (rows = denoising steps) and for the action encoder (rows = action tokens, dt = 0).
extern "C" __global__ void agi_timestep_embedding(bf16* out, unsigned rows, unsigned dim, unsigned out_stride,
                                                   float t0, float dt) {
  grid_dependency_wait();
  const unsigned half = dim / 2;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < rows * half; i += gridDim.x * blockDim.x) {
    const unsigned r = i / half, k = i % half;
    const float freq = expf(-9.210340371976184f * float(k) / float(half));
    float s, c;
    sincosf((t0 + float(r) * dt) * freq, &s, &c);
    out[size_t(r) * out_stride + k] = __float2bfloat16_rn(c);
    out[size_t(r) * out_stride + half + k] = __float2bfloat16_rn(s);
  }
}

// Elementwise SiLU on bf16 (conditioning vector before the AdaLN projections).
extern "C" __global__ void agi_silu_bf16(const bf16* in, bf16* out, unsigned count) {
  grid_dependency_wait();
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
    out[i] = __float2bfloat16_rn(silu(__bfloat162float(in[i])));
}

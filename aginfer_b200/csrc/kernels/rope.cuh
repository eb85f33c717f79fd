// Rotary position embedding, applied in place to the first `heads` heads of every row
// (Q and K sit side by side in the fused QKV buffer, V is left alone).
#pragma once

#include "common.cuh"

// Half-split ("rotate_half") convention: element i pairs with i + head_dim/2,
//   out[i]       = x[i] * cos(a_i) - x[i + h] * sin(a_i)
//   out[i + h]   = x[i + h] * cos(a_i) + x[i] * sin(a_i),   a_i = pos * theta^(-2 i / head_dim).
// 1-D positions: pos = row + pos_offset.
extern "C" __global__ void agi_rope_bf16(bf16* x, unsigned rows, unsigned heads, unsigned head_dim,
                                          unsigned row_stride, float log2_theta, unsigned pos_offset) {
  grid_dependency_wait();
  const unsigned half = head_dim / 2;
  const unsigned total = rows * heads * half;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned pair = i % half, head = (i / half) % heads, row = i / (half * heads);
    const float inv_freq = exp2f(-log2_theta * (2.f * float(pair) / float(head_dim)));
    float s, c;
    sincosf(float(row + pos_offset) * inv_freq, &s, &c);
    bf16* p = x + size_t(row) * row_stride + head * head_dim + pair;
    const float a = __bfloat162float(p[0]), b = __bfloat162float(p[half]);
    p[0] = __float2bfloat16_rn(a * c - b * s);
    p[half] = __float2bfloat16_rn(b * c + a * s);
  }
}

// The same over two tensors in one launch (queries and the new keys of a decode step live in different buffers):
// heads [0, heads0) are x0's, heads [heads0, heads0 + heads1) are x1's.
extern "C" __global__ void agi_rope_pair_bf16(bf16* x0, unsigned heads0, unsigned row_stride0, bf16* x1, unsigned heads1,
                                               unsigned row_stride1, unsigned rows, unsigned head_dim, float log2_theta,
                                               unsigned pos_offset) {
  grid_dependency_wait();
  const unsigned half = head_dim / 2, heads = heads0 + heads1;
  const unsigned total = rows * heads * half;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned pair = i % half, head = (i / half) % heads, row = i / (half * heads);
    const float inv_freq = exp2f(-log2_theta * (2.f * float(pair) / float(head_dim)));
    float s, c;
    sincosf(float(row + pos_offset) * inv_freq, &s, &c);
    bf16* p = head < heads0 ? x0 + size_t(row) * row_stride0 + head * head_dim + pair
                            : x1 + size_t(row) * row_stride1 + (head - heads0) * head_dim + pair;
    const float a = __bfloat162float(p[0]), b = __bfloat162float(p[half]);
    p[0] = __float2bfloat16_rn(a * c - b * s);
    p[half] = __float2bfloat16_rn(b * c + a * s);
  }
}

// Multimodal RoPE: three position streams (temporal, height, width) given as int32
// pos[3][rows]; rotary pair i takes its position from stream 0 for i < s0, stream 1 for
// i < s0 + s1, else stream 2 (sections (16, 24, 24) for head_dim 128).  `ladder` = rotary pairs per frequency
// ladder: pair i turns at theta^(-(i mod ladder) / ladder).  head_dim / 2 gives the one ladder of a language
// model; the vision tower's 2-D rotary uses head_dim / 4: one ladder for the rows, the same one again for the
// columns.
extern "C" __global__ void agi_mrope_bf16(bf16* x, const int* pos, unsigned rows, unsigned heads, unsigned head_dim,
                                           unsigned row_stride, float log2_theta, unsigned s0, unsigned s1,
                                           unsigned ladder) {
  grid_dependency_wait();
  const unsigned half = head_dim / 2;
  const unsigned total = rows * heads * half;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned pair = i % half, head = (i / half) % heads, row = i / (half * heads);
    const unsigned stream = pair < s0 ? 0u : (pair < s0 + s1 ? 1u : 2u);
    const float inv_freq = exp2f(-log2_theta * (float(pair % ladder) / float(ladder)));
    float s, c;
    sincosf(float(pos[stream * rows + row]) * inv_freq, &s, &c);
    bf16* p = x + size_t(row) * row_stride + head * head_dim + pair;
    const float a = __bfloat162float(p[0]), b = __bfloat162float(p[half]);
    p[0] = __float2bfloat16_rn(a * c - b * s);
    p[half] = __float2bfloat16_rn(b * c + a * s);
  }
}

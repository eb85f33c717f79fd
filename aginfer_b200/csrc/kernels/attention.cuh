// Softmax attention for the small sequence lengths of this workload (17 ... 768 rows):
// one warp per query row, 8 rows of one head per block, keys/values staged through shared
// memory 32 at a time, fp32 online softmax.  Covers GQA causal (decoder), block-diagonal
// (vision windows / per-image full attention), plain self attention and cross attention.
#pragma once

#include "common.cuh"

constexpr int kAttnWarps = 8;
constexpr int kAttnChunk = 32;
constexpr int kAttnMaxDim = 128;

// q: [q_rows, *] with head h at column h * head_dim, row stride q_stride (elements);
// k, v: [kv_rows, *] with kv head g at column g * head_dim, row strides k_stride / v_stride;
// o: [q_rows, q_heads * head_dim], row stride o_stride.  Query head h reads kv head
// h / (q_heads / kv_heads).  mask_mode: 0 = none, 1 = causal (key j visible to query i when
// j <= i + causal_shift), 2 = block diagonal (key j visible when j / block == i / block).
// grid = (ceil(q_rows / 8), q_heads), block = 256 threads; head_dim <= 128, multiple of 2.
extern "C" __global__ void __launch_bounds__(kAttnWarps * 32)
agi_attention_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows,
                   unsigned q_heads, unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride,
                   unsigned v_stride, unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg) {
  __shared__ __align__(16) bf16 k_tile[kAttnChunk][kAttnMaxDim + 2];  // +2: odd word stride, conflict-free rows
  __shared__ __align__(16) bf16 v_tile[kAttnChunk][kAttnMaxDim];
  __shared__ float q_tile[kAttnWarps][kAttnMaxDim];
  grid_dependency_wait();

  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned head = blockIdx.y, kv_head = head / (q_heads / kv_heads);
  const unsigned row = blockIdx.x * kAttnWarps + warp;
  const bool live = row < q_rows;
  const unsigned dims_per_lane = (head_dim + 31) / 32;  // <= 4

  for (unsigned d = lane; d < head_dim; d += 32)
    q_tile[warp][d] = live ? __bfloat162float(q[size_t(row) * q_stride + head * head_dim + d]) * scale : 0.f;

  // Range of keys any row of this block can see (skips whole chunks outside it).
  const unsigned first_row = blockIdx.x * kAttnWarps;
  const unsigned last_row = min(first_row + kAttnWarps, q_rows) - 1;
  unsigned key_begin = 0, key_end = kv_rows;
  if (mask_mode == 1) key_end = min(kv_rows, last_row + mask_arg + 1);
  if (mask_mode == 2) {
    key_begin = (first_row / mask_arg) * mask_arg;
    key_end = min(kv_rows, (last_row / mask_arg + 1) * mask_arg);
  }

  float running_max = -3.0e38f, running_sum = 0.f;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (unsigned base = key_begin - key_begin % kAttnChunk; base < key_end; base += kAttnChunk) {
    __syncthreads();  // previous tile fully consumed (and q_tile written, first time round)
    for (unsigned i = threadIdx.x; i < kAttnChunk * (head_dim / 2); i += blockDim.x) {
      const unsigned j = i / (head_dim / 2), d = (i % (head_dim / 2)) * 2;
      const unsigned key = base + j;
      bf162 kk = __floats2bfloat162_rn(0.f, 0.f), vv = kk;
      if (key < kv_rows) {
        kk = *reinterpret_cast<const bf162*>(k + size_t(key) * k_stride + kv_head * head_dim + d);
        vv = *reinterpret_cast<const bf162*>(v + size_t(key) * v_stride + kv_head * head_dim + d);
      }
      *reinterpret_cast<bf162*>(&k_tile[j][d]) = kk;
      *reinterpret_cast<bf162*>(&v_tile[j][d]) = vv;
    }
    __syncthreads();
    if (!live) continue;

    // Lane j scores key base + j.
    const unsigned key = base + lane;
    bool visible = key < kv_rows;
    if (mask_mode == 1) visible = visible && key <= row + mask_arg;
    if (mask_mode == 2) visible = visible && key / mask_arg == row / mask_arg;
    float score = 0.f;
    for (unsigned d = 0; d < head_dim; d += 2) {
      const float2 kk = __bfloat1622float2(*reinterpret_cast<const bf162*>(&k_tile[lane][d]));
      score += q_tile[warp][d] * kk.x + q_tile[warp][d + 1] * kk.y;
    }
    score = visible ? score : -3.0e38f;
    const float chunk_max = warp_max(score);
    if (chunk_max <= -3.0e38f) continue;  // nothing visible in this chunk
    const float new_max = fmaxf(running_max, chunk_max);
    const float rescale = __expf(running_max - new_max);
    const float p = visible ? __expf(score - new_max) : 0.f;
    running_sum = running_sum * rescale + warp_sum(p);
    running_max = new_max;
#pragma unroll
    for (int t = 0; t < 4; ++t) acc[t] *= rescale;
    for (int j = 0; j < kAttnChunk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const unsigned d = lane + 32 * t;
        if (t < dims_per_lane && d < head_dim) acc[t] += pj * __bfloat162float(v_tile[j][d]);
      }
    }
  }
  if (!live) return;
  const float inv = running_sum > 0.f ? 1.f / running_sum : 0.f;
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const unsigned d = lane + 32 * t;
    if (t < dims_per_lane && d < head_dim) o[size_t(row) * o_stride + head * head_dim + d] = __float2bfloat16_rn(acc[t] * inv);
  }
}

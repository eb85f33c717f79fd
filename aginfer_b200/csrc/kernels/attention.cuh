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
  AGI_TRACE_KERNEL(4);
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

// Same contract as agi_attention_bf16, for the case where every key a block of 8 query rows can see
// fits in shared memory (the action head: 17 or 300 keys; a 288-token decoder layer; one vision
// window).  All visible K and V rows of the head are fetched with one round of independent 16-byte
// loads, then each warp handles one query row without further block-wide synchronisation:
// scores for all keys (lane j takes keys j, j + 32, ...), one max and one sum reduction, then P.V.
// grid = (ceil(q_rows / 8), q_heads), block = 256,
// dynamic shared memory = span * ((head_dim + 2) + head_dim) * 2 + 16 + 8 * head_dim * 4 + 8 * span_pad * 4,
// span = number of visible keys for a block of rows (all kv_rows for mask 0/1), span_pad = span rounded
// up to 32.  head_dim a multiple of 8, <= 128.
extern "C" __global__ void __launch_bounds__(kAttnWarps * 32)
agi_attention_smem_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows,
                        unsigned q_heads, unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride,
                        unsigned v_stride, unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg,
                        unsigned span_max) {
  AGI_TRACE_KERNEL(3);
  extern __shared__ __align__(16) unsigned char attn_smem[];
  grid_dependency_wait();
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned head = blockIdx.y, kv_head = head / (q_heads / kv_heads);
  const unsigned first_row = blockIdx.x * kAttnWarps;
  const unsigned last_row = min(first_row + kAttnWarps, q_rows) - 1;
  unsigned key_begin = 0, key_end = kv_rows;
  if (mask_mode == 1) key_end = min(kv_rows, last_row + mask_arg + 1);
  if (mask_mode == 2) {
    key_begin = (first_row / mask_arg) * mask_arg;
    key_end = min(kv_rows, (last_row / mask_arg + 1) * mask_arg);
  }
  const unsigned span = min(key_end - key_begin, span_max);
  const unsigned span_pad = (span_max + 31) & ~31u;
  const unsigned k_pitch = head_dim + 2;  // elements; odd word count -> conflict-free row-per-lane reads
  bf16* k_tile = reinterpret_cast<bf16*>(attn_smem);
  bf16* v_tile = k_tile + ((size_t(span_max) * k_pitch + 7) & ~size_t(7));  // keep V rows 16-byte aligned
  float* q_tile = reinterpret_cast<float*>(v_tile + size_t(span_max) * head_dim);
  float* p_tile = q_tile + kAttnWarps * head_dim;

  // Batches of independent 16-byte loads (8 elements of K and of V each), all issued before any is
  // stored, so a batch costs one memory round trip.
  const unsigned vec_per_row = head_dim / 8;
  const unsigned vectors = span * vec_per_row;
  constexpr int kBatch = 4;
  for (unsigned i0 = threadIdx.x; i0 < vectors; i0 += kBatch * blockDim.x) {
    uint4 kk[kBatch], vv[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const unsigned i = i0 + b * blockDim.x;
      if (i < vectors) {
        const unsigned j = i / vec_per_row, d = (i % vec_per_row) * 8;
        const size_t key = key_begin + j;
        kk[b] = __ldg(reinterpret_cast<const uint4*>(k + key * k_stride + kv_head * head_dim + d));
        vv[b] = __ldg(reinterpret_cast<const uint4*>(v + key * v_stride + kv_head * head_dim + d));
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const unsigned i = i0 + b * blockDim.x;
      if (i < vectors) {
        const unsigned j = i / vec_per_row, d = (i % vec_per_row) * 8;
        unsigned* kd = reinterpret_cast<unsigned*>(&k_tile[j * k_pitch + d]);  // 4-byte aligned (pitch is even)
        kd[0] = kk[b].x; kd[1] = kk[b].y; kd[2] = kk[b].z; kd[3] = kk[b].w;
        *reinterpret_cast<uint4*>(&v_tile[j * head_dim + d]) = vv[b];
      }
    }
  }
  const unsigned row = first_row + warp;
  const bool live = row < q_rows;
  for (unsigned d = lane; d < head_dim; d += 32)
    q_tile[warp * head_dim + d] = live ? __bfloat162float(q[size_t(row) * q_stride + head * head_dim + d]) * scale : 0.f;
  __syncthreads();
  if (!live) return;

  float* p = p_tile + warp * span_pad;
  const float* qr = q_tile + warp * head_dim;
  float best = -3.0e38f;
  // Scores: 8 keys per lane per pass (keys lane, lane + 32, ...), the query pair read once per pass.
  for (unsigned j0 = 0; j0 < span; j0 += 256) {
    float score[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) score[i] = 0.f;
    const unsigned groups = min(8u, (span - j0 + 31) / 32);  // 32-key groups that exist in this pass
    for (unsigned d = 0; d < head_dim; d += 2) {
      const float2 qq = *reinterpret_cast<const float2*>(qr + d);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i >= groups) break;
        const unsigned j = min(j0 + lane + 32 * i, span - 1);  // clamped lanes recompute the last key; dropped below
        const float2 kk = __bfloat1622float2(*reinterpret_cast<const bf162*>(k_tile + j * k_pitch + d));
        score[i] += qq.x * kk.x + qq.y * kk.y;
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const unsigned j = j0 + lane + 32 * i;
      if (j >= span) continue;
      const unsigned key = key_begin + j;
      bool visible = true;
      if (mask_mode == 1) visible = key <= row + mask_arg;
      if (mask_mode == 2) visible = key / mask_arg == row / mask_arg;
      const float sc = visible ? score[i] : -3.0e38f;
      p[j] = sc;
      best = fmaxf(best, sc);
    }
  }
  best = warp_max(best);
  float sum = 0.f;
  for (unsigned j = lane; j < span; j += 32) {
    const float sc = p[j];
    const float e = sc > -1.0e38f ? __expf(sc - best) : 0.f;
    p[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  __syncwarp();
  const float inv = sum > 0.f ? 1.f / sum : 0.f;
  // P.V: a lane owns two adjacent output dimensions; four keys per step on independent accumulators.
  for (unsigned d = 2 * lane; d < head_dim; d += 64) {
    float2 acc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) acc[u] = make_float2(0.f, 0.f);
    unsigned j = 0;
    for (; j + 4 <= span; j += 4) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float pj = p[j + u];
        const float2 vv = __bfloat1622float2(*reinterpret_cast<const bf162*>(v_tile + (j + u) * head_dim + d));
        acc[u].x += pj * vv.x;
        acc[u].y += pj * vv.y;
      }
    }
    for (; j < span; ++j) {
      const float pj = p[j];
      const float2 vv = __bfloat1622float2(*reinterpret_cast<const bf162*>(v_tile + j * head_dim + d));
      acc[0].x += pj * vv.x;
      acc[0].y += pj * vv.y;
    }
    const float ox = (acc[0].x + acc[1].x) + (acc[2].x + acc[3].x), oy = (acc[0].y + acc[1].y) + (acc[2].y + acc[3].y);
    *reinterpret_cast<bf162*>(o + size_t(row) * o_stride + head * head_dim + d) = __floats2bfloat162_rn(ox * inv, oy * inv);
  }
}

// Softmax attention for the small sequence lengths of this workload (17 ... 768 rows):
// one warp per query row, 8 rows of one head per block, keys/values staged through shared
// memory 32 at a time, fp32 online softmax.  Covers GQA causal (decoder), block-diagonal
// (vision windows / per-image full attention), plain self attention and cross attention.
#pragma once

#include "common.cuh"

// m16n8k16 bf16 MMA with fp32 accumulation (D = A.B + D).
__device__ __forceinline__ void skinny_mma_bf16(float c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                                unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

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

// Attention for a handful of query rows (the action head: 17 queries against 17 or 300 keys).  One block
// per head.  The head's K and V rows are fetched once; the 8 warps split the KEYS (flash-decoding style),
// each computing scores, a local softmax and a partial P.V for all query rows over its own key range; the
// partial results are merged through shared memory with the usual max/sum rescaling.  Latency, not
// throughput, decides this kernel: every phase is a short loop over registers and shared memory.
// grid = (q_heads), block = 256; q_rows <= 32, head_dim <= 64 and a multiple of 8.
// dynamic shared memory: see attention_rows_smem_bytes in the recipe builder.
constexpr int kRowsMax = 32;

extern "C" __global__ void __launch_bounds__(kAttnWarps * 32)
agi_attention_rows_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows,
                        unsigned q_heads, unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride,
                        unsigned v_stride, unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  grid_dependency_wait();
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned head = blockIdx.x, kv_head = head / (q_heads / kv_heads);
  const unsigned k_pitch = head_dim + 2, kv_pad = (kv_rows + 31) & ~31u;
  bf16* k_tile = reinterpret_cast<bf16*>(attn_smem);
  bf16* v_tile = k_tile + ((size_t(kv_rows) * k_pitch + 7) & ~size_t(7));
  float* q_tile = reinterpret_cast<float*>(v_tile + size_t(kv_rows) * head_dim);   // [rows][head_dim]
  float* p_tile = q_tile + q_rows * head_dim;                                       // [rows][kv_pad]
  float* o_part = p_tile + q_rows * kv_pad;                                         // [warps][rows][head_dim]
  float* m_part = o_part + kAttnWarps * q_rows * head_dim;                          // [warps][rows]
  float* l_part = m_part + kAttnWarps * q_rows;

  // ---- stage K, V (batches of independent 16-byte loads) and Q (pre-scaled) ----
  const unsigned vec_per_row = head_dim / 8, vectors = kv_rows * vec_per_row;
  constexpr int kBatch = 4;
  for (unsigned i0 = threadIdx.x; i0 < vectors; i0 += kBatch * blockDim.x) {
    uint4 kk[kBatch], vv[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const unsigned i = i0 + b * blockDim.x;
      if (i < vectors) {
        const size_t key = i / vec_per_row;
        const unsigned d = (i % vec_per_row) * 8;
        kk[b] = __ldg(reinterpret_cast<const uint4*>(k + key * k_stride + kv_head * head_dim + d));
        vv[b] = __ldg(reinterpret_cast<const uint4*>(v + key * v_stride + kv_head * head_dim + d));
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const unsigned i = i0 + b * blockDim.x;
      if (i < vectors) {
        const unsigned j = i / vec_per_row, d = (i % vec_per_row) * 8;
        unsigned* kd = reinterpret_cast<unsigned*>(&k_tile[j * k_pitch + d]);
        kd[0] = kk[b].x; kd[1] = kk[b].y; kd[2] = kk[b].z; kd[3] = kk[b].w;
        *reinterpret_cast<uint4*>(&v_tile[j * head_dim + d]) = vv[b];
      }
    }
  }
  for (unsigned i = threadIdx.x; i < q_rows * head_dim; i += blockDim.x) {
    const unsigned r = i / head_dim, d = i % head_dim;
    q_tile[i] = __bfloat162float(q[size_t(r) * q_stride + head * head_dim + d]) * scale;
  }
  __syncthreads();

  // ---- this warp's key range ----
  const unsigned per_warp = (kv_rows + kAttnWarps - 1) / kAttnWarps;
  const unsigned key_lo = min(warp * per_warp, kv_rows), key_hi = min(key_lo + per_warp, kv_rows);

  // scores: a lane keeps one key row in registers and visits every query row
  for (unsigned key = key_lo + lane; key < key_hi; key += 32) {
    bf162 kr[32];  // head_dim / 2 <= 32 pairs
#pragma unroll
    for (int d2 = 0; d2 < 32; ++d2)
      if (2 * d2 < head_dim) kr[d2] = *reinterpret_cast<const bf162*>(k_tile + key * k_pitch + 2 * d2);
    for (unsigned r = 0; r < q_rows; ++r) {
      const float2* qr = reinterpret_cast<const float2*>(q_tile + r * head_dim);
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int d2 = 0; d2 < 32; ++d2)
        if (2 * d2 < head_dim) {
          const float2 kk = __bfloat1622float2(kr[d2]);
          const float2 qq = qr[d2];
          s0 += qq.x * kk.x;
          s1 += qq.y * kk.y;
        }
      bool visible = true;
      if (mask_mode == 1) visible = key <= r + mask_arg;
      if (mask_mode == 2) visible = key / mask_arg == r / mask_arg;
      p_tile[r * kv_pad + key] = visible ? s0 + s1 : -3.0e38f;
    }
  }
  __syncwarp();
  // local softmax over this warp's keys, row by row
  for (unsigned r = 0; r < q_rows; ++r) {
    float best = -3.0e38f;
    for (unsigned key = key_lo + lane; key < key_hi; key += 32) best = fmaxf(best, p_tile[r * kv_pad + key]);
    best = warp_max(best);
    float sum = 0.f;
    for (unsigned key = key_lo + lane; key < key_hi; key += 32) {
      const float s = p_tile[r * kv_pad + key];
      const float e = s > -1.0e38f ? __expf(s - best) : 0.f;
      p_tile[r * kv_pad + key] = e;
      sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) {
      m_part[warp * q_rows + r] = best;
      l_part[warp * q_rows + r] = sum;
    }
  }
  __syncwarp();
  // partial P.V: a lane owns one pair of output dimensions for every query row
  if (2 * lane < head_dim) {
    float2 acc[kRowsMax];
#pragma unroll
    for (int r = 0; r < kRowsMax; ++r) acc[r] = make_float2(0.f, 0.f);
    for (unsigned key = key_lo; key < key_hi; ++key) {
      const float2 vv = __bfloat1622float2(*reinterpret_cast<const bf162*>(v_tile + key * head_dim + 2 * lane));
#pragma unroll
      for (int r = 0; r < kRowsMax; ++r)
        if (r < q_rows) {
          const float pj = p_tile[r * kv_pad + key];
          acc[r].x += pj * vv.x;
          acc[r].y += pj * vv.y;
        }
    }
#pragma unroll
    for (int r = 0; r < kRowsMax; ++r)
      if (r < q_rows) *reinterpret_cast<float2*>(o_part + (warp * q_rows + r) * head_dim + 2 * lane) = acc[r];
  }
  __syncthreads();
  // merge the 8 partial results
  for (unsigned i = threadIdx.x; i < q_rows * head_dim; i += blockDim.x) {
    const unsigned r = i / head_dim, d = i % head_dim;
    float best = -3.0e38f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) best = fmaxf(best, m_part[w * q_rows + r]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float mw = m_part[w * q_rows + r];
      const float f = mw > -1.0e38f ? __expf(mw - best) : 0.f;
      num += f * o_part[(w * q_rows + r) * head_dim + d];
      den += f * l_part[w * q_rows + r];
    }
    o[size_t(r) * o_stride + head * head_dim + d] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
  }
}

// Tensor-core attention for a handful of query rows (the action head: 17 queries, 17 or 300 keys,
// head_dim 48).  One block of 8 warps per (head, 16-row tile of queries).  K and V are staged row-major in shared memory (K rows are the
// "B" operand of Q.K^T as they are, V goes through ldmatrix.trans for P.V); Q stays in registers as the "A" operand.  Each warp
// takes every eighth 16-key block, three blocks at a time (their score MMAs are independent: one rescale of the running
// max / sum per group instead of per block), P re-used directly as the A operand of P.V; the eight warps'
// (max, sum, O) are merged through shared memory at the end.  With at most 32 keys the warps split the value
// columns instead of the keys and nothing is merged.  About 25 MMAs per 16 keys instead of
// thousands of scalar instructions: the kernel is latency-bound, so instruction count is what matters.
// grid = (q_heads, ceil(q_rows / 16)), block = 256; head_dim a multiple of 16, <= 64 (agi_attention_mma_bf16_d128: <= 128).
// dynamic shared memory = 2 * kv16 * (head_dim + 8) * 2 (K and V) + merge area 8 * 16 * (head_dim + 2) * 4,
// kv16 = kv_rows rounded up to 16.
template <int kKsteps, int kDtiles, bool kAliasMerge>
__device__ __forceinline__ void attention_mma_body(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows,
                                                   unsigned kv_rows, unsigned q_heads, unsigned kv_heads, unsigned head_dim,
                                                   unsigned q_stride, unsigned k_stride, unsigned v_stride, unsigned o_stride,
                                                   float scale, unsigned mask_mode, unsigned mask_arg) {
  extern __shared__ __align__(16) unsigned char attn_smem[];
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned head = blockIdx.x, kv_head = head / (q_heads / kv_heads);
  const unsigned row_base = blockIdx.y * 16;   // this block's query rows
  const unsigned kv16 = (kv_rows + 15) & ~15u;
  // K and V both row-major with a pitch of head_dim + 8 elements: rows stay 16-byte aligned (cp.async,
  // ldmatrix) and the eight rows a fragment touches fall into different banks.
  const unsigned pitch = head_dim + 8;
  bf16* k_tile = reinterpret_cast<bf16*>(attn_smem);               // [kv16][pitch]
  bf16* v_tile = k_tile + size_t(kv16) * pitch;                    // [kv16][pitch]
  // the merge area follows the tiles, or (kAliasMerge: wide heads, where both would not fit) re-uses their space
  // once every warp is done with keys and values
  float* merge = kAliasMerge ? reinterpret_cast<float*>(attn_smem) : reinterpret_cast<float*>(v_tile + size_t(kv16) * pitch);

  // Keys and values that were written long before the previous kernel (cross-attention over context tokens
  // projected once per chunk, the prefix of a KV cache; bit 8 of mask_mode, bits 16-31 = how many leading rows,
  // 0 = all) are requested BEFORE the grid-dependency wait, like weights; the rest after it.
  const bool early_kv = (mask_mode & 0x100u) != 0;
  const unsigned static_rows = !early_kv ? 0u : ((mask_mode >> 16) != 0 ? min(mask_mode >> 16, kv_rows) : kv16);
  mask_mode &= 0xffu;
  // ---- stage K and V with 16-byte asynchronous copies, all in flight at once; rows past kv_rows are zero-filled.
  // Thread t moves 16-byte vector t % kDtiles of rows t / kDtiles, t / kDtiles + 256 / kDtiles, ...
  const unsigned vec_per_row = head_dim / 8;
  auto stage = [&](unsigned first, unsigned last) {
    if ((threadIdx.x % kDtiles) >= vec_per_row) return;
    const unsigned d = (threadIdx.x % kDtiles) * 8;
    for (unsigned j = first + threadIdx.x / kDtiles; j < last; j += blockDim.x / kDtiles) {
      const unsigned src_row = min(j, kv_rows - 1), bytes = j < kv_rows ? 16u : 0u;
      const unsigned kd = static_cast<unsigned>(__cvta_generic_to_shared(k_tile + j * pitch + d));
      const unsigned vd = static_cast<unsigned>(__cvta_generic_to_shared(v_tile + j * pitch + d));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd),
                   "l"(k + size_t(src_row) * k_stride + kv_head * head_dim + d), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd),
                   "l"(v + size_t(src_row) * v_stride + kv_head * head_dim + d), "r"(bytes) : "memory");
    }
  };
  stage(0, static_rows);
  grid_dependency_wait();
  stage(static_rows, kv16);
  asm volatile("cp.async.commit_group;" ::: "memory");
  // ---- Q fragments (A operand), pre-scaled: rows g, g + 8 of each 16-row tile; zero past q_rows ----
  const unsigned ksteps = head_dim / 16;   // <= kKsteps
  unsigned qa[1][kKsteps][4];
#pragma unroll
  for (int mt = 0; mt < 1; ++mt)
#pragma unroll
    for (int ks = 0; ks < kKsteps; ++ks)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        qa[mt][ks][r] = 0;
        const unsigned row = row_base + g + (r & 1) * 8, col = ks * 16 + 2 * t + (r >> 1) * 8;
        if (ks < ksteps && row < q_rows) {
          const bf162 pair = *reinterpret_cast<const bf162*>(q + size_t(row) * q_stride + head * head_dim + col);
          const float2 f = __bfloat1622float2(pair);
          const bf162 scaled = __floats2bfloat162_rn(f.x * scale, f.y * scale);
          qa[mt][ks][r] = *reinterpret_cast<const unsigned*>(&scaled);
        }
      }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();

  // running softmax state of this thread's rows g, g + 8 and its output accumulators (8 dims per tile)
  float row_max[2], row_sum[2], out[kDtiles][4];
  row_max[0] = row_max[1] = -3.0e38f;
  row_sum[0] = row_sum[1] = 0.f;
#pragma unroll
  for (int nt = 0; nt < kDtiles; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) out[nt][i] = 0.f;
  const unsigned dtiles = head_dim / 8;    // <= kDtiles
  // Few keys (at most two 16-key blocks, e.g. self-attention over 17 tokens): splitting the keys over warps would
  // leave six warps idle and still pay the merge.  Instead every warp w < dtiles scores ALL keys (the same few
  // MMAs in each warp) and multiplies P with the 8 value columns of ITS tile only: no merge, no second barrier,
  // the warp stores its slice of the output straight from its accumulators.
  const bool by_dims = kv16 <= 32 && dtiles <= 8;   // eight warps: one value tile each
  if (by_dims && warp >= dtiles) return;
  const unsigned first_key = by_dims ? 0u : warp * 16u, key_step = by_dims ? 16u : 128u;
  constexpr int kGroup = 3;   // 16-key blocks scored together: their MMAs are independent, one rescale per group

  for (unsigned base = first_key; base < kv16; base += key_step * kGroup) {
    float s[kGroup][2][4];
#pragma unroll
    for (int b = 0; b < kGroup; ++b) {
      const unsigned key0 = base + b * key_step;
#pragma unroll
      for (int half = 0; half < 2; ++half) s[b][half][0] = s[b][half][1] = s[b][half][2] = s[b][half][3] = -3.0e38f;
      if (key0 >= kv16) continue;
      // B fragments of K for the two 8-key tiles: b0 = (d 2t..2t+1, key g), b1 = (d 2t+8.., key g)
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        s[b][half][0] = s[b][half][1] = s[b][half][2] = s[b][half][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < kKsteps; ++ks)
          if (ks < ksteps) {
            const bf16* row = k_tile + (key0 + half * 8 + g) * pitch + ks * 16 + 2 * t;
            skinny_mma_bf16(s[b][half], qa[0][ks][0], qa[0][ks][1], qa[0][ks][2], qa[0][ks][3],
                            *reinterpret_cast<const unsigned*>(row), *reinterpret_cast<const unsigned*>(row + 8));
          }
      }
      // mask
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned key = key0 + half * 8 + 2 * t + (i & 1), row = row_base + g + (i >> 1) * 8;
          bool visible = key < kv_rows;
          if (mask_mode == 1) visible = visible && key <= row + mask_arg;
          if (mask_mode == 2) visible = visible && key / mask_arg == row / mask_arg;
          if (!visible) s[b][half][i] = -3.0e38f;
        }
    }
    // per-row maximum over the group's keys (own values, then across the quad), one rescale of the running state
    unsigned pa[kGroup][4];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {  // hr 0: row g (c0, c1), hr 1: row g + 8 (c2, c3)
      float group_max = -3.0e38f;
#pragma unroll
      for (int b = 0; b < kGroup; ++b)
        group_max = fmaxf(group_max, fmaxf(fmaxf(s[b][0][2 * hr], s[b][0][2 * hr + 1]), fmaxf(s[b][1][2 * hr], s[b][1][2 * hr + 1])));
      group_max = fmaxf(group_max, __shfl_xor_sync(0xffffffffu, group_max, 1));
      group_max = fmaxf(group_max, __shfl_xor_sync(0xffffffffu, group_max, 2));
      const float new_max = fmaxf(row_max[hr], group_max);
      const float rescale = new_max > -1.0e38f ? __expf(row_max[hr] - new_max) : 1.f;
      float group_sum = 0.f;
#pragma unroll
      for (int b = 0; b < kGroup; ++b) {
        float p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float sc = s[b][j >> 1][2 * hr + (j & 1)];
          p[j] = sc > -1.0e38f ? __expf(sc - new_max) : 0.f;
        }
        group_sum += (p[0] + p[1]) + (p[2] + p[3]);
        // P as the A operand of P.V: a0/a1 = keys 2t..2t+1 (first tile), a2/a3 = keys 2t+8.. (second tile)
        const bf162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
        pa[b][hr] = *reinterpret_cast<const unsigned*>(&lo);
        pa[b][2 + hr] = *reinterpret_cast<const unsigned*>(&hi);
      }
      group_sum += __shfl_xor_sync(0xffffffffu, group_sum, 1);
      group_sum += __shfl_xor_sync(0xffffffffu, group_sum, 2);
      row_sum[hr] = row_sum[hr] * rescale + group_sum;
      row_max[hr] = new_max;
#pragma unroll
      for (int nt = 0; nt < kDtiles; ++nt) {
        out[nt][2 * hr] *= rescale;
        out[nt][2 * hr + 1] *= rescale;
      }
    }
    // O += P (16 x 16 keys) . V (16 keys x 8 dims) per 8-dim tile.  ldmatrix with transpose turns two
    // 8 x 8 blocks of row-major V (keys 0-7 and 8-15 of a block) into the B fragment (key pair, dim g).
#pragma unroll
    for (int b = 0; b < kGroup; ++b) {
      const unsigned key0 = base + b * key_step;
      if (key0 >= kv16) continue;
#pragma unroll
      for (int nt = 0; nt < kDtiles; ++nt)
        if (nt < dtiles && (!by_dims || nt == int(warp))) {
          const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(v_tile + (key0 + (lane & 15)) * pitch + nt * 8));
          unsigned b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
          skinny_mma_bf16(out[nt], pa[b][0], pa[b][1], pa[b][2], pa[b][3], b0, b1);
        }
    }
  }

  if (by_dims) {
    // this warp's 8 output columns of rows g, g + 8, normalised and stored from the accumulators
#pragma unroll
    for (int nt = 0; nt < kDtiles; ++nt)
      if (nt == int(warp)) {
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
          const unsigned row = row_base + g + hr * 8;
          if (row >= q_rows) continue;
          const float inv = row_sum[hr] > 0.f ? 1.f / row_sum[hr] : 0.f;
          *reinterpret_cast<bf162*>(o + size_t(row) * o_stride + head * head_dim + nt * 8 + 2 * t) =
              __floats2bfloat162_rn(out[nt][2 * hr] * inv, out[nt][2 * hr + 1] * inv);
        }
      }
    return;
  }

  // ---- merge the eight warps: [warp][row 0..15][head_dim + 2] with max and sum in the last two columns ----
  const unsigned mp = head_dim + 2;
  if (kAliasMerge) __syncthreads();   // nobody reads keys or values any more: their space becomes the merge area
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    float* dst = merge + (size_t(warp) * 16 + g + hr * 8) * mp;
#pragma unroll
    for (int nt = 0; nt < kDtiles; ++nt)
      if (nt < dtiles) {
        dst[nt * 8 + 2 * t] = out[nt][2 * hr];
        dst[nt * 8 + 2 * t + 1] = out[nt][2 * hr + 1];
      }
    if (t == 0) {
      dst[head_dim] = row_max[hr];
      dst[head_dim + 1] = row_sum[hr];
    }
  }
  __syncthreads();
  // thread = (row, one of 16 column lanes): the eight warps' weights are worked out once per row
  const unsigned r = threadIdx.x >> 4, c = threadIdx.x & 15;
  if (row_base + r < q_rows) {
    float weight[8], best = -3.0e38f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      weight[w] = merge[(w * 16 + r) * mp + head_dim];
      best = fmaxf(best, weight[w]);
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      weight[w] = weight[w] > -1.0e38f ? __expf(weight[w] - best) : 0.f;
      den += weight[w] * merge[(w * 16 + r) * mp + head_dim + 1];
    }
    const float inv = den > 0.f ? 1.f / den : 0.f;
    for (unsigned d = c; d < head_dim; d += 16) {
      float num = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) num += weight[w] * merge[(w * 16 + r) * mp + d];
      o[size_t(row_base + r) * o_stride + head * head_dim + d] = __float2bfloat16_rn(num * inv);
    }
  }
}

extern "C" __global__ void __launch_bounds__(256)
agi_attention_mma_bf16(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows,
                       unsigned q_heads, unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride,
                       unsigned v_stride, unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg) {
  attention_mma_body<4, 8, false>(q, k, v, o, q_rows, kv_rows, q_heads, kv_heads, head_dim, q_stride, k_stride, v_stride,
                                  o_stride, scale, mask_mode, mask_arg);
}

// The same for heads up to 128 wide (a 50-token action expert over a 256-token prefix: 8 heads of 128).  The streaming
// kernel gives each warp ALL keys of its 16 query rows (640 dependent MMAs at these sizes, with 8 CTAs on the whole
// part); here 8 warps x ceil(q_rows / 16) x heads CTAs split the keys.  Keys, values and the merge area do not fit
// side by side, so the merge re-uses the tiles' space: dynamic shared memory =
// max(2 * kv16 * (head_dim + 8) * 2, 8 * 16 * (head_dim + 2) * 4).
extern "C" __global__ void __launch_bounds__(256)
agi_attention_mma_bf16_d128(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows,
                            unsigned q_heads, unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride,
                            unsigned v_stride, unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg) {
  attention_mma_body<8, 16, true>(q, k, v, o, q_rows, kv_rows, q_heads, kv_heads, head_dim, q_stride, k_stride, v_stride,
                                  o_stride, scale, mask_mode, mask_arg);
}

// Prefill GEMM on the sm_100a tensor cores with a 256 x TN output tile per CTA:
//   Y[M, N] = epilogue(X[M, K] . W[N, K]^T), bf16 or E4M3 operands, fp32 accumulation in TMEM.
//
// The 128-row kernel (gemm_tc.cuh) moves 16 KB of weights and TN * 128 B of activations from L2
// into shared memory for every 128 x TN x (128 B of K) block of work, and at a few hundred tokens
// that traffic, not the tensor core, sets its speed.  Here one CTA owns 256 weight rows, i.e. two
// 128-row MMA tiles that share the activation tile, with two accumulators side by side in tensor
// memory (2 x TN columns, all 512 when TN = 256): a third less shared-memory fill per flop.
//
//   * warps 0-7 are producers: 16-byte cp.async into the 128-byte-swizzled K-major tiles
//     (weights: 256 rows x 128 B, activations: TN rows x 128 B per ring slot), published to the
//     tensor core by fence.proxy.async + mbarrier two commit groups later;
//   * warp 8 issues tcgen05.mma: per 32 bytes of K one instruction per accumulator; tcgen05.commit
//     hands ring slots back to the producers;
//   * afterwards warps 0-7 are the epilogue: warp w reads TMEM lanes 32 * (w % 4) ... of accumulator
//     w / 4 with tcgen05.ld and stores 16 tokens at a time.
//
// Split-K (grid.z slices): every slice stores its partial tile into its own fp32 slab; the slice that
// arrives last at the tile's counter adds the slabs in slice order and runs the epilogue, so the result
// does not depend on timing.  No CTA waits for another.  Every mbarrier wait is bounded (status word).
#pragma once

#include "gemm_tc.cuh"

namespace tcw {

using namespace tc;

constexpr unsigned kRows = 256;                        // weight rows per CTA: two MMA tiles
constexpr unsigned kWideATileBytes = kRows * kRowBytes;  // 32 KB per ring slot
constexpr unsigned kWideProducers = 256;
constexpr unsigned kWideThreads = kWideProducers + 32;

// grid = (ceil(N / 256), ceil(M / TN), splits), block = 288,
// dynamic shared memory = stages * (32768 + TN * 128) + 1024; TN a multiple of 16, <= 256.
template <bool kFp8, bool kPacked = false>
__device__ __forceinline__ void gemm_wide_body(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias,
                                               const bf16* residual, const float* scale_a, const float* scale_w,
                                               float* partial, unsigned* counters, unsigned* status, unsigned M,
                                               unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags,
                                               unsigned TN, unsigned stages) {
  extern __shared__ unsigned char dynamic_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kMaxStages];
  __shared__ __align__(8) unsigned long long empty_bar[kMaxStages];
  __shared__ __align__(8) unsigned long long accum_bar;
  __shared__ unsigned tmem_slot;
  __shared__ unsigned last_flag;

  const unsigned tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned elem = kFp8 ? 1u : 2u;
  const unsigned n0 = blockIdx.x * kRows, m0 = blockIdx.y * TN;
  const unsigned splits = gridDim.z, split = blockIdx.z;
  const unsigned k_blocks_total = (K * elem) / kRowBytes;
  const unsigned per_split = (k_blocks_total + splits - 1) / splits;
  const unsigned kb_begin = min(split * per_split, k_blocks_total);
  const unsigned kb_end = min(kb_begin + per_split, k_blocks_total);
  const unsigned nkb = kb_end - kb_begin;
  const unsigned stage_bytes = kWideATileBytes + TN * kRowBytes;
  const unsigned ring = (smem_u32(dynamic_smem) + 1023u) & ~1023u;
  const unsigned acc_columns = tmem_columns_for(TN);  // columns of one accumulator (power of two >= 32)
  const unsigned columns = 2 * acc_columns;
  const unsigned Np = gridDim.x * kRows;               // row stride of the split-K slabs
  if (stages > kMaxStages) stages = kMaxStages;
  constexpr unsigned kMmaWarp = kWideProducers / 32;

  if (tid == 0) {
    for (unsigned s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], kPacked ? 1 : kWideProducers);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) tmem_alloc(&tmem_slot, columns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_slot;

  const size_t w_row_bytes = size_t(K) * elem, x_row_bytes = size_t(ldx) * elem;
  const unsigned early = min(stages, nkb);
  // A producer thread copies chunk c of rows r0, r0 + 32, ...: eight lanes fetch one row's 128 contiguous
  // bytes; the swizzled destination moves by a constant from row to row (32 rows = 4096 B, r & 7 fixed)
  // and the source by 32 row pitches.  Rows past the matrix are skipped: what the tensor core reads there
  // only reaches accumulator rows / columns that are never stored.
  const unsigned r0 = tid >> 3, chunk = tid & 7;
  const unsigned dst_off = r0 * kRowBytes + ((chunk ^ (r0 & 7)) << 4);
  const unsigned a_rows = (warp < kMmaWarp && n0 + r0 < N) ? (min(kRows, N - n0) - r0 + 31) / 32 : 0;
  const unsigned b_rows = (warp < kMmaWarp && m0 + r0 < M && r0 < TN) ? (min(TN, M - m0) - r0 + 31) / 32 : 0;
  const uint8_t* w_src = w + size_t(n0 + r0) * w_row_bytes + size_t(kb_begin) * kRowBytes + (chunk << 4);
  const uint8_t* x_src = x + size_t(m0 + r0) * x_row_bytes + size_t(kb_begin) * kRowBytes + (chunk << 4);
  const size_t w_step = 32 * w_row_bytes, x_step = 32 * x_row_bytes;
  auto load_weights = [&](unsigned i) {
    const uint8_t* src = w_src + size_t(i) * kRowBytes;
    const unsigned dst = ring + (i % stages) * stage_bytes + dst_off;
#pragma unroll
    for (unsigned j = 0; j < 8; ++j)
      if (j < a_rows) cp_async_16(dst + j * 4096, src + j * w_step);
  };
  // packed operands (see gemm_tc.cuh): a 256-row weight tile of one K block is one contiguous 32 KB run
  const unsigned w_rows_padded = ((N + kRows - 1) / kRows) * kRows;
  const unsigned b_tile_bytes = TN * kRowBytes;
  auto packed_weights = [&](unsigned i) {
    bulk_copy(ring + (i % stages) * stage_bytes, w + (size_t(kb_begin + i) * w_rows_padded + n0) * kRowBytes,
              kWideATileBytes, &full_bar[i % stages]);
  };
  auto packed_tokens = [&](unsigned i) {
    bulk_copy(ring + (i % stages) * stage_bytes + kWideATileBytes, x + (size_t(kb_begin + i) * ldx + m0) * kRowBytes,
              b_tile_bytes, &full_bar[i % stages]);
  };
  // Weights do not depend on the previous kernel: the first ring slots are requested before waiting for it.
  if (kPacked) {
    if (tid == 0)
      for (unsigned i = 0; i < early; ++i) {
        expect_bytes(&full_bar[i], kWideATileBytes + b_tile_bytes);
        packed_weights(i);
      }
  } else if (warp < kMmaWarp) {
    for (unsigned i = 0; i < early; ++i) load_weights(i);
  }

  grid_dependency_wait();

  if (kPacked && warp < kMmaWarp) {
    // warp 0 is the producer: two bulk copies per ring slot, issued by its lane 0; the whole warp walks the
    // loop so that it reaches the epilogue converged; the other warps go straight there
    if (warp == 0) {
      if (lane == 0)
        for (unsigned i = 0; i < early; ++i) packed_tokens(i);
      for (unsigned i = early; i < nkb; ++i) {
        const unsigned s = i % stages;
        mbar_wait(&empty_bar[s], (i / stages - 1) & 1, status, kTimeoutEmpty | s);
        if (lane == 0) {
          expect_bytes(&full_bar[s], kWideATileBytes + b_tile_bytes);
          packed_weights(i);
          packed_tokens(i);
        }
        __syncwarp();
      }
    }
  } else if (warp < kMmaWarp) {
    // ---------------- producers ----------------
    for (unsigned i = 0; i < nkb + kLag; ++i) {
      if (i < nkb) {
        const unsigned s = i % stages, round = i / stages;
        if (round > 0) mbar_wait(&empty_bar[s], (round - 1) & 1, status, kTimeoutEmpty | s);
        if (i >= early) load_weights(i);
        const uint8_t* src = x_src + size_t(i) * kRowBytes;
        const unsigned dst = ring + s * stage_bytes + kWideATileBytes + dst_off;
#pragma unroll
        for (unsigned j = 0; j < 8; ++j)
          if (j < b_rows) cp_async_16(dst + j * 4096, src + j * x_step);
      }
      cp_async_commit();  // an empty group past the end keeps the wait arithmetic uniform
      if (i >= kLag) {
        cp_async_wait<kLag>();
        fence_async_shared();
        mbar_arrive(&full_bar[(i - kLag) % stages]);
      }
    }
  } else {
    // ---------------- MMA warp: every lane waits, lane 0 issues ----------------
    const unsigned idesc = instr_descriptor<kFp8>(TN);
    for (unsigned i = 0; i < nkb; ++i) {
      const unsigned s = i % stages, round = i / stages;
      mbar_wait(&full_bar[s], round & 1, status, kTimeoutFull | s);
      tc_fence_after();
      if (lane == 0) {
        const unsigned a_base = ring + s * stage_bytes, b_base = a_base + kWideATileBytes;
        const unsigned long long a0 = smem_descriptor(a_base), a1 = smem_descriptor(a_base + kATileBytes);
        const unsigned long long b_desc = smem_descriptor(b_base);
#pragma unroll
        for (unsigned k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per ring slot
          mma<kFp8>(tmem_base, a0 + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0);
          mma<kFp8>(tmem_base + acc_columns, a1 + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0);
        }
        tc_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (lane == 0) tc_commit(&accum_bar);
    __syncwarp();
  }

  // ---------------- epilogue: warp w -> accumulator w / 4, TMEM lanes 32 * (w % 4) ... ----------------
  if (warp < kMmaWarp) {
    if (nkb > 0) mbar_wait(&accum_bar, 0, status, kTimeoutAccum);
    tc_fence_after();
    const unsigned half = warp >> 2, quarter = warp & 3;
    const unsigned n = n0 + half * kTileN + quarter * 32 + lane;
    const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
    const float bias_v = ((flags & kFlagBias) && n < N) ? __bfloat162float(bias[n]) : 0.f;
    const unsigned lane_addr = tmem_base + half * acc_columns + ((quarter * 32u) << 16);
    const bool f32 = (flags & kFlagOutF32) != 0;
    for (unsigned c0 = 0; c0 < TN; c0 += 16) {
      if (m0 + c0 >= M) break;
      float v[16];
      if (nkb > 0) {
        tmem_load16(lane_addr + c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      if (n >= N) continue;
      const unsigned count = min(16u, M - (m0 + c0));
      if (splits == 1) {
        const size_t offset = size_t(m0 + c0) * ldy + n;
        if (count == 16) {
          if (f32) store_tokens16<true, true>(v, 16, y, residual, offset, ldy, alpha, bias_v, flags);
          else store_tokens16<false, true>(v, 16, y, residual, offset, ldy, alpha, bias_v, flags);
        } else {
          if (f32) store_tokens16<true, false>(v, count, y, residual, offset, ldy, alpha, bias_v, flags);
          else store_tokens16<false, false>(v, count, y, residual, offset, ldy, alpha, bias_v, flags);
        }
      } else {
        float* slab = partial + (size_t(split) * M + m0 + c0) * Np + n;
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (unsigned(i) < count) __stcg(slab + size_t(i) * Np, v[i]);
      }
    }
    if (splits > 1) __threadfence();  // partial sums ordered before this CTA's arrival count
    tc_fence_before();
  }
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_free(tmem_base, columns);
  }
  if (splits == 1) return;

  // ---------------- split-K: the last slice to arrive finishes the tile ----------------
  const unsigned tile = blockIdx.y * gridDim.x + blockIdx.x;
  if (tid == 0) {
    __threadfence();
    last_flag = atomicAdd(&counters[tile], 1u) == splits - 1;
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  if (warp < kMmaWarp) {
    // Warp w finishes token rows w, w + 8, ...; lane l owns features n0 + 4l ... + 3 of each 128-row half.
    const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
    const unsigned rows = min(TN, M - m0);
    const size_t slab = size_t(M) * Np / 4;
    // two token rows x two 128-row halves per pass: all their slab loads are in flight before the first sum
    for (unsigned i0 = warp; i0 < rows; i0 += 2 * kMmaWarp) {
      float4 part[4][8];
#pragma unroll
      for (unsigned u = 0; u < 4; ++u) {
        const unsigned i = i0 + (u >> 1) * kMmaWarp, n = n0 + (u & 1) * kTileN + lane * 4;
        if (i >= rows || n >= N) continue;
        const float4* cell = reinterpret_cast<const float4*>(partial + size_t(m0 + i) * Np + n);
#pragma unroll
        for (unsigned z = 0; z < 8; ++z)
          if (z < splits) part[u][z] = __ldcg(cell + z * slab);
      }
#pragma unroll
      for (unsigned u = 0; u < 4; ++u) {
        const unsigned i = i0 + (u >> 1) * kMmaWarp, n = n0 + (u & 1) * kTileN + lane * 4;
        if (i >= rows || n >= N) continue;
        float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (unsigned z = 0; z < 8; ++z)
          if (z < splits) {
            total.x += part[u][z].x; total.y += part[u][z].y; total.z += part[u][z].z; total.w += part[u][z].w;
          }
        const float t4[4] = {total.x, total.y, total.z, total.w};
        store_features4(t4, m0 + i, n, N, y, ldy, bias, residual, alpha, flags);
      }
    }
  }
  if (tid == 0) counters[tile] = 0;
}

}  // namespace tcw

// At most 8 K slices.
extern "C" __global__ void __launch_bounds__(tcw::kWideThreads, 1)
agi_gemm_tc_wide_bf16(const bf16* x, const bf16* w, void* y, const bf16* bias, const bf16* residual,
                      const float* scale_a, const float* scale_w, float* partial, unsigned* counters, unsigned* status,
                      unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN,
                      unsigned stages) {
  tcw::gemm_wide_body<false>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias, residual,
                             scale_a, scale_w, partial, counters, status, M, N, K, ldx, ldy, flags, TN, stages);
}

extern "C" __global__ void __launch_bounds__(tcw::kWideThreads, 1)
agi_gemm_tc_wide_e4m3(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias, const bf16* residual,
                      const float* scale_a, const float* scale_w, float* partial, unsigned* counters, unsigned* status,
                      unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN,
                      unsigned stages) {
  tcw::gemm_wide_body<true>(x, w, y, bias, residual, scale_a, scale_w, partial, counters, status, M, N, K, ldx, ldy,
                            flags, TN, stages);
}

// The same over packed operands (bulk-copy producers; ldx = padded row count of the activation matrix; the
// weight matrix is padded to whole 256-row tiles).
extern "C" __global__ void __launch_bounds__(tcw::kWideThreads, 1)
agi_gemm_tcp_wide_e4m3(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias, const bf16* residual,
                       const float* scale_a, const float* scale_w, float* partial, unsigned* counters, unsigned* status,
                       unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN,
                       unsigned stages) {
  tcw::gemm_wide_body<true, true>(x, w, y, bias, residual, scale_a, scale_w, partial, counters, status, M, N, K, ldx,
                                  ldy, flags, TN, stages);
}

// Persistent tensor-core GEMM over packed operands, for shapes with more output tiles than SMs:
//   Y[M, N] = epilogue(X[M, K] . W[N, K]^T), E4M3 operands in the packed layout of recipes/layout.py,
//   fp32 accumulation in tensor memory, bf16 or fp32 output.
//
// One CTA per SM walks the output tiles (128 weight rows x TN tokens) t = blockIdx.x, + gridDim.x, ...
// with three kinds of warps that never wait for each other except through mbarriers:
//   * warp 0, the producer: for every K block of every tile of this CTA, two bulk copies (16 KB of weights,
//     TN * 128 B of activations) into the next ring slot; the ring runs on across tile boundaries, so the first
//     K blocks of tile i + 1 are in flight while tile i is still being multiplied;
//   * warp 1 issues tcgen05.mma into one of TWO accumulators in tensor memory (2 x TN columns) and hands a
//     finished accumulator to the epilogue with tcgen05.commit;
//   * warps 2-5, the epilogue: tcgen05.ld of the finished accumulator (warp w reads TMEM lanes 32 * (w % 4) ...),
//     scale / bias / activation / residual, store, then give the accumulator back.  The epilogue of tile i
//     therefore overlaps the multiplication of tile i + 1, which is what the one-tile-per-CTA kernels lack.
// Every wait is bounded; after the first expiry a CTA stops waiting altogether (its status word says so), so a
// logic error costs one time-out per warp, not one per K block.
#pragma once

#include "gemm_tc.cuh"

namespace tcq {

using namespace tc;

constexpr unsigned kPersistThreads = 192;   // producer warp, MMA warp, four epilogue warps

__device__ __forceinline__ bool wait_or_give_up(unsigned long long* bar, unsigned parity, unsigned* status, unsigned code,
                                                volatile unsigned* gave_up) {
  if (*gave_up) return false;
  if (mbar_wait(bar, parity, status, code)) return true;
  *gave_up = 1;
  return false;
}

// grid = (min(tiles, SMs), 1, 1), block = 192, dynamic shared memory = stages * (16384 + TN * 128) + 1024;
// TN a multiple of 16, <= 256; ldx = padded row count of the packed activation matrix.
__device__ __forceinline__ void persistent_body(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias,
                                                const bf16* residual, const float* scale_a, const float* scale_w,
                                                unsigned* status, unsigned M, unsigned N, unsigned K, unsigned ldx,
                                                unsigned ldy, unsigned flags, unsigned TN, unsigned stages) {
  extern __shared__ unsigned char dynamic_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kMaxStages];
  __shared__ __align__(8) unsigned long long empty_bar[kMaxStages];
  __shared__ __align__(8) unsigned long long acc_full[2];
  __shared__ __align__(8) unsigned long long acc_empty[2];
  __shared__ unsigned tmem_slot;
  __shared__ unsigned gave_up;

  const unsigned tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned n_tiles = (N + kTileN - 1) / kTileN, m_tiles = (M + TN - 1) / TN, tiles = n_tiles * m_tiles;
  const unsigned nkb = K / kRowBytes;                       // E4M3: one byte per element
  const unsigned stage_bytes = kATileBytes + TN * kRowBytes;
  const unsigned ring = (smem_u32(dynamic_smem) + 1023u) & ~1023u;
  const unsigned acc_columns = tmem_columns_for(TN);
  const unsigned w_rows_padded = ((N + 255u) / 256u) * 256u;
  if (stages > kMaxStages) stages = kMaxStages;

  if (tid == 0) {
    for (unsigned s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (unsigned b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 4);   // one arrival per epilogue warp
    }
    gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(&tmem_slot, 2 * acc_columns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_slot;
  grid_dependency_wait();

  if (warp == 0) {
    // ---------------- producer ----------------
    unsigned g = 0;                                          // ring position, running across tiles
    for (unsigned tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
      const unsigned n0 = (tile % n_tiles) * kTileN, m0 = (tile / n_tiles) * TN;
      for (unsigned kb = 0; kb < nkb; ++kb, ++g) {
        const unsigned s = g % stages, round = g / stages;
        wait_or_give_up(&empty_bar[s], (round & 1) ^ 1, status, kTimeoutEmpty | s, &gave_up);
        if (lane == 0) {
          expect_bytes(&full_bar[s], stage_bytes);
          bulk_copy(ring + s * stage_bytes, w + (size_t(kb) * w_rows_padded + n0) * kRowBytes, kATileBytes, &full_bar[s]);
          bulk_copy(ring + s * stage_bytes + kATileBytes, x + (size_t(kb) * ldx + m0) * kRowBytes, TN * kRowBytes,
                    &full_bar[s]);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const unsigned idesc = instr_descriptor<true>(TN);
    unsigned g = 0, it = 0;
    for (unsigned tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const unsigned buf = it & 1, use = it >> 1;
      wait_or_give_up(&acc_empty[buf], (use & 1) ^ 1, status, kTimeoutAccum | 0x10 | buf, &gave_up);
      tc_fence_after();
      const unsigned acc = tmem_base + buf * acc_columns;
      for (unsigned kb = 0; kb < nkb; ++kb, ++g) {
        const unsigned s = g % stages, round = g / stages;
        wait_or_give_up(&full_bar[s], round & 1, status, kTimeoutFull | s, &gave_up);
        tc_fence_after();
        if (lane == 0) {
          const unsigned a_base = ring + s * stage_bytes, b_base = a_base + kATileBytes;
          const unsigned long long a_desc = smem_descriptor(a_base), b_desc = smem_descriptor(b_base);
#pragma unroll
          for (unsigned k = 0; k < 4; ++k) mma<true>(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0);
          tc_commit(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (lane == 0) tc_commit(&acc_full[buf]);
      __syncwarp();
    }
  } else {
    // ---------------- epilogue warps 2-5: TMEM lane quarter = warp % 4 ----------------
    const unsigned quarter = warp & 3;
    const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
    const bool f32 = (flags & kFlagOutF32) != 0;
    unsigned it = 0;
    for (unsigned tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++it) {
      const unsigned buf = it & 1, use = it >> 1;
      const unsigned n0 = (tile % n_tiles) * kTileN, m0 = (tile / n_tiles) * TN;
      const unsigned n = n0 + quarter * 32 + lane;
      const float bias_v = ((flags & kFlagBias) && n < N) ? __bfloat162float(bias[n]) : 0.f;
      wait_or_give_up(&acc_full[buf], use & 1, status, kTimeoutAccum | buf, &gave_up);
      tc_fence_after();
      const unsigned lane_addr = tmem_base + buf * acc_columns + ((quarter * 32u) << 16);
      for (unsigned c0 = 0; c0 < TN; c0 += 16) {
        if (m0 + c0 >= M) break;
        float v[16];
        tmem_load16(lane_addr + c0, v);
        if (n >= N) continue;
        const unsigned count = min(16u, M - (m0 + c0));
        const size_t offset = size_t(m0 + c0) * ldy + n;
        if (count == 16) {
          if (f32) store_tokens16<true, true>(v, 16, y, residual, offset, ldy, alpha, bias_v, flags);
          else store_tokens16<false, true>(v, 16, y, residual, offset, ldy, alpha, bias_v, flags);
        } else {
          if (f32) store_tokens16<true, false>(v, count, y, residual, offset, ldy, alpha, bias_v, flags);
          else store_tokens16<false, false>(v, count, y, residual, offset, ldy, alpha, bias_v, flags);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);   // this warp has read its quarter: the accumulator may be reused
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_free(tmem_base, 2 * acc_columns);
  }
}

}  // namespace tcq

extern "C" __global__ void __launch_bounds__(tcq::kPersistThreads, 1)
agi_gemm_tcq_e4m3(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias, const bf16* residual,
                  const float* scale_a, const float* scale_w, unsigned* status, unsigned M, unsigned N, unsigned K,
                  unsigned ldx, unsigned ldy, unsigned flags, unsigned TN, unsigned stages) {
  tcq::persistent_body(x, w, y, bias, residual, scale_a, scale_w, status, M, N, K, ldx, ldy, flags, TN, stages);
}

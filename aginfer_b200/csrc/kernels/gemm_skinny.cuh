// Weight-streaming skinny GEMM for the batch-1 action head: Y[M, N] = epilogue(X[M, K] . W[N, K]^T)
// with M <= 64 tokens.  HBM-bound: every weight byte is read exactly once, straight from global
// memory into registers with 16-byte loads, and nothing is reduced across CTAs.
//
// A CTA owns `rows` (8 or 16) consecutive output features and all of K; its 8 warps take
// interleaved 64-byte windows of K (a warp's four-lane groups read 64 contiguous bytes of one
// weight row, the 8 warps together 512 contiguous bytes per row).  Each thread's 16-byte
// chunk feeds two warp-level MMAs (m16n8k16 bf16, or m16n8k32 E4M3) using the chunk's own
// element order along K for both operands: a dot product does not care in which order K is
// visited as long as weights and activations agree.  Activations come from global memory
// through L1 (they are at most a few hundred KB and shared by every warp of the SM).  After
// the K loop the 8 partial tiles are summed through shared memory in warp order and the
// usual epilogue (scale, bias, activation, residual) writes bf16 or fp32.
//
// Grid = ceil(N / rows); rows = 8 is chosen when N / 16 would leave SMs idle.
#pragma once

#include "common.cuh"
#include "gemm_simt.cuh"  // gemm_store

namespace skinny {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ uint4 load_stream(const void* p) {  // weights: read once, keep out of L1
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 load_cached(const void* p) {  // activations: reused by every warp
  return __ldg(reinterpret_cast<const uint4*>(p));
}

template <bool kFp8>
__device__ __forceinline__ void mma16n8(float c[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                        unsigned b1) {
  if (kFp8) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// NT = number of 8-token tiles (M <= 8 * NT).
template <bool kFp8, int NT>
__device__ __forceinline__ void body(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias,
                                     const bf16* residual, const float* scale_a, const float* scale_w, unsigned M,
                                     unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags,
                                     unsigned rows, float* partial_buf) {
  constexpr int kUnroll = NT <= 4 ? 4 : 2;  // K windows in flight per thread (x2: the next batch is prefetched)
  constexpr int kPitch = NT * 8 + 1;        // +1: rows of the 16 x tokens tile land in different banks
  float (*partial)[16][kPitch] = reinterpret_cast<float (*)[16][kPitch]>(partial_buf);
  const unsigned elem = kFp8 ? 1u : 2u;
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned row0 = blockIdx.x * rows;
  const bool two_halves = rows == 16;
  const unsigned windows = K * elem / 64;
  const size_t w_row = size_t(K) * elem, x_row = size_t(ldx) * elem;

  // Weight rows of this lane group (clamped: rows past N are computed from the last row and dropped).
  const uint8_t* w_lo = w + size_t(min(row0 + g, N - 1)) * w_row + t * 16;
  const uint8_t* w_hi = w + size_t(min(row0 + g + 8, N - 1)) * w_row + t * 16;
  const uint8_t* x_tok[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) x_tok[nt] = x + size_t(min(unsigned(nt * 8) + g, M - 1)) * x_row + t * 16;

  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nt][i] = 0.f;

  // Weights do not depend on the previous kernel: the first batch of loads is issued before waiting
  // for it, so under programmatic dependent launch the stream from HBM starts early.
  uint4 lo[kUnroll], hi[kUnroll];
  const uint4 zero = make_uint4(0, 0, 0, 0);
  unsigned win = warp;
#pragma unroll
  for (int u = 0; u < kUnroll; ++u) {
    const unsigned wi = win + u * kWarps;
    lo[u] = wi < windows ? load_stream(w_lo + size_t(wi) * 64) : zero;
    hi[u] = (two_halves && wi < windows) ? load_stream(w_hi + size_t(wi) * 64) : zero;
  }
  grid_dependency_wait();
  grid_dependency_release();

  for (; win < windows; win += kUnroll * kWarps) {
    uint4 nlo[kUnroll], nhi[kUnroll];
    const unsigned next = win + kUnroll * kWarps;
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {  // prefetch the following batch while this one is multiplied
      const unsigned wi = next + u * kWarps;
      nlo[u] = wi < windows ? load_stream(w_lo + size_t(wi) * 64) : zero;
      nhi[u] = (two_halves && wi < windows) ? load_stream(w_hi + size_t(wi) * 64) : zero;
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const unsigned wi = win + u * kWarps;
      if (wi >= windows) break;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const uint4 b = load_cached(x_tok[nt] + size_t(wi) * 64);
        mma16n8<kFp8>(acc[nt], lo[u].x, hi[u].x, lo[u].y, hi[u].y, b.x, b.y);
        mma16n8<kFp8>(acc[nt], lo[u].z, hi[u].z, lo[u].w, hi[u].w, b.z, b.w);
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      lo[u] = nlo[u];
      hi[u] = nhi[u];
    }
  }

  // c0,c1: row g, tokens 2t, 2t+1 of the tile; c2,c3: row g + 8.
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    partial[warp][g][nt * 8 + 2 * t] = acc[nt][0];
    partial[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
    partial[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
    partial[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
  }
  __syncthreads();
  const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
  for (unsigned i = threadIdx.x; i < rows * M; i += kThreads) {
    const unsigned r = i % rows, m = i / rows;  // consecutive threads -> consecutive output features
    const unsigned n = row0 + r;
    if (n >= N) continue;
    float total = 0.f;
#pragma unroll
    for (int wq = 0; wq < kWarps; ++wq) total += partial[wq][r][m];
    gemm_store(total, m, n, y, ldy, bias, residual, alpha, flags);
  }
}

}  // namespace skinny

// grid = (ceil(N / rows), 1, 1), block = 256; M <= 8 * tiles; K bytes a multiple of 64; rows in {8, 16}.
// One kernel per token-tile count so that each gets its own register budget.
#define AGI_SKINNY_KERNEL(NAME, TYPE, FP8, NT)                                                                       \
  extern "C" __global__ void __launch_bounds__(skinny::kThreads, 2)                                                  \
  NAME(const TYPE* x, const TYPE* w, void* y, const bf16* bias, const bf16* residual, const float* scale_a,         \
       const float* scale_w, unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags,        \
       unsigned rows) {                                                                                              \
    __shared__ float partial_buf[skinny::kWarps * 16 * (NT * 8 + 1)];                                                \
    skinny::body<FP8, NT>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias,         \
                          residual, scale_a, scale_w, M, N, K, ldx, ldy, flags, rows, partial_buf);                 \
  }

AGI_SKINNY_KERNEL(agi_gemm_skinny_bf16_t1, bf16, false, 1)
AGI_SKINNY_KERNEL(agi_gemm_skinny_bf16_t2, bf16, false, 2)
AGI_SKINNY_KERNEL(agi_gemm_skinny_bf16_t3, bf16, false, 3)
AGI_SKINNY_KERNEL(agi_gemm_skinny_bf16_t4, bf16, false, 4)
AGI_SKINNY_KERNEL(agi_gemm_skinny_bf16_t6, bf16, false, 6)
AGI_SKINNY_KERNEL(agi_gemm_skinny_bf16_t8, bf16, false, 8)
AGI_SKINNY_KERNEL(agi_gemm_skinny_e4m3_t1, uint8_t, true, 1)
AGI_SKINNY_KERNEL(agi_gemm_skinny_e4m3_t2, uint8_t, true, 2)
AGI_SKINNY_KERNEL(agi_gemm_skinny_e4m3_t3, uint8_t, true, 3)
AGI_SKINNY_KERNEL(agi_gemm_skinny_e4m3_t4, uint8_t, true, 4)
AGI_SKINNY_KERNEL(agi_gemm_skinny_e4m3_t6, uint8_t, true, 6)
AGI_SKINNY_KERNEL(agi_gemm_skinny_e4m3_t8, uint8_t, true, 8)
#undef AGI_SKINNY_KERNEL

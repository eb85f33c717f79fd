// Weight-streaming tensor-core GEMM for a handful of tokens: Y[M, N] = epilogue(X[M, K] . W[N, K]^T), M <= 32,
// bf16, weights in the packed layout (K-block-major, swizzled: recipes/layout.py), tcgen05.mma with the
// accumulators in tensor memory.
//
//   * a CTA owns 128 output features x one K slice of at most 10 blocks of 64 elements: a "slab" that is
//     requested in full - one bulk copy of 16 KB per K block, issued by one thread - BEFORE the grid-dependency
//     wait.  There is no ring: nothing is ever waited for twice.
//   * after the wait, four warps bring the K slice of the M activation rows (row-major bf16, a few KB) through
//     registers into the swizzled K-major tile the tensor core reads; one thread issues 4 MMAs per K block
//     (128 x 32 x 16 each: the weights are the A operand, tokens are the accumulator columns) into four
//     accumulators, so that consecutive MMAs do not depend on one another; the same four warps read and add the
//     accumulators (one output feature per thread) with tcgen05.ld.
//   * K slices of one tile meet either in a thread-block cluster (kCluster > 1: grid.z = cluster size; every
//     rank owns the tokens t with t % C == rank and receives their partial sums through distributed shared
//     memory) or, without a cluster, in fp32 slabs in global memory where the last slice to arrive adds them.
//     Both add in slice order, so the result does not depend on timing.  With kCluster > 1 and grid.y = G > 1,
//     G clusters share a tile (K is cut into G * C slices): each rank writes its cluster's sum for its tokens
//     and the last of the G to arrive adds those, again in order.
//   * up to three weight matrices side by side along N (queries | keys | values) share a launch.
//
// Measured on B200 (17 tokens, launches chained by programmatic dependent launch, globaltimer stamps of every
// CTA).  A launch whose successor's CTAs all fit beside its own (1536 x 1536: 96 CTAs of 79 KB) repeats every
// 4.6 us: 3.8 us from the release of the grid-dependency wait to the last store (activation copy 0.6, MMAs
// 0.3-0.5, tcgen05.ld and remote stores 0.5, cluster barrier and epilogue 1.1, the rest barrier hand-overs) and
// 0.8 us until the successor's wait is released - the same as the bulk-stream mma.sync kernel at this size
// (4.3 us).  For the 19 MB matrices (6144 x 1536, 1536 x 6144) the successor's CTAs do not fit beside the
// running ones (two GEMMs need 256 KB of weights per SM); they enter only as CTAs exit, the last of them 6-9 us
// after the first, and the wait is released when the last one is in: 9.2-10.9 us per launch against 7.0 / 10.5 us
// of the bulk-stream kernel, whose smaller CTAs (16 rows, 73-104 KB, three or two per SM) hand the SMs over more
// evenly.  Inside the action head's graph the packed path therefore costs 3.57 ms per chunk against 2.93 ms
// (per matrix family: output projection +0.01 ms, Q|K|V +0.08, MLP up +0.25, MLP down +0.30), and recipes use
// it only when the checkpoint was packaged in the packed layout.  Two things tried on the way and dropped,
// neither of which shortened a launch: an L2 prefetch (cp.async.bulk.prefetch.L2 or
// prefetch.global.L2) of the next launch's weights issued by every CTA, and a single accumulator (an MMA of
// this shape occupies the pipe ~128 cycles whatever N is: the A operand streams at 32 B per clock).
//
// Every wait is bounded and reports through the status word.
#pragma once

#include "common.cuh"
#include "gemm_tc.cuh"

namespace tcs {

constexpr unsigned kThreads = 160;       // 4 copy / epilogue warps + the MMA warp
constexpr unsigned kMaxBlocks = 10;      // K blocks (64 bf16) per slice
constexpr unsigned kTokens = 32;         // accumulator columns
constexpr unsigned kAccumulators = 4;    // independent accumulators: consecutive MMAs do not wait for one another
constexpr unsigned kATile = 128 * 128;   // bytes of one K block of the slab
constexpr unsigned kBTile = kTokens * 128;
constexpr unsigned kTimeoutWeights = 0xA00, kTimeoutTokens = 0xA10, kTimeoutAccum = 0xA20;

struct Parts {
  const uint8_t* w[3];
  const bf16* bias[3];
  unsigned n[3];
};

// Dynamic shared memory: [slab: nkb x 16 KB][token tiles: nkb x 4 KB][gather: C x ceil(32 / C) x 512 B], after
// alignment to 1024 bytes.
template <int kCluster>
__device__ __forceinline__ void body(const bf16* x, const Parts& parts, bf16* y, const bf16* residual, float* partial,
                                     unsigned* counters, unsigned* status, unsigned M, unsigned K, unsigned ldx,
                                     unsigned ldy, unsigned flags, unsigned kb_per_slice) {
  extern __shared__ unsigned char dynamic_smem[];
  __shared__ __align__(8) unsigned long long weights_bar[kMaxBlocks];
  __shared__ __align__(8) unsigned long long tokens_bar, accum_bar;
  __shared__ unsigned tmem_slot, last_flag;

  const unsigned tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // which weight matrix this tile belongs to
  const unsigned t0 = parts.n[0] / 128, t1 = parts.n[1] / 128;
  unsigned tile = blockIdx.x, col0 = 0, N = parts.n[0];
  const uint8_t* w = parts.w[0];
  const bf16* bias = parts.bias[0];
  if (tile >= t0 + t1) {
    w = parts.w[2]; bias = parts.bias[2]; N = parts.n[2]; tile -= t0 + t1; col0 = parts.n[0] + parts.n[1];
  } else if (tile >= t0) {
    w = parts.w[1]; bias = parts.bias[1]; N = parts.n[1]; tile -= t0; col0 = parts.n[0];
  }
  const unsigned n0 = tile * 128;
  const unsigned Np = gridDim.x * 128;                     // row pitch of the global slabs: all tiles side by side
  const unsigned slices = kCluster > 1 ? kCluster * gridDim.y : gridDim.z;
  const unsigned split = kCluster > 1 ? blockIdx.y * kCluster + blockIdx.z : blockIdx.z;
  const unsigned rank = kCluster > 1 ? blockIdx.z : 0;
  const unsigned k_blocks = K / 64;
  const unsigned kb_begin = min(split * kb_per_slice, k_blocks);
  const unsigned nkb = min(min(kb_per_slice, kMaxBlocks), k_blocks - kb_begin);
  const unsigned ring = (tc::smem_u32(dynamic_smem) + 1023u) & ~1023u;
  const unsigned tokens_base = ring + kb_per_slice * kATile;
  constexpr unsigned kGatherCols = (kTokens + kCluster - 1) / kCluster;
  const unsigned gather_base = tokens_base + kb_per_slice * kBTile;

  if (tid == 0) {
    for (unsigned i = 0; i < nkb; ++i) tc::mbar_init(&weights_bar[i], 1);
    tc::mbar_init(&tokens_bar, 128);
    tc::mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    // the whole slab, now: weights do not depend on the previous kernel
    const unsigned rows_padded = ((N + 255u) / 256u) * 256u;
    for (unsigned i = 0; i < nkb; ++i) {
      tc::expect_bytes(&weights_bar[i], kATile);
      tc::bulk_copy(ring + i * kATile, w + (size_t(kb_begin + i) * rows_padded + n0) * 128, kATile, &weights_bar[i]);
    }
  }
  if (warp == 4) tc::tmem_alloc(&tmem_slot, kTokens * kAccumulators);
  tc::tc_fence_before();
  __syncthreads();
  tc::tc_fence_after();
  const unsigned tmem_base = tmem_slot;
  if (kCluster > 1) tc::cluster_arrive();   // paired with the wait just before the first remote store

  grid_dependency_wait();

  if (warp < 4) {
    // ---------------- activations: M rows x nkb blocks x 8 chunks of 16 bytes ----------------
    // thread t moves 16-byte chunk (t & 7) of rows t / 8, t / 8 + 16 of every K block: all loads first
    const unsigned c = tid & 7, r0 = tid >> 3;
    const bf16* src = x + size_t(r0) * ldx + size_t(kb_begin) * 64 + c * 8;
    uint4 held[kMaxBlocks][2];
#pragma unroll
    for (unsigned kb = 0; kb < kMaxBlocks; ++kb)
#pragma unroll
      for (unsigned h = 0; h < 2; ++h)
        if (kb < nkb && r0 + 16 * h < M)
          held[kb][h] = __ldcg(reinterpret_cast<const uint4*>(src + size_t(16 * h) * ldx + kb * 64));
#pragma unroll
    for (unsigned kb = 0; kb < kMaxBlocks; ++kb)
#pragma unroll
      for (unsigned h = 0; h < 2; ++h)
        if (kb < nkb && r0 + 16 * h < M) {
          const unsigned r = r0 + 16 * h;
          const unsigned dst = tokens_base + kb * kBTile + r * 128 + ((c ^ (r & 7)) << 4);
          asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst), "r"(held[kb][h].x), "r"(held[kb][h].y),
                       "r"(held[kb][h].z), "r"(held[kb][h].w) : "memory");
        }
    tc::fence_async_shared();
    tc::mbar_arrive(&tokens_bar);
  } else {
    // ---------------- MMA warp ----------------
    const unsigned idesc = tc::instr_descriptor<false>(kTokens);
    tc::mbar_wait(&tokens_bar, 0, status, kTimeoutTokens);
    for (unsigned i = 0; i < nkb; ++i) {
      tc::mbar_wait(&weights_bar[i], 0, status, kTimeoutWeights | i);
      tc::tc_fence_after();
      if (lane == 0) {
        const unsigned long long a_desc = tc::smem_descriptor(ring + i * kATile);
        const unsigned long long b_desc = tc::smem_descriptor(tokens_base + i * kBTile);
#pragma unroll
        for (unsigned k = 0; k < 4; ++k)   // the four 16-element steps of a K block go to four accumulators
          tc::mma<false>(tmem_base + kTokens * k, a_desc + 2 * k, b_desc + 2 * k, idesc, i != 0);
      }
      __syncwarp();
    }
    if (lane == 0) tc::tc_commit(&accum_bar);
    __syncwarp();
    if (kCluster > 1) tc::cluster_wait();
  }

  // ---------------- accumulator -> registers (thread = output feature n0 + 32 * warp + lane) ----------------
  const unsigned row = warp * 32 + lane, n = n0 + row;
  if (warp < 4) {
    float v[32];
    if (nkb > 0) {
      tc::mbar_wait(&accum_bar, 0, status, kTimeoutAccum);
      tc::tc_fence_after();
      const unsigned lane_addr = tmem_base + ((warp * 32u) << 16);
      tc::tmem_load16(lane_addr, v);
      if (M > 16) tc::tmem_load16(lane_addr + 16, v + 16);
#pragma unroll
      for (unsigned a = 1; a < kAccumulators; ++a) {   // fixed order: the sum does not depend on timing
        float t[16];
        tc::tmem_load16(lane_addr + kTokens * a, t);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] += t[i];
        if (M > 16) {
          tc::tmem_load16(lane_addr + kTokens * a + 16, t);
#pragma unroll
          for (int i = 0; i < 16; ++i) v[16 + i] += t[i];
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = 0.f;
    }
    if (kCluster > 1) {
      tc::cluster_wait();   // peers are running: their gather buffers may be written
#pragma unroll
      for (unsigned c = 0; c < kTokens; ++c) {
        if (c >= M) break;
        const unsigned cell = gather_base + ((rank * kGatherCols + c / kCluster) * 128 + row) * 4;
        tc::store_peer_f32(tc::peer_smem(cell, c % kCluster), v[c]);
      }
    } else if (slices == 1) {
      if (n < N) {
        const float bias_v = (flags & kFlagBias) ? __bfloat162float(bias[n]) : 0.f;
        const size_t offset = col0 + n;
        if (M >= 16) tc::store_tokens16<false, true>(v, 16, y, residual, offset, ldy, 1.f, bias_v, flags);
        else tc::store_tokens16<false, false>(v, M, y, residual, offset, ldy, 1.f, bias_v, flags);
        if (M > 16) tc::store_tokens16<false, false>(v + 16, M - 16, y, residual, offset + size_t(16) * ldy, ldy, 1.f, bias_v, flags);
      }
    } else {
      float* cell = partial + size_t(split) * M * Np + col0 + n;
#pragma unroll
      for (unsigned c = 0; c < kTokens; ++c)
        if (c < M) __stcg(cell + size_t(c) * Np, v[c]);
    }
    tc::tc_fence_before();
  }
  __syncthreads();
  if (warp == 4) {
    tc::tc_fence_after();
    tc::tmem_free(tmem_base, kTokens * kAccumulators);
  }

  if (kCluster > 1) {
    // ---------------- this rank finishes tokens rank, rank + C, ... ----------------
    const unsigned groups = gridDim.y, group = blockIdx.y;
    const unsigned mine = (warp < 4 && n < N && rank < M) ? (M - rank + kCluster - 1) / kCluster : 0;
    bf16 early_bias = __float2bfloat16_rn(0.f), early_res[kGatherCols];
    if (mine != 0 && (flags & kFlagBias)) early_bias = bias[n];
#pragma unroll
    for (unsigned j = 0; j < kGatherCols; ++j)
      if (j < mine && (flags & kFlagResidual)) early_res[j] = residual[size_t(rank + j * kCluster) * ldy + col0 + n];
    tc::cluster_arrive();
    tc::cluster_wait();   // every slice's stores into this CTA's gather buffer are complete and visible
    const float* gathered = reinterpret_cast<const float*>(dynamic_smem + (gather_base - tc::smem_u32(dynamic_smem)));
    float total[kGatherCols];
#pragma unroll
    for (unsigned j = 0; j < kGatherCols; ++j) {
      total[j] = 0.f;
      if (j >= mine) continue;
#pragma unroll
      for (int z = 0; z < kCluster; ++z) total[j] += gathered[(z * kGatherCols + j) * 128 + row];   // slice order
    }
    if (groups > 1) {
      // several clusters share the tile: file this cluster's sums, the last cluster to arrive for this rank adds them
      float* cell = partial + size_t(group) * M * Np + col0 + n;
#pragma unroll
      for (unsigned j = 0; j < kGatherCols; ++j)
        if (j < mine) __stcg(cell + size_t(rank + j * kCluster) * Np, total[j]);
      __threadfence();
      __syncthreads();
      if (tid == 0) {
        __threadfence();
        last_flag = atomicAdd(&counters[blockIdx.x * kCluster + rank], 1u) == groups - 1;
      }
      __syncthreads();
      if (!last_flag) return;
      __threadfence();
      float part_sum[kGatherCols][4];
#pragma unroll
      for (unsigned j = 0; j < kGatherCols; ++j)
#pragma unroll
        for (unsigned g = 0; g < 4; ++g)
          if (j < mine && g < groups)
            part_sum[j][g] = __ldcg(partial + (size_t(g) * M + rank + j * kCluster) * Np + col0 + n);
#pragma unroll
      for (unsigned j = 0; j < kGatherCols; ++j) {
        total[j] = 0.f;
#pragma unroll
        for (unsigned g = 0; g < 4; ++g)
          if (j < mine && g < groups) total[j] += part_sum[j][g];
      }
      if (tid == 0) counters[blockIdx.x * kCluster + rank] = 0;
    }
#pragma unroll
    for (unsigned j = 0; j < kGatherCols; ++j) {
      if (j >= mine) continue;
      float r = total[j];
      if (flags & kFlagBias) r += __bfloat162float(early_bias);
      r = apply_activation(r, flags);
      if (flags & kFlagResidual) r += __bfloat162float(early_res[j]);
      y[size_t(rank + j * kCluster) * ldy + col0 + n] = __float2bfloat16_rn(r);
    }
    return;
  }
  if (slices == 1) return;

  // ---------------- no cluster: the last slice to arrive adds the slabs ----------------
  if (tid == 0) {
    __threadfence();
    last_flag = atomicAdd(&counters[blockIdx.x], 1u) == slices - 1;
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  if (warp < 4) {
    const unsigned nq = n0 + lane * 4;
    const size_t slab = size_t(M) * Np / 4;
    bf16* yp = y + col0;
    const bf16* rp = residual + col0;
    const float* pp = partial + col0;
    if (slices <= 4) tc::finish_rows<8, 4>(pp, slab, slices, warp, 4, M, 0, nq, N, Np, yp, ldy, bias, rp, 1.f, flags);
    else if (slices <= 8) tc::finish_rows<4, 8>(pp, slab, slices, warp, 4, M, 0, nq, N, Np, yp, ldy, bias, rp, 1.f, flags);
    else tc::finish_rows<2, 16>(pp, slab, slices, warp, 4, M, 0, nq, N, Np, yp, ldy, bias, rp, 1.f, flags);
  }
  if (tid == 0) counters[blockIdx.x] = 0;
}

}  // namespace tcs

// grid = (sum of N_i / 128, 1, slices), block = 160; N_i multiples of 128, K a multiple of 64, M <= 32,
// slices * kb_per_slice >= K / 64, slices <= 16.  Dynamic shared memory = kb_per_slice * 20480 + 1024.
extern "C" __global__ void __launch_bounds__(tcs::kThreads, 2)
agi_gemm_tcs_bf16(const bf16* x, const bf16* w0, const bf16* w1, const bf16* w2, bf16* y, const bf16* b0, const bf16* b1,
                  const bf16* b2, const bf16* residual, float* partial, unsigned* counters, unsigned* status, unsigned M,
                  unsigned N0, unsigned N1, unsigned N2, unsigned K, unsigned ldx, unsigned ldy, unsigned flags,
                  unsigned kb_per_slice) {
  const tcs::Parts parts = {{reinterpret_cast<const uint8_t*>(w0), reinterpret_cast<const uint8_t*>(w1),
                             reinterpret_cast<const uint8_t*>(w2)}, {b0, b1, b2}, {N0, N1, N2}};
  tcs::body<1>(x, parts, y, residual, partial, counters, status, M, K, ldx, ldy, flags, kb_per_slice);
}

// Cluster variants: grid = (tiles, G, C) with cluster (1, 1, C); K is cut into G * C slices.  G <= 4.
// Dynamic shared memory = kb_per_slice * 20480 + 1024 + C * ceil(32 / C) * 512.
#define AGI_TCS_CLUSTER_KERNEL(C)                                                                                      \
  extern "C" __global__ void __cluster_dims__(1, 1, C) __launch_bounds__(tcs::kThreads, 3)                             \
  agi_gemm_tcs_bf16_c##C(const bf16* x, const bf16* w0, const bf16* w1, const bf16* w2, bf16* y, const bf16* b0,       \
                         const bf16* b1, const bf16* b2, const bf16* residual, float* partial, unsigned* counters,    \
                         unsigned* status, unsigned M, unsigned N0, unsigned N1, unsigned N2, unsigned K,             \
                         unsigned ldx, unsigned ldy, unsigned flags, unsigned kb_per_slice) {                         \
    const tcs::Parts parts = {{reinterpret_cast<const uint8_t*>(w0), reinterpret_cast<const uint8_t*>(w1),            \
                               reinterpret_cast<const uint8_t*>(w2)}, {b0, b1, b2}, {N0, N1, N2}};                     \
    tcs::body<C>(x, parts, y, residual, partial, counters, status, M, K, ldx, ldy, flags, kb_per_slice);              \
  }
AGI_TCS_CLUSTER_KERNEL(2)
AGI_TCS_CLUSTER_KERNEL(3)
AGI_TCS_CLUSTER_KERNEL(4)
AGI_TCS_CLUSTER_KERNEL(6)
AGI_TCS_CLUSTER_KERNEL(8)
#undef AGI_TCS_CLUSTER_KERNEL

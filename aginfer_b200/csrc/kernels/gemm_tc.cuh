// Tensor-core GEMM for sm_100a: Y[M, N] = epilogue(X[M, K] . W[N, K]^T), bf16 or E4M3 operands,
// fp32 accumulation in tensor memory (TMEM) with tcgen05.mma.
//
// Orientation.  The weight matrix is the MMA's A operand: a CTA owns 128 consecutive rows of
// W (128 output features) and `TN` tokens, TN a multiple of 16 up to 256.  The accumulator
// tile D[128 x TN] has one output feature per TMEM lane and one token per column.  This way
// a batch-1 action head (17 or 50 tokens) and a 1024-token prefill run the same code: few
// tokens only make the tile narrower, the 128-row weight stream per CTA stays the same.
//
// Data movement.  W is checkpoint bytes, [N, K] row-major, i.e. already K-major.  The kernel
// ABI passes only pointers and scalars, so no tensor-map object can be handed to the kernel;
// tiles are brought in with 16-byte cp.async copies into the 128-byte-swizzled K-major
// layout tcgen05 reads (row r, 16-byte chunk c stored at chunk c ^ (r & 7)).  Four producer
// warps fill a ring of `stages` slots; one thread issues the MMAs; a slot is released by
// tcgen05.commit.  After the main loop the producer warps become the epilogue: each reads
// its 32 TMEM lanes with tcgen05.ld and writes bf16 (or fp32) rows.
//
// Split-K.  grid.z > 1 slices K.  Each slice stores its partial tile into its own fp32 slab
// of a scratch buffer laid out [slice][M][N]; a per-tile arrival counter elects the last slice
// to arrive, which adds the slabs in slice order (so the result does not depend on arrival
// order), applies the epilogue, writes Y and resets the counter.  Nobody spins on another CTA.
//
// Every wait on an mbarrier is bounded; on expiry the kernel records a code in `status`
// and carries on with whatever data it has, so a logic error shows up as a status word and
// wrong numbers, never as a hang.
#pragma once

#include "common.cuh"
#include "gemm_simt.cuh"  // gemm_store

namespace tc {

constexpr unsigned kTileN = 128;          // weight rows per CTA (MMA M)
constexpr unsigned kRowBytes = 128;       // K bytes per row per stage (one swizzle atom)
constexpr unsigned kATileBytes = kTileN * kRowBytes;
constexpr unsigned kProducers = 128;
constexpr unsigned kThreads = 160;        // 4 producer/epilogue warps + 1 MMA warp
constexpr unsigned kMaxStages = 12;
constexpr int kLag = 2;                   // a stage is published two commits after it was issued
constexpr unsigned kSpinLimit = 1u << 22;

enum Status : unsigned { kOkStatus = 0, kTimeoutFull = 0x100, kTimeoutEmpty = 0x200, kTimeoutAccum = 0x300 };

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
  asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned long long* bar, unsigned parity) {
  unsigned done;
  asm volatile(
      "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
// Bounded wait; on expiry writes `code` to the status word once and returns false.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, unsigned* status, unsigned code) {
  for (unsigned spin = 0; spin < kSpinLimit; ++spin) {
    if (mbar_test(bar, parity)) return true;
    if (spin > 64) __nanosleep(32);
  }
  atomicCAS(status, 0u, code);
  return false;
}

__device__ __forceinline__ void cp_async_16(unsigned dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Make this thread's completed shared-memory writes visible to the tensor core's (async proxy) reads.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bulk (TMA, no tensor map) copy of a contiguous run of global memory into shared memory; completion is
// counted in bytes on an mbarrier armed with expect_bytes.
__device__ __forceinline__ void bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void expect_bytes(unsigned long long* bar, unsigned bytes) {
  asm volatile("{ .reg .b64 t; mbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1; }" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tmem_alloc(unsigned* slot, unsigned columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(columns) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(unsigned base, unsigned columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned long long* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows 128 B apart, 8-row groups
// 1024 B apart (stride byte offset), leading byte offset 1 (unused for swizzled K-major),
// descriptor version 1, layout type 2 (SWIZZLE_128B) in bits 61-63.
__device__ __forceinline__ unsigned long long smem_descriptor(unsigned addr) {
  return (unsigned long long)((addr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, A and B both K-major, M = 128, N = tokens.
// kind::f16 -> a/b format 1 (bf16); kind::f8f6f4 -> a/b format 0 (E4M3).
template <bool kFp8>
__device__ __forceinline__ unsigned instr_descriptor(unsigned tokens) {
  const unsigned fmt = kFp8 ? 0u : 1u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((tokens >> 3) << 17) | ((kTileN >> 4) << 24);
}
template <bool kFp8>
__device__ __forceinline__ void mma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                    unsigned accumulate) {
  if (kFp8) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_load16(unsigned addr, float v[16]) {
  unsigned r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Thread-block cluster helpers (split-K slices of one output tile form a cluster along grid z).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync() {
  cluster_arrive();
  cluster_wait();
}
// Address of `local_smem_addr` in the shared memory of cluster rank `rank`.
__device__ __forceinline__ unsigned peer_smem(unsigned local_smem_addr, unsigned rank) {
  unsigned remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_smem_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ void store_peer_f32(unsigned remote_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr), "f"(v) : "memory");
}

__device__ __forceinline__ unsigned tmem_columns_for(unsigned tokens) {
  unsigned c = 32;
  while (c < tokens) c <<= 1;
  return c;
}

// Epilogue of one thread for 16 consecutive tokens of its output feature: scale, bias, activation,
// residual, store.  Written as whole-array passes (flag tests once per 16 values, loads before
// uses) because only four warps run it: every dependent instruction chain is paid in full.
template <bool kOutF32, bool kFull>
__device__ __forceinline__ void store_tokens16(const float v[16], unsigned count, void* y, const bf16* residual,
                                               size_t offset, unsigned ldy, float alpha, float bias_v, unsigned flags) {
  float r[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) r[i] = fmaf(v[i], alpha, bias_v);
  const unsigned act = flags & kFlagActMask;
  if (act == kActGeluTanh) {
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = gelu_tanh(r[i]);
  } else if (act == kActSilu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = silu(r[i]);
  } else if (act == kActRelu) {
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = fmaxf(r[i], 0.f);
  }
  if (flags & kFlagResidual) {
    bf16 res[16];
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (kFull || unsigned(i) < count) res[i] = residual[offset + size_t(i) * ldy];
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (kFull || unsigned(i) < count) r[i] += __bfloat162float(res[i]);
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    if (!kFull && unsigned(i) >= count) continue;
    if (kOutF32) static_cast<float*>(y)[offset + size_t(i) * ldy] = r[i];
    else static_cast<bf16*>(y)[offset + size_t(i) * ldy] = __float2bfloat16_rn(r[i]);
  }
}

// Split-K finish of one thread: four consecutive output features of one token.  Vector loads and stores
// when the row pitch keeps them aligned, the scalar path otherwise (and at the ragged edge of N).
__device__ __forceinline__ void store_features4(const float t4[4], unsigned m, unsigned n, unsigned N, void* y,
                                                unsigned ldy, const bf16* bias, const bf16* residual, float alpha,
                                                unsigned flags) {
  const size_t at = size_t(m) * ldy + n;
  const bool aligned = ((reinterpret_cast<size_t>(y) | reinterpret_cast<size_t>(bias) |
                         reinterpret_cast<size_t>(residual)) & 15) == 0;  // unused pointers are arena-aligned
  if (n + 3 < N && (ldy & 3) == 0 && aligned) {
    float r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = t4[j] * alpha;
    if (flags & kFlagBias) {
      const uint2 b = *reinterpret_cast<const uint2*>(bias + n);
      const float2 b01 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&b.x));
      const float2 b23 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&b.y));
      r[0] += b01.x; r[1] += b01.y; r[2] += b23.x; r[3] += b23.y;
    }
    const unsigned act = flags & kFlagActMask;
    if (act != 0) {
#pragma unroll
      for (int j = 0; j < 4; ++j) r[j] = apply_activation(r[j], flags);
    }
    if (flags & kFlagResidual) {
      const uint2 q = *reinterpret_cast<const uint2*>(residual + at);
      const float2 q01 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&q.x));
      const float2 q23 = __bfloat1622float2(*reinterpret_cast<const bf162*>(&q.y));
      r[0] += q01.x; r[1] += q01.y; r[2] += q23.x; r[3] += q23.y;
    }
    if (flags & kFlagOutF32) {
      *reinterpret_cast<float4*>(static_cast<float*>(y) + at) = make_float4(r[0], r[1], r[2], r[3]);
    } else {
      const bf162 lo = __floats2bfloat162_rn(r[0], r[1]), hi = __floats2bfloat162_rn(r[2], r[3]);
      uint2 out;
      out.x = *reinterpret_cast<const unsigned*>(&lo);
      out.y = *reinterpret_cast<const unsigned*>(&hi);
      *reinterpret_cast<uint2*>(static_cast<bf16*>(y) + at) = out;
    }
    return;
  }
#pragma unroll
  for (unsigned j = 0; j < 4; ++j)
    if (n + j < N) gemm_store(t4[j], m, n + j, y, ldy, bias, residual, alpha, flags);
}

// grid = (ceil(N / 128), ceil(M / TN), splits), block = 160 threads,
// dynamic shared memory = stages * (16384 + TN * 128) + 1024.
// Split-K finish of one warp: token rows first, first + stride, ... of a tile, lane l owning four output features.
// ROWS rows are summed per pass, over at most SLICES slabs each: every load of a pass is issued before the first
// addition, so a pass costs one L2 round trip.  ROWS * SLICES = 32 float4 in flight per thread.
template <int ROWS, int SLICES>
__device__ __forceinline__ void finish_rows(const float* partial, size_t slab, unsigned splits, unsigned first,
                                            unsigned stride, unsigned rows, unsigned m0, unsigned n, unsigned N,
                                            unsigned Np, void* y, unsigned ldy, const bf16* bias, const bf16* residual,
                                            float alpha, unsigned flags) {
  for (unsigned i0 = first; i0 < rows; i0 += ROWS * stride) {
    float4 part[ROWS][SLICES];
#pragma unroll
    for (int b = 0; b < ROWS; ++b) {
      const unsigned i = i0 + b * stride;
      if (i >= rows) continue;
      const float4* cell = reinterpret_cast<const float4*>(partial + size_t(m0 + i) * Np + n);
#pragma unroll
      for (int z = 0; z < SLICES; ++z)
        if (unsigned(z) < splits) part[b][z] = __ldcg(cell + z * slab);
    }
#pragma unroll
    for (int b = 0; b < ROWS; ++b) {
      const unsigned i = i0 + b * stride;
      if (i >= rows) continue;
      float4 total = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int z = 0; z < SLICES; ++z)   // slice order: the sum does not depend on which CTA arrived when
        if (unsigned(z) < splits) {
          total.x += part[b][z].x; total.y += part[b][z].y; total.z += part[b][z].z; total.w += part[b][z].w;
        }
      const float t4[4] = {total.x, total.y, total.z, total.w};
      store_features4(t4, m0 + i, n, N, y, ldy, bias, residual, alpha, flags);
    }
  }
}

// kPacked: both operands are stored "K-block-major, swizzled" (see recipes/layout.py): the 128-byte K block kb
// of row r lives at ((kb * rows_padded + r) * 128) with its 16-byte chunk c at position c ^ (r & 7), i.e. the
// image of the shared-memory tile.  A ring slot is then filled by two bulk copies (16 KB of weights, TN * 128 B
// of activations) issued by one thread, instead of 16-byte copies by 128 threads; `ldx` carries the padded
// row count of the activation matrix.
template <bool kFp8, int kCluster = 1, bool kPacked = false>
__device__ __forceinline__ void gemm_body(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias,
                                          const bf16* residual, const float* scale_a, const float* scale_w,
                                          float* partial, unsigned* counters, unsigned* status, unsigned M,
                                          unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags,
                                          unsigned TN, unsigned stages, unsigned tile_x = 0xffffffffu) {
  extern __shared__ unsigned char dynamic_smem[];
  __shared__ __align__(8) unsigned long long full_bar[kMaxStages];
  __shared__ __align__(8) unsigned long long empty_bar[kMaxStages];
  __shared__ __align__(8) unsigned long long accum_bar;
  __shared__ unsigned tmem_slot;
  __shared__ unsigned last_flag;

  const unsigned tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const unsigned elem = kFp8 ? 1u : 2u;
  if (tile_x == 0xffffffffu) tile_x = blockIdx.x;  // batched launches pass the tile index inside their matrix
  const unsigned n0 = tile_x * kTileN, m0 = blockIdx.y * TN;
  const unsigned splits = gridDim.z, split = blockIdx.z;
  const unsigned k_blocks_total = (K * elem) / kRowBytes;
  const unsigned per_split = (k_blocks_total + splits - 1) / splits;
  const unsigned kb_begin = min(split * per_split, k_blocks_total);
  const unsigned kb_end = min(kb_begin + per_split, k_blocks_total);
  const unsigned nkb = kb_end - kb_begin;
  const unsigned stage_bytes = kATileBytes + TN * kRowBytes;
  const unsigned ring = (smem_u32(dynamic_smem) + 1023u) & ~1023u;  // tiles need 1024-byte alignment
  const unsigned columns = tmem_columns_for(TN);
  // Cluster mode: [slice][token / kCluster][128 rows] fp32 gather buffer behind the ring.
  const unsigned gather_cols = (TN + kCluster - 1) / kCluster;
  const unsigned gather_base = ring + stages * stage_bytes;
  const unsigned Np = gridDim.x * kTileN;  // row stride of the split-K slabs: N rounded up to whole tiles
  if (stages > kMaxStages) stages = kMaxStages;

  if (tid == 0) {
    for (unsigned s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], kPacked ? 1 : kProducers);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&accum_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 4) tmem_alloc(&tmem_slot, columns);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const unsigned tmem_base = tmem_slot;
  // Cluster split-K: every slice must be running (its shared memory live) before anyone writes into it.
  // Arrive now, wait only just before the first remote store: by then the barrier has long completed.
  if (kCluster > 1) cluster_arrive();

  // Weights do not depend on the previous kernel: the weight tiles of the first ring slots are requested
  // before the grid-dependency wait (they join the first commit group below).
  const size_t w_row_bytes = size_t(K) * elem, x_row_bytes = size_t(ldx) * elem;
  const unsigned early = min(stages, nkb);
  // A producer thread copies chunk c of rows r0, r0 + 16, ...: the swizzled destination differs from row
  // to row by a constant (16 rows = 2048 B, and r & 7 does not change), the source by 16 row pitches, so
  // one copy costs an add, not an address computation.  Rows past the matrix are skipped: what the
  // tensor core reads there only reaches accumulator rows / columns that are never stored.
  const unsigned r0 = tid >> 3, chunk = tid & 7;
  const unsigned dst_off = r0 * kRowBytes + ((chunk ^ (r0 & 7)) << 4);
  const unsigned a_rows = n0 + r0 < N ? (min(kTileN, N - n0) - r0 + 15) / 16 : 0;
  const unsigned b_rows = (m0 + r0 < M && r0 < TN) ? (min(TN, M - m0) - r0 + 15) / 16 : 0;
  const uint8_t* w_src = w + size_t(n0 + r0) * w_row_bytes + size_t(kb_begin) * kRowBytes + (chunk << 4);
  const uint8_t* x_src = x + size_t(m0 + r0) * x_row_bytes + size_t(kb_begin) * kRowBytes + (chunk << 4);
  const size_t w_step = 16 * w_row_bytes, x_step = 16 * x_row_bytes;
  auto load_weights = [&](unsigned i) {
    const uint8_t* src = w_src + size_t(i) * kRowBytes;
    const unsigned dst = ring + (i % stages) * stage_bytes + dst_off;
#pragma unroll
    for (unsigned j = 0; j < 8; ++j)
      if (j < a_rows) cp_async_16(dst + j * 2048, src + j * w_step);
  };
  // packed operands: tile (first row r0, K block kb) is one contiguous run
  const unsigned w_rows_padded = ((N + 255u) / 256u) * 256u;   // packed weights are padded to whole 256-row tiles
  const unsigned b_tile_bytes = TN * kRowBytes;
  auto packed_weights = [&](unsigned i) {
    bulk_copy(ring + (i % stages) * stage_bytes, w + (size_t(kb_begin + i) * w_rows_padded + n0) * kRowBytes, kATileBytes,
              &full_bar[i % stages]);
  };
  auto packed_tokens = [&](unsigned i) {
    bulk_copy(ring + (i % stages) * stage_bytes + kATileBytes, x + (size_t(kb_begin + i) * ldx + m0) * kRowBytes,
              b_tile_bytes, &full_bar[i % stages]);
  };
  if (kPacked) {
    if (tid == 0)
      for (unsigned i = 0; i < early; ++i) {
        expect_bytes(&full_bar[i], kATileBytes + b_tile_bytes);
        packed_weights(i);
      }
  } else if (warp < 4) {
    for (unsigned i = 0; i < early; ++i) load_weights(i);
  }

  grid_dependency_wait();

  if (kPacked && warp < 4) {
    // ---------------- warp 0 is the producer: two bulk copies per ring slot, issued by its lane 0 ----------------
    // (the whole warp walks the loop so that it reaches the epilogue converged; warps 1-3 go straight there)
    if (warp == 0) {
      if (lane == 0)
        for (unsigned i = 0; i < early; ++i) packed_tokens(i);
      for (unsigned i = early; i < nkb; ++i) {
        const unsigned s = i % stages;
        mbar_wait(&empty_bar[s], (i / stages - 1) & 1, status, kTimeoutEmpty | s);
        if (lane == 0) {
          expect_bytes(&full_bar[s], kATileBytes + b_tile_bytes);
          packed_weights(i);
          packed_tokens(i);
        }
        __syncwarp();
      }
    }
  } else if (warp < 4) {
    // ---------------- producers ----------------
    for (unsigned i = 0; i < nkb + kLag; ++i) {
      if (i < nkb) {
        const unsigned s = i % stages, round = i / stages;
        if (round > 0) mbar_wait(&empty_bar[s], (round - 1) & 1, status, kTimeoutEmpty | s);
        if (i >= early) load_weights(i);
        const uint8_t* src = x_src + size_t(i) * kRowBytes;
        const unsigned dst = ring + s * stage_bytes + kATileBytes + dst_off;
#pragma unroll
        for (unsigned j = 0; j < 16; ++j)
          if (j < b_rows) cp_async_16(dst + j * 2048, src + j * x_step);
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
        const unsigned a_base = ring + s * stage_bytes, b_base = a_base + kATileBytes;
        const unsigned long long a_desc = smem_descriptor(a_base), b_desc = smem_descriptor(b_base);
#pragma unroll
        for (unsigned k = 0; k < 4; ++k)  // 4 x 32 bytes of K per stage; +2 advances the start address by 32 B
          mma<kFp8>(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (i | k) != 0);
        tc_commit(&empty_bar[s]);
      }
      __syncwarp();
    }
    if (lane == 0) tc_commit(&accum_bar);
    __syncwarp();
    if (kCluster > 1) cluster_wait();  // every thread pairs its early arrive with one wait
  }

  // ---------------- epilogue (warps 0-3: TMEM lanes 32 * warp ... +31) ----------------
  if (warp < 4) {
    if (nkb > 0) mbar_wait(&accum_bar, 0, status, kTimeoutAccum);
    tc_fence_after();
    const unsigned n = n0 + warp * 32 + lane;
    const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
    const float bias_v = ((flags & kFlagBias) && n < N) ? __bfloat162float(bias[n]) : 0.f;
    const unsigned lane_addr = tmem_base + ((warp * 32u) << 16);
    if (kCluster > 1) cluster_wait();  // peers are running: their gather buffers may be written
    for (unsigned c0 = 0; c0 < TN; c0 += 16) {
      if (kCluster > 1 && m0 + c0 >= M) break;  // token columns past M carry nothing
      float v[16];
      if (nkb > 0) {
        tmem_load16(lane_addr + c0, v);
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = 0.f;
      }
      if (kCluster == 1 && splits == 1) {
        // direct store: bias was fetched once per thread, flags are tested once per 16 tokens
        if (n < N && m0 + c0 < M) {
          const unsigned count = min(16u, M - (m0 + c0));
          const size_t offset = size_t(m0 + c0) * ldy + n;
          const bool f32 = (flags & kFlagOutF32) != 0;
          if (count == 16) {
            if (f32) store_tokens16<true, true>(v, 16, y, residual, offset, ldy, alpha, bias_v, flags);
            else store_tokens16<false, true>(v, 16, y, residual, offset, ldy, alpha, bias_v, flags);
          } else {
            if (f32) store_tokens16<true, false>(v, count, y, residual, offset, ldy, alpha, bias_v, flags);
            else store_tokens16<false, false>(v, count, y, residual, offset, ldy, alpha, bias_v, flags);
          }
        }
      } else if (kCluster == 1) {
        // split-K slab: one base address per 16 tokens, rows Np apart
        if (n < N && m0 + c0 < M) {
          const unsigned count = min(16u, M - (m0 + c0));
          float* cell = partial + (size_t(split) * M + m0 + c0) * Np + n;
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (unsigned(i) < count) __stcg(cell + size_t(i) * Np, v[i]);
        }
      } else if (n < N) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const unsigned m = m0 + c0 + i;
          if (m >= M) continue;
          if (kCluster > 1) {
            // token m is finished by cluster rank m % kCluster: send it this slice's partial sum,
            // filed under [this rank][m / kCluster][row of W]
            const unsigned c = c0 + i, owner = c % kCluster;
            const unsigned cell = gather_base + (((split * gather_cols) + c / kCluster) * kTileN + warp * 32 + lane) * 4;
            store_peer_f32(peer_smem(cell, owner), v[i]);
          }
        }
      }
    }
    if (kCluster == 1 && splits > 1) __threadfence();  // partial sums ordered before this CTA's arrival count
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_free(tmem_base, columns);
  }
  if (kCluster > 1) {
    // ---------------- split-K inside a cluster: partial sums travelled through distributed shared memory ----
    // This rank finishes tokens split, split + C, ...: their bias and residual values are fetched while the
    // cluster barrier completes.
    constexpr int kMine = (64 + kCluster - 1) / kCluster;   // at most 64 tokens in cluster mode
    const unsigned n = n0 + warp * 32 + lane;
    const unsigned my_tokens = warp < 4 && n < N && split < min(TN, M - m0)
                                   ? (min(TN, M - m0) - split + kCluster - 1) / kCluster : 0;
    bf16 early_bias = __float2bfloat16_rn(0.f), early_res[kMine];
    if (my_tokens != 0 && (flags & kFlagBias)) early_bias = bias[n];
#pragma unroll
    for (int j = 0; j < kMine; ++j)
      if (unsigned(j) < my_tokens && (flags & kFlagResidual))
        early_res[j] = residual[size_t(m0 + split + j * kCluster) * ldy + n];
    cluster_arrive();
    cluster_wait();  // every slice's stores into this CTA's gather buffer are complete and visible
    if (my_tokens != 0) {
      const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
      const float* mine = reinterpret_cast<const float*>(dynamic_smem + (gather_base - smem_u32(dynamic_smem)));
#pragma unroll
      for (int j = 0; j < kMine; ++j) {
        if (unsigned(j) >= my_tokens) break;
        float total = 0.f;
#pragma unroll
        for (int z = 0; z < kCluster; ++z) total += mine[((z * gather_cols) + j) * kTileN + warp * 32 + lane];  // slice order
        float r = total * alpha;
        if (flags & kFlagBias) r += __bfloat162float(early_bias);
        r = apply_activation(r, flags);
        if (flags & kFlagResidual) r += __bfloat162float(early_res[j]);
        const size_t at = size_t(m0 + split + j * kCluster) * ldy + n;
        if (flags & kFlagOutF32) static_cast<float*>(y)[at] = r;
        else static_cast<bf16*>(y)[at] = __float2bfloat16_rn(r);
      }
    }
    return;
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
  if (warp < 4) {
    // Warp w reduces token rows w, w + 4, ...; lane l owns output features n0 + 4l .. 4l + 3.  The
    // loads of one row's slabs are independent, so they are all in flight together; the additions
    // run in slice order, which makes the sum independent of which CTA arrived when.
    const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
    const unsigned n = n0 + lane * 4;
    const unsigned rows = min(TN, M - m0);
    const size_t slab = size_t(M) * Np / 4;
    if (splits <= 2) finish_rows<16, 2>(partial, slab, splits, warp, 4, rows, m0, n, N, Np, y, ldy, bias, residual, alpha, flags);
    else if (splits <= 4) finish_rows<8, 4>(partial, slab, splits, warp, 4, rows, m0, n, N, Np, y, ldy, bias, residual, alpha, flags);
    else if (splits <= 8) finish_rows<4, 8>(partial, slab, splits, warp, 4, rows, m0, n, N, Np, y, ldy, bias, residual, alpha, flags);
    else finish_rows<2, 16>(partial, slab, splits, warp, 4, rows, m0, n, N, Np, y, ldy, bias, residual, alpha, flags);
  }
  if (tid == 0) counters[tile] = 0;
}

}  // namespace tc

// Cluster split-K variants: grid.z = cluster size = number of K slices (2, 3, 4, 6 or 8); partial sums are
// exchanged through distributed shared memory, so `partial` and `counters` are unused.  For up to 64 tokens.
// Dynamic shared memory = stages * (16384 + TN * 128) + 1024 + C * ceil(TN / C) * 512.
#define AGI_TC_CLUSTER_KERNEL(NAME, TYPE, FP8, C)                                                                     \
  extern "C" __global__ void __cluster_dims__(1, 1, C) __launch_bounds__(tc::kThreads, 1)                            \
  NAME(const TYPE* x, const TYPE* w, void* y, const bf16* bias, const bf16* residual, const float* scale_a,         \
       const float* scale_w, float* partial, unsigned* counters, unsigned* status, unsigned M, unsigned N,          \
       unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN, unsigned stages) {                      \
    tc::gemm_body<FP8, C>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias,         \
                          residual, scale_a, scale_w, partial, counters, status, M, N, K, ldx, ldy, flags, TN,      \
                          stages);                                                                                   \
  }
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_bf16_c2, bf16, false, 2)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_bf16_c3, bf16, false, 3)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_bf16_c4, bf16, false, 4)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_bf16_c6, bf16, false, 6)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_bf16_c8, bf16, false, 8)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_e4m3_c2, uint8_t, true, 2)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_e4m3_c4, uint8_t, true, 4)
AGI_TC_CLUSTER_KERNEL(agi_gemm_tc_e4m3_c8, uint8_t, true, 8)
#undef AGI_TC_CLUSTER_KERNEL

// Up to 16 independent GEMMs that share the activation matrix (e.g. the K and V projections of every
// cross-attention block over the same context tokens) as ONE launch: grid.x = segments * ceil(N / 128);
// segment s multiplies by w[s], adds bias[s] and writes y + s * seg_stride elements.  No split-K.
extern "C" __global__ void __launch_bounds__(tc::kThreads, 1)
agi_gemm_tc_bf16_x16(const bf16* x, void* y, unsigned* status, unsigned M, unsigned N, unsigned K, unsigned ldx,
                     unsigned ldy, unsigned flags, unsigned TN, unsigned stages, unsigned seg_stride,
                     const bf16* w0, const bf16* w1, const bf16* w2, const bf16* w3, const bf16* w4, const bf16* w5,
                     const bf16* w6, const bf16* w7, const bf16* w8, const bf16* w9, const bf16* w10,
                     const bf16* w11, const bf16* w12, const bf16* w13, const bf16* w14, const bf16* w15,
                     const bf16* b0, const bf16* b1, const bf16* b2, const bf16* b3, const bf16* b4, const bf16* b5,
                     const bf16* b6, const bf16* b7, const bf16* b8, const bf16* b9, const bf16* b10,
                     const bf16* b11, const bf16* b12, const bf16* b13, const bf16* b14, const bf16* b15) {
  const unsigned tiles = (N + tc::kTileN - 1) / tc::kTileN;
  const unsigned seg = blockIdx.x / tiles;
  const bf16 *w, *b;
  switch (seg) {
    case 0: w = w0; b = b0; break;    case 1: w = w1; b = b1; break;    case 2: w = w2; b = b2; break;
    case 3: w = w3; b = b3; break;    case 4: w = w4; b = b4; break;    case 5: w = w5; b = b5; break;
    case 6: w = w6; b = b6; break;    case 7: w = w7; b = b7; break;    case 8: w = w8; b = b8; break;
    case 9: w = w9; b = b9; break;    case 10: w = w10; b = b10; break; case 11: w = w11; b = b11; break;
    case 12: w = w12; b = b12; break; case 13: w = w13; b = b13; break; case 14: w = w14; b = b14; break;
    default: w = w15; b = b15; break;
  }
  tc::gemm_body<false>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w),
                       static_cast<bf16*>(y) + size_t(seg) * seg_stride, b, b, nullptr, nullptr, nullptr, nullptr, status,
                       M, N, K, ldx, ldy, flags, TN, stages, blockIdx.x % tiles);
}

// Up to three GEMMs over the same activation matrix as ONE launch (Q | K | V, gate | up): part i multiplies
// by w_i [N_i, K], scales by scale_a * sw_i, adds bias_i and writes y_i with row pitch ldy_i.  The parts'
// 128-row tiles are laid end to end along grid.x = sum of ceil(N_i / 128); no split-K.
#define AGI_TC_GROUP_KERNEL(NAME, TYPE, FP8, PACKED)                                                                  \
  extern "C" __global__ void __launch_bounds__(tc::kThreads, 1)                                                      \
  NAME(const TYPE* x, const float* scale_a, unsigned* status, unsigned M, unsigned K, unsigned ldx, unsigned flags,   \
       unsigned TN, unsigned stages, const TYPE* w0, const bf16* bias0, const float* sw0, void* y0, unsigned N0,      \
       unsigned ldy0, const TYPE* w1, const bf16* bias1, const float* sw1, void* y1, unsigned N1, unsigned ldy1,      \
       const TYPE* w2, const bf16* bias2, const float* sw2, void* y2, unsigned N2, unsigned ldy2) {                   \
    const unsigned t0 = (N0 + tc::kTileN - 1) / tc::kTileN, t1 = (N1 + tc::kTileN - 1) / tc::kTileN;                  \
    const TYPE* w = w0;                                                                                               \
    const bf16* bias = bias0;                                                                                         \
    const float* sw = sw0;                                                                                            \
    void* y = y0;                                                                                                     \
    unsigned N = N0, ldy = ldy0, tile = blockIdx.x;                                                                   \
    if (tile >= t0 + t1) {                                                                                            \
      w = w2; bias = bias2; sw = sw2; y = y2; N = N2; ldy = ldy2; tile -= t0 + t1;                                    \
    } else if (tile >= t0) {                                                                                          \
      w = w1; bias = bias1; sw = sw1; y = y1; N = N1; ldy = ldy1; tile -= t0;                                         \
    }                                                                                                                 \
    tc::gemm_body<FP8, 1, PACKED>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias,  \
                                  bias, scale_a, sw, nullptr, nullptr, status, M, N, K, ldx, ldy, flags, TN, stages,  \
                                  tile);                                                                              \
  }
AGI_TC_GROUP_KERNEL(agi_gemm_tc_bf16_x3, bf16, false, false)
AGI_TC_GROUP_KERNEL(agi_gemm_tc_e4m3_x3, uint8_t, true, false)
// the same over packed operands (bulk-copy producers; ldx = padded row count of the activation matrix)
AGI_TC_GROUP_KERNEL(agi_gemm_tcp_e4m3_x3, uint8_t, true, true)
#undef AGI_TC_GROUP_KERNEL

// The grouped launch with K slices in a thread-block cluster (up to 64 tokens, bf16): grid = (sum of ceil(N_i / 128),
// 1, C), cluster (1, 1, C); the slices of a tile exchange partial sums through distributed shared memory as in
// agi_gemm_tc_bf16_c*.  Three small projections of one layer (queries | keys | values, gate | up) become one launch.
// Dynamic shared memory = stages * (16384 + TN * 128) + 1024 + C * ceil(TN / C) * 512.
#define AGI_TC_GROUP_CLUSTER_KERNEL(NAME, C)                                                                          \
  extern "C" __global__ void __cluster_dims__(1, 1, C) __launch_bounds__(tc::kThreads, 1)                            \
  NAME(const bf16* x, const float* scale_a, unsigned* status, unsigned M, unsigned K, unsigned ldx, unsigned flags,   \
       unsigned TN, unsigned stages, const bf16* w0, const bf16* bias0, const float* sw0, void* y0, unsigned N0,      \
       unsigned ldy0, const bf16* w1, const bf16* bias1, const float* sw1, void* y1, unsigned N1, unsigned ldy1,      \
       const bf16* w2, const bf16* bias2, const float* sw2, void* y2, unsigned N2, unsigned ldy2) {                   \
    const unsigned t0 = (N0 + tc::kTileN - 1) / tc::kTileN, t1 = (N1 + tc::kTileN - 1) / tc::kTileN;                  \
    const bf16* w = w0;                                                                                               \
    const bf16* bias = bias0;                                                                                         \
    void* y = y0;                                                                                                     \
    unsigned N = N0, ldy = ldy0, tile = blockIdx.x;                                                                   \
    if (tile >= t0 + t1) {                                                                                            \
      w = w2; bias = bias2; y = y2; N = N2; ldy = ldy2; tile -= t0 + t1;                                              \
    } else if (tile >= t0) {                                                                                          \
      w = w1; bias = bias1; y = y1; N = N1; ldy = ldy1; tile -= t0;                                                   \
    }                                                                                                                 \
    tc::gemm_body<false, C, false>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias, \
                                   bias, nullptr, nullptr, nullptr, nullptr, status, M, N, K, ldx, ldy, flags, TN,    \
                                   stages, tile);                                                                     \
  }
AGI_TC_GROUP_CLUSTER_KERNEL(agi_gemm_tc_bf16_x3_c2, 2)
AGI_TC_GROUP_CLUSTER_KERNEL(agi_gemm_tc_bf16_x3_c4, 4)
AGI_TC_GROUP_CLUSTER_KERNEL(agi_gemm_tc_bf16_x3_c8, 8)
#undef AGI_TC_GROUP_CLUSTER_KERNEL

// Single GEMM over packed operands, split-K slabs as in agi_gemm_tc_*.
#define AGI_TC_PACKED_KERNEL(NAME, TYPE, FP8)                                                                         \
  extern "C" __global__ void __launch_bounds__(tc::kThreads, 1)                                                      \
  NAME(const TYPE* x, const TYPE* w, void* y, const bf16* bias, const bf16* residual, const float* scale_a,          \
       const float* scale_w, float* partial, unsigned* counters, unsigned* status, unsigned M, unsigned N,           \
       unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN, unsigned stages) {                       \
    tc::gemm_body<FP8, 1, true>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias,    \
                                residual, scale_a, scale_w, partial, counters, status, M, N, K, ldx, ldy, flags, TN,  \
                                stages);                                                                              \
  }
AGI_TC_PACKED_KERNEL(agi_gemm_tcp_e4m3, uint8_t, true)
#undef AGI_TC_PACKED_KERNEL

extern "C" __global__ void __launch_bounds__(tc::kThreads, 1)
agi_gemm_tc_bf16(const bf16* x, const bf16* w, void* y, const bf16* bias, const bf16* residual, const float* scale_a,
                 const float* scale_w, float* partial, unsigned* counters, unsigned* status, unsigned M, unsigned N,
                 unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN, unsigned stages) {
  tc::gemm_body<false>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias, residual,
                       scale_a, scale_w, partial, counters, status, M, N, K, ldx, ldy, flags, TN, stages);
}

extern "C" __global__ void __launch_bounds__(tc::kThreads, 1)
agi_gemm_tc_e4m3(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias, const bf16* residual,
                 const float* scale_a, const float* scale_w, float* partial, unsigned* counters, unsigned* status,
                 unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned TN,
                 unsigned stages) {
  tc::gemm_body<true>(x, w, y, bias, residual, scale_a, scale_w, partial, counters, status, M, N, K, ldx, ldy, flags,
                      TN, stages);
}

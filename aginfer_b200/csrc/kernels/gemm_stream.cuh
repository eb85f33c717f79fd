// Weight-streaming skinny GEMM, bulk-copy version: Y[M, N] = epilogue(X[M, K] . W[N, K]^T), M <= 64.
//
// The batch-1 action head is a chain of small dependent GEMMs whose cost is the time to pull
// each weight matrix out of HBM once.  What decides that time is how many bytes an SM has in
// flight and how few dependent round trips a CTA makes, so this kernel moves BOTH operands with
// bulk copies (cp.async.bulk, completing on mbarriers) and computes out of shared memory only:
//
//   * a CTA owns `rows` (8 or 16) output features.  K is cut into chunks of `chunk_windows`
//     64-byte windows; one chunk of the CTA's weight rows plus the same K range of all M
//     activation rows forms a slot (~100 KB); two slots form a ring.  For K <= one chunk (most
//     of the action head) the CTA's entire input is requested at once.
//   * a producer warp issues one bulk copy per row.  Weights never depend on the previous
//     kernel, so the first slots' weight copies are issued BEFORE the grid-dependency wait: under
//     programmatic dependent launch the next layer's weights stream while this layer finishes.
//     Activation copies follow the wait.
//   * four consumer warps walk the chunk in 64-byte windows (warp w takes windows w, w + 4, ...),
//     read weight and activation fragments from shared memory (row pitch = chunk bytes + 16, which
//     spreads the eight rows of a fragment over all banks) and issue warp-level MMAs (m16n8k16
//     bf16 / m16n8k32 E4M3, fp32 accumulate); both operands use the 16-byte chunk's own element
//     order along K.  Partial tiles of the four warps are added through shared memory in warp
//     order; the epilogue applies scale, bias, activation, residual.
//
// Every mbarrier wait is bounded and reports through the status word instead of hanging.
#pragma once

#include "common.cuh"
#include "gemm_simt.cuh"    // gemm_store
#include "gemm_skinny.cuh"  // mma16n8
#include "gemm_tc.cuh"      // cluster barrier and distributed-shared-memory helpers

namespace stream {

// Consumer warps per CTA (plus one producer warp).  Four: the MMA phase is bound by the warp-level MMA
// issue rate of the SM, not by the number of warps, and small CTAs let several share an SM.
__host__ __device__ constexpr int consumer_warps(int) { return 4; }
__host__ __device__ constexpr int threads(int token_tiles) { return (consumer_warps(token_tiles) + 1) * 32; }
constexpr int kSlots = 2;
constexpr unsigned kSpinLimit = 1u << 22;
constexpr unsigned kTimeoutFull = 0x400, kTimeoutEmpty = 0x500;

__device__ __forceinline__ unsigned smem_u32(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void bulk_copy(unsigned dst, const void* src, unsigned bytes, unsigned bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void expect_bytes(unsigned bar, unsigned bytes) {
  asm volatile("{ .reg .b64 t; mbarrier.arrive.expect_tx.shared::cta.b64 t, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void arrive(unsigned bar) {
  asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_done(unsigned bar, unsigned parity) {
  unsigned done;
  asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  return done != 0;
}
__device__ __forceinline__ void bounded_wait(unsigned bar, unsigned parity, unsigned* status, unsigned code) {
  for (unsigned spin = 0; !bar_done(bar, parity); ++spin) {
    if (spin > kSpinLimit) {
      atomicCAS(status, 0u, code);
      return;
    }
    if (spin > 32) __nanosleep(20);
  }
}
__device__ __forceinline__ uint4 lds128(unsigned addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// Optional extras of the fused bf16 family: up to three weight matrices side by side along N (e.g. Q | K | V,
// each a multiple of `rows` wide, written to consecutive column blocks of y) and a LayerNorm prologue.
struct Extra {
  const uint8_t* w1 = nullptr;
  const uint8_t* w2 = nullptr;
  const bf16* bias1 = nullptr;
  const bf16* bias2 = nullptr;
  unsigned n1 = 0, n2 = 0;
  const bf16* ln_scale = nullptr;
  const bf16* ln_shift = nullptr;
  float ln_eps = 0.f;
};

// kSplit > 1: the K range is cut into kSplit slices handled by the CTAs of a thread-block cluster along grid z
// (K is then the length of ONE slice and `ldw` the row pitch of the weight matrix in elements).  Slice s > 0
// sends its 16 x M tile of partial sums to slice 0 through distributed shared memory; slice 0 adds them in slice
// order and runs the epilogue.  A long K thereby becomes kSplit short rings side by side instead of one ring
// that wraps many times, each wrap a round trip to memory.
template <bool kFp8, int NT, bool kLn = false, int kSplit = 1>
__device__ __forceinline__ void body(const uint8_t* x, const uint8_t* w, void* y, const bf16* bias,
                                     const bf16* residual, const float* scale_a, const float* scale_w,
                                     unsigned* status, unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy,
                                     unsigned flags, unsigned rows, unsigned chunk_windows, const Extra extra = Extra(),
                                     unsigned ldw = 0) {
  constexpr int kConsumerWarps = consumer_warps(NT);
  constexpr int kThreads = threads(NT);
  // dynamic shared memory: ring of slots (rows + M rows each), then the warps' partial tiles
  extern __shared__ __align__(128) unsigned char ring[];
  __shared__ __align__(8) unsigned long long full_bar[kSlots], empty_bar[kSlots];

  const unsigned elem = kFp8 ? 1u : 2u;
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned row0 = blockIdx.x * rows;
  const unsigned k_bytes = K * elem;
  const size_t w_pitch = kSplit > 1 ? size_t(ldw) * elem : size_t(k_bytes);
  const unsigned split = kSplit > 1 ? blockIdx.z : 0;
  x += size_t(split) * k_bytes;   // this slice's columns of the activations and (below) of the weights
  const unsigned windows = k_bytes / 64;
  const unsigned chunks = (windows + chunk_windows - 1) / chunk_windows;
  // Slab mode: K is one chunk and both operands are contiguous in global memory, so each arrives with a
  // single bulk copy into unpadded rows (fragment reads then take twice the shared-memory wavefronts,
  // which is cheap; issuing dozens of small bulk copies is not).
  const bool slab = (flags & kFlagSlab) != 0;
  const unsigned pitch = chunk_windows * 64 + (slab ? 0u : 16u);
  constexpr unsigned mod_rows = 0;
  const unsigned slot_bytes = (rows + M + mod_rows) * pitch;
  const unsigned ring_base = smem_u32(ring);
  const unsigned ring_slots = chunks < unsigned(kSlots) ? chunks : unsigned(kSlots);
  const unsigned mp = M | 1u;  // odd pitch of a partial-tile row: rows land in different banks
  float* partial = reinterpret_cast<float*>(ring + ((ring_slots * slot_bytes + 15u) & ~15u));  // [warp][16][mp]
  float* gathered = partial + kConsumerWarps * 16 * mp;   // [slice - 1][rows * M], written by the other slices
  // Which of the side-by-side weight matrices this CTA's rows belong to.
  unsigned seg_rows = N, local0 = row0, col0 = 0;
  const uint8_t* w_seg = w;
  const bf16* bias_seg = bias;
  if (local0 >= seg_rows && extra.n1 != 0) {
    local0 -= seg_rows; col0 += seg_rows; seg_rows = extra.n1; w_seg = extra.w1; bias_seg = extra.bias1;
    if (local0 >= seg_rows && extra.n2 != 0) {
      local0 -= seg_rows; col0 += seg_rows; seg_rows = extra.n2; w_seg = extra.w2; bias_seg = extra.bias2;
    }
  }

  if (threadIdx.x == 0) {
#pragma unroll
    for (int s = 0; s < kSlots; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full_bar[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&empty_bar[s])), "r"(kConsumerWarps));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (kSplit > 1) tc::cluster_arrive();   // "this slice is running": waited for before anyone stores into it

  // Each thread's first output element (i = threadIdx.x): its bias and residual are fetched early, as soon
  // as the previous kernel's results are known to be visible, and used after the reduction.
  float early_bias = 0.f, early_residual = 0.f;
  bool early_valid = false;
  auto fetch_early = [&]() {
    const unsigned i = threadIdx.x;
    if (i < rows * M) {
      const unsigned r = i % rows, m = i / rows;
      if (local0 + r < seg_rows) {
        const unsigned n = col0 + local0 + r;
        if (flags & kFlagBias) early_bias = __bfloat162float(bias_seg[local0 + r]);
        if (flags & kFlagResidual) early_residual = __bfloat162float(residual[size_t(m) * ldy + n]);
        early_valid = true;
      }
    }
  };
  if (warp == kConsumerWarps) {
    // ---------------- producer warp ----------------
    const size_t x_row = size_t(ldx) * elem;
    bool waited = false;
    for (unsigned c = 0; c < chunks; ++c) {
      const unsigned slot = c % kSlots, round = c / kSlots;
      const unsigned first = c * chunk_windows, count = min(chunk_windows, windows - first);
      const unsigned bytes = count * 64;
      const unsigned base = ring_base + slot * slot_bytes;
      const unsigned bar = smem_u32(&full_bar[slot]);
      if (round > 0) bounded_wait(smem_u32(&empty_bar[slot]), (round - 1) & 1, status, kTimeoutEmpty | slot);
      const unsigned live_rows = min(rows, seg_rows - local0);
      if (lane == 0) expect_bytes(bar, bytes * ((slab ? live_rows : rows) + M + mod_rows));
      __syncwarp();
      if (slab) {
        if (lane == 0) bulk_copy(base, w_seg + size_t(local0) * w_pitch, bytes * live_rows, bar);
      } else
      for (unsigned r = lane; r < rows; r += 32)  // rows past N re-read the last row; their results are dropped
        bulk_copy(base + r * pitch, w_seg + size_t(min(local0 + r, seg_rows - 1)) * w_pitch + size_t(split) * k_bytes + size_t(first) * 64, bytes, bar);
      if (!waited && (c + 1 == kSlots || c + 1 == chunks)) {
        // The weight copies of the first slots are in flight; only now wait for the previous kernel,
        // then fetch the activations it produced for those slots.
        grid_dependency_wait();
        waited = true;
        for (unsigned cc = 0; cc <= c; ++cc) {
          const unsigned f = cc * chunk_windows, n = min(chunk_windows, windows - f);
          const unsigned b2 = ring_base + (cc % kSlots) * slot_bytes + rows * pitch;
          if (slab) {
            if (lane == 0) bulk_copy(b2, x, n * 64 * M, smem_u32(&full_bar[cc % kSlots]));
          } else
          for (unsigned m = lane; m < M; m += 32)
            bulk_copy(b2 + m * pitch, x + m * x_row + size_t(f) * 64, n * 64, smem_u32(&full_bar[cc % kSlots]));
        }
      } else if (waited) {
        for (unsigned m = lane; m < M; m += 32)
          bulk_copy(base + (rows + m) * pitch, x + m * x_row + size_t(first) * 64, bytes, bar);
      }
    }
    if (!waited) grid_dependency_wait();
    fetch_early();
  } else {
    // ---------------- consumer warps ----------------
    // Two accumulator sets (one per MMA of a 16-byte chunk) keep consecutive MMAs independent; fragments
    // of the next window are read from shared memory while the current window multiplies.
    float acc[2][NT][4];
#pragma unroll
    for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h2][nt][i] = 0.f;
    const bool two_halves = rows == 16;
    unsigned b_off[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) b_off[nt] = (rows + min(unsigned(nt * 8) + g, M - 1)) * pitch + t * 16;
    uint4 fa_lo[2], fa_hi[2], fb[2][NT];
    for (unsigned c = 0; c < chunks; ++c) {
      const unsigned slot = c % kSlots, round = c / kSlots;
      const unsigned count = min(chunk_windows, windows - c * chunk_windows);
      const unsigned base = ring_base + slot * slot_bytes;
      // AdaLN vectors (one value per column, up to 6 x 8 columns per lane: K <= 1536) are fetched from global
      // memory while the slot is still filling.
      Bf16x8 mod_scale[6], mod_shift[6];
      if (kLn && (flags & kFlagLnModulate) && c == 0) {
#pragma unroll
        for (int i = 0; i < 6; ++i) {
          const unsigned v = lane + 32 * i;
          if (v < K / 8) {
            mod_scale[i] = *reinterpret_cast<const Bf16x8*>(extra.ln_scale + 8 * v);
            mod_shift[i] = *reinterpret_cast<const Bf16x8*>(extra.ln_shift + 8 * v);
          }
        }
      }
      bounded_wait(smem_u32(&full_bar[slot]), round & 1, status, kTimeoutFull | slot);
      if (c == 0) fetch_early();  // the slot landed, so the producer has passed the grid-dependency wait
      if (kLn && (flags & kFlagLayerNorm) && c == 0) {
        // Fused LayerNorm (whole rows are in this slot: the recipe only sets the flag when K is one chunk).
        // Warp w normalises rows w, w + W, ... in place, rounding to bf16 exactly where the stand-alone
        // kernel would have stored them; then the consumer warps meet before anyone multiplies.
        unsigned char* slot_ptr = ring + slot * slot_bytes;
        const unsigned vecs = K / 8;
        for (unsigned m = warp; m < M; m += kConsumerWarps) {
          Bf16x8* xr = reinterpret_cast<Bf16x8*>(slot_ptr + (rows + m) * pitch);
          // the row (up to 6 x 8 values per lane, K <= 1536) stays in registers across the three passes
          float f[6][8];
          float sum = 0.f;
#pragma unroll
          for (int q = 0; q < 6; ++q) {
            const unsigned i = lane + 32 * q;
            if (i < vecs) {
              unpack8(xr[i], f[q]);
#pragma unroll
              for (int j = 0; j < 8; ++j) sum += f[q][j];
            }
          }
          const float mean = warp_sum(sum) / float(K);
          float var = 0.f;
#pragma unroll
          for (int q = 0; q < 6; ++q)
            if (lane + 32 * q < vecs) {
#pragma unroll
              for (int j = 0; j < 8; ++j) var += (f[q][j] - mean) * (f[q][j] - mean);
            }
          const float rstd = rsqrtf(warp_sum(var) / float(K) + extra.ln_eps);
#pragma unroll
          for (int q = 0; q < 6; ++q) {
            const unsigned i = lane + 32 * q;
            if (i < vecs) {
              if (flags & kFlagLnModulate) {
                float a[8], b[8];
                unpack8(mod_scale[q], a);
                unpack8(mod_shift[q], b);
#pragma unroll
                for (int j = 0; j < 8; ++j) f[q][j] = (f[q][j] - mean) * rstd * (1.f + a[j]) + b[j];
              } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) f[q][j] = (f[q][j] - mean) * rstd;
              }
              xr[i] = pack8(f[q]);
            }
          }
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
      }
      const unsigned a_lo = base + g * pitch + t * 16, a_hi = a_lo + 8 * pitch;
      auto fetch = [&](int buf, unsigned win) {
        fa_lo[buf] = lds128(a_lo + win * 64);
        fa_hi[buf] = two_halves ? lds128(a_hi + win * 64) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) fb[buf][nt] = lds128(base + b_off[nt] + win * 64);
      };
      auto multiply = [&](int buf) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          skinny::mma16n8<kFp8>(acc[0][nt], fa_lo[buf].x, fa_hi[buf].x, fa_lo[buf].y, fa_hi[buf].y, fb[buf][nt].x, fb[buf][nt].y);
          skinny::mma16n8<kFp8>(acc[1][nt], fa_lo[buf].z, fa_hi[buf].z, fa_lo[buf].w, fa_hi[buf].w, fb[buf][nt].z, fb[buf][nt].w);
        }
      };
      unsigned win = warp;
      if (win < count) fetch(0, win);
      while (win < count) {
        unsigned next = win + kConsumerWarps;
        if (next < count) fetch(1, next);
        multiply(0);
        win = next;
        if (win >= count) break;
        next = win + kConsumerWarps;
        if (next < count) fetch(0, next);
        multiply(1);
        win = next;
      }
      __syncwarp();
      if (lane == 0 && c + kSlots < chunks) arrive(smem_u32(&empty_bar[slot]));
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float* tile = partial + size_t(warp) * 16 * mp;
      const unsigned col = nt * 8 + 2 * t;  // columns past M are padding of the token tile: not stored
      if (col < M) {
        tile[g * mp + col] = acc[0][nt][0] + acc[1][nt][0];
        tile[(g + 8) * mp + col] = acc[0][nt][2] + acc[1][nt][2];
      }
      if (col + 1 < M) {
        tile[g * mp + col + 1] = acc[0][nt][1] + acc[1][nt][1];
        tile[(g + 8) * mp + col + 1] = acc[0][nt][3] + acc[1][nt][3];
      }
    }
  }
  grid_dependency_release();
  __syncthreads();
  if (kSplit > 1) {
    tc::cluster_wait();   // every slice of the cluster is running
    if (split != 0) {
      const unsigned cell0 = tc::peer_smem(smem_u32(gathered + (split - 1) * rows * M), 0);
      for (unsigned i = threadIdx.x; i < rows * M; i += kThreads) {
        const unsigned r = i % rows, m = i / rows;
        float total = 0.f;
#pragma unroll
        for (int wq = 0; wq < kConsumerWarps; ++wq) total += partial[(wq * 16 + r) * mp + m];
        tc::store_peer_f32(cell0 + i * 4, total);
      }
    }
    tc::cluster_arrive();
    tc::cluster_wait();   // the partial sums of every slice have landed in slice 0
    if (split != 0) return;
  }
  const float alpha = (flags & kFlagScaled) ? (*scale_a) * (*scale_w) : 1.f;
  for (unsigned i = threadIdx.x; i < rows * M; i += kThreads) {
    const unsigned r = i % rows, m = i / rows;
    if (local0 + r >= seg_rows) continue;
    float total = 0.f;
#pragma unroll
    for (int wq = 0; wq < kConsumerWarps; ++wq) total += partial[(wq * 16 + r) * mp + m];
#pragma unroll
    for (int s = 1; s < kSplit; ++s) total += gathered[(s - 1) * rows * M + i];   // slice order
    // bias is indexed inside its own matrix, the output column across all of them
    const unsigned n = col0 + local0 + r;
    if (i == threadIdx.x && early_valid) {
      // first output of this thread: bias and residual were fetched while the MMAs ran
      float v = total * alpha;
      if (flags & kFlagBias) v += early_bias;
      v = apply_activation(v, flags);
      if (flags & kFlagResidual) v += early_residual;
      if (flags & kFlagOutF32) static_cast<float*>(y)[size_t(m) * ldy + n] = v;
      else static_cast<bf16*>(y)[size_t(m) * ldy + n] = __float2bfloat16_rn(v);
    } else {
      gemm_store(total, m, n, y, ldy, bias_seg - col0, residual, alpha, flags);
    }
  }
}

}  // namespace stream

// grid = (ceil(N / rows), 1, 1), block = 288 threads for up to 32 tokens, 160 above,
// dynamic shared memory = min(2, chunks) * (rows + M) * pitch + 16 + warps * 16 * (M | 1) * 4,
// pitch = chunk_windows * 64 (+ 16 unless the slab flag is set);
// M <= 8 * tiles; K bytes a multiple of 64; rows in {8, 16}.
#define AGI_STREAM_KERNEL(NAME, TYPE, FP8, NT)                                                                       \
  extern "C" __global__ void __launch_bounds__(stream::threads(NT), NT <= 4 ? 3 : 1)                                                  \
  NAME(const TYPE* x, const TYPE* w, void* y, const bf16* bias, const bf16* residual, const float* scale_a,         \
       const float* scale_w, unsigned* status, unsigned M, unsigned N, unsigned K, unsigned ldx, unsigned ldy,      \
       unsigned flags, unsigned rows, unsigned chunk_windows) {                                                             \
    stream::body<FP8, NT>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y, bias,         \
                          residual, scale_a, scale_w, status, M, N, K, ldx, ldy, flags, rows, chunk_windows);       \
  }

// The fused bf16 families: up to three weight matrices side by side along N (N0 | N1 | N2, zeros when unused);
// the `lnfused` kernels add an optional LayerNorm / AdaLN prologue over the activation rows (flags kFlagLayerNorm, kFlagLnModulate;
// needs K in one chunk, and K <= 1536 when modulating).
#define AGI_STREAM_FUSED_KERNEL(NAME, NT, LN)                                                                          \
  extern "C" __global__ void __launch_bounds__(stream::threads(NT), NT <= 4 ? 3 : 1)                                                  \
  NAME(const bf16* x, const bf16* w0, const bf16* w1, const bf16* w2, void* y, const bf16* bias0, const bf16* bias1, \
       const bf16* bias2, const bf16* residual, const bf16* ln_scale, const bf16* ln_shift, unsigned* status,        \
       unsigned M, unsigned N0, unsigned N1, unsigned N2, unsigned K, unsigned ldx, unsigned ldy, unsigned flags,    \
       unsigned rows, unsigned chunk_windows, float ln_eps) {                                                        \
    stream::Extra extra;                                                                                             \
    extra.w1 = reinterpret_cast<const uint8_t*>(w1);                                                                 \
    extra.w2 = reinterpret_cast<const uint8_t*>(w2);                                                                 \
    extra.bias1 = bias1;                                                                                             \
    extra.bias2 = bias2;                                                                                             \
    extra.n1 = N1;                                                                                                   \
    extra.n2 = N2;                                                                                                   \
    extra.ln_scale = ln_scale;                                                                                       \
    extra.ln_shift = ln_shift;                                                                                       \
    extra.ln_eps = ln_eps;                                                                                           \
    stream::body<false, NT, LN>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w0), y, bias0, \
                            residual, nullptr, nullptr, status, M, N0, K, ldx, ldy, flags, rows, chunk_windows,     \
                            extra);                                                                                  \
  }

AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_fused_bf16_t1, 1, false)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_lnfused_bf16_t1, 1, true)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_fused_bf16_t2, 2, false)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_lnfused_bf16_t2, 2, true)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_fused_bf16_t3, 3, false)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_lnfused_bf16_t3, 3, true)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_fused_bf16_t4, 4, false)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_lnfused_bf16_t4, 4, true)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_fused_bf16_t6, 6, false)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_lnfused_bf16_t6, 6, true)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_fused_bf16_t8, 8, false)
AGI_STREAM_FUSED_KERNEL(agi_gemm_stream_lnfused_bf16_t8, 8, true)
#undef AGI_STREAM_FUSED_KERNEL

// K slices in a cluster of S CTAs along grid z: grid = (ceil(N / rows), 1, S); K = elements per slice, ldw = row
// pitch of w in elements (S * K); shared memory as above for the slice, + (S - 1) * rows * M * 4.
#define AGI_STREAM_SPLIT_KERNEL(NAME, NT, S)                                                                          \
  extern "C" __global__ void __cluster_dims__(1, 1, S) __launch_bounds__(stream::threads(NT), 3)                     \
  NAME(const bf16* x, const bf16* w, void* y, const bf16* bias, const bf16* residual, unsigned* status, unsigned M,  \
       unsigned N, unsigned K, unsigned ldx, unsigned ldy, unsigned flags, unsigned rows, unsigned chunk_windows,   \
       unsigned ldw) {                                                                                               \
    stream::body<false, NT, false, S>(reinterpret_cast<const uint8_t*>(x), reinterpret_cast<const uint8_t*>(w), y,   \
                                      bias, residual, nullptr, nullptr, status, M, N, K, ldx, ldy, flags, rows,     \
                                      chunk_windows, stream::Extra(), ldw);                                          \
  }
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t1_k2, 1, 2)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t2_k2, 2, 2)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t3_k2, 3, 2)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t4_k2, 4, 2)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t1_k4, 1, 4)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t2_k4, 2, 4)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t3_k4, 3, 4)
AGI_STREAM_SPLIT_KERNEL(agi_gemm_stream_bf16_t4_k4, 4, 4)
#undef AGI_STREAM_SPLIT_KERNEL

AGI_STREAM_KERNEL(agi_gemm_stream_bf16_t1, bf16, false, 1)
AGI_STREAM_KERNEL(agi_gemm_stream_bf16_t2, bf16, false, 2)
AGI_STREAM_KERNEL(agi_gemm_stream_bf16_t3, bf16, false, 3)
AGI_STREAM_KERNEL(agi_gemm_stream_bf16_t4, bf16, false, 4)
AGI_STREAM_KERNEL(agi_gemm_stream_bf16_t6, bf16, false, 6)
AGI_STREAM_KERNEL(agi_gemm_stream_bf16_t8, bf16, false, 8)
AGI_STREAM_KERNEL(agi_gemm_stream_e4m3_t1, uint8_t, true, 1)
AGI_STREAM_KERNEL(agi_gemm_stream_e4m3_t2, uint8_t, true, 2)
AGI_STREAM_KERNEL(agi_gemm_stream_e4m3_t3, uint8_t, true, 3)
AGI_STREAM_KERNEL(agi_gemm_stream_e4m3_t4, uint8_t, true, 4)
AGI_STREAM_KERNEL(agi_gemm_stream_e4m3_t6, uint8_t, true, 6)
AGI_STREAM_KERNEL(agi_gemm_stream_e4m3_t8, uint8_t, true, 8)
#undef AGI_STREAM_KERNEL

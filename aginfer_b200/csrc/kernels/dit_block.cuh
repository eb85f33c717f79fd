// Persistent transformer-block kernel for the batch-1 action head: ONE launch walks a whole stack of DiT
// blocks (AdaLN LayerNorm -> Q|K|V -> attention -> output projection + residual -> LayerNorm -> MLP up with
// GELU -> MLP down + residual), every block's weights streamed from HBM exactly once.
//
// Why one launch.  At 17 tokens a block is five dependent matrix products of 5-19 MB each: 0.7-2.9 us of HBM
// time apiece, against ~3 us of fixed cost when each is its own kernel (launch, ring fill, drain).  Here the
// grid is one CTA per SM and stays resident; the only thing that separates dependent phases is a grid-wide
// arrival counter, and the weight stream never stops at a phase boundary:
//
//   * a producer warp per CTA walks the CTA's share of every weight matrix of every block, in execution order,
//     and keeps a ring of shared-memory slots (16 weight rows x 1 KB each) full with bulk copies.  Weights do
//     not depend on anything computed here, so the ring runs ahead of the consumers by its whole depth: while
//     the CTAs meet at a phase boundary, the next phase's weights are already landing.
//   * eight consumer warps hold the activations of the phase (17 x 1536 bf16, normalised on the way in) in
//     shared memory, keep their own K windows of them in registers as MMA B fragments for the whole phase, and
//     multiply each arriving 16-row weight chunk with warp-level MMAs (m16n8k16, fp32 accumulate).  A "unit" is
//     16 output features x one K span of at most 1536; units of a phase are dealt to the CTAs in contiguous
//     ranges.  The wide-K product (MLP down, K = 6144) is cut into K spans whose partial sums meet in global
//     memory; the last CTA to arrive for a group of 16 features adds them in span order (bit-reproducible) and
//     applies bias and residual.
//   * attention is a phase of its own: CTA i < heads x query tiles runs one (head, 16-query tile) with the
//     tensor-core streaming softmax used elsewhere in the bundle; the other CTAs go straight to the boundary.
//
// Phase boundaries are bounded waits on a monotonic counter in the arena (released with a device-scope fence,
// polled with acquire loads).  They need every CTA resident at once, which is why the grid is the SM count and
// the loader launches kernels named agi_coop_* cooperatively: the driver then refuses the launch instead of
// letting it wait for itself.  A wait that runs out records a code in the status word; every CTA sees the word
// at its next wait and leaves, so a fault surfaces as a status and wrong numbers, never as a hang.
#pragma once

#include "common.cuh"
#include "gemm_skinny.cuh"  // mma16n8
#include "gemm_stream.cuh"  // bulk copy and mbarrier helpers

namespace ditb {

constexpr int kConsumerWarps = 8;
constexpr unsigned kConsumers = kConsumerWarps * 32;
constexpr unsigned kThreads = kConsumers + 32;   // + the producer warp
constexpr unsigned kMaxSlots = 12;
constexpr unsigned kChunkWindows = 16;           // 64-byte K windows per ring slot row: 1 KB
constexpr unsigned kUnitRows = 16;               // output features per unit = rows of one MMA tile
constexpr unsigned kRingPitch = kChunkWindows * 64 + 64;   // +64: rows g, g+1 of a fragment fall into different bank halves
constexpr unsigned kSlotBytes = kUnitRows * kRingPitch;
constexpr unsigned kMaxSpan = 1536;              // K elements a consumer warp can keep as B fragments (6 windows x 8 warps)
constexpr unsigned kMaxChunks = kMaxSpan / 32 / kChunkWindows;   // 3
constexpr unsigned kHeaderBytes = 256;           // mbarriers and flags in front of the dynamic shared memory
constexpr unsigned kTableStride = 16;            // pointers per block in the table
constexpr unsigned kTimeoutFull = 0x700, kTimeoutEmpty = 0x800, kTimeoutGrid = 0x900;
constexpr unsigned long long kGridWaitNs = 200ull * 1000 * 1000;

// Entries of a block's row in the pointer table.
enum : unsigned { kWq = 0, kBq, kWk, kBk, kWv, kBv, kWo, kBo, kW1, kB1, kW2, kB2, kMod, kCtxK, kCtxV };

struct Dims {
  unsigned layers, T, D, heads, head_dim, mlp, mlp_span, ctx, cross_mask, mod_offset, slots;
  float eps, attn_scale;
};

// One matrix-product phase of a block: up to three weight matrices side by side along the output features.
struct Gemm {
  const uint8_t* w[3];
  const bf16* bias[3];
  unsigned rows_per_mat, N, K, span, slices;
};

__device__ __forceinline__ Gemm phase_gemm(const unsigned long long* row, unsigned phase, bool cross, const Dims& d) {
  Gemm g;
  auto weight = [&](unsigned i) { return reinterpret_cast<const uint8_t*>(row[i]); };
  auto vector = [&](unsigned i) { return reinterpret_cast<const bf16*>(row[i]); };
  g.w[1] = g.w[2] = nullptr;
  g.bias[1] = g.bias[2] = nullptr;
  g.rows_per_mat = d.D;
  g.K = g.span = d.D;
  g.slices = 1;
  if (phase == 0) {          // queries (cross-attention blocks) or queries | keys | values
    g.w[0] = weight(kWq); g.bias[0] = vector(kBq);
    g.N = d.D;
    if (!cross) {
      g.w[1] = weight(kWk); g.bias[1] = vector(kBk);
      g.w[2] = weight(kWv); g.bias[2] = vector(kBv);
      g.N = 3 * d.D;
    }
  } else if (phase == 1) {   // attention output projection
    g.w[0] = weight(kWo); g.bias[0] = vector(kBo);
    g.N = d.D;
  } else if (phase == 2) {   // MLP up
    g.w[0] = weight(kW1); g.bias[0] = vector(kB1);
    g.N = g.rows_per_mat = d.mlp;
  } else {                   // MLP down: K = mlp in spans
    g.w[0] = weight(kW2); g.bias[0] = vector(kB2);
    g.N = d.D;
    g.K = d.mlp;
    g.span = d.mlp_span;
    g.slices = d.mlp / d.mlp_span;
  }
  return g;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ unsigned load_acquire(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned load_relaxed(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

// mbarrier wait with a spin limit; false (and a status code) when it runs out or another CTA already failed.
__device__ __forceinline__ bool wait_slot(unsigned bar, unsigned parity, unsigned* status, unsigned code) {
  for (unsigned spin = 0; !stream::bar_done(bar, parity); ++spin) {
    if (spin > stream::kSpinLimit) {
      atomicCAS(status, 0u, code);
      return false;
    }
    if (spin > 64) {
      __nanosleep(32);
      if ((spin & 1023u) == 0 && load_relaxed(status) != 0) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------------------------------------------------
// Producer warp: the CTA's weight rows of every phase of every block, in execution order.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void produce(const unsigned long long* table, const Dims& d, unsigned* status,
                                        unsigned ring_base, unsigned long long* full_bar, unsigned long long* empty_bar) {
  const unsigned lane = threadIdx.x & 31, cta = blockIdx.x, ctas = gridDim.x;
  unsigned slot = 0, round = 0;
  for (unsigned layer = 0; layer < d.layers; ++layer) {
    const unsigned long long* row = table + size_t(layer) * kTableStride;
    const bool cross = (d.cross_mask >> layer) & 1u;
    for (unsigned phase = 0; phase < 4; ++phase) {
      const Gemm gm = phase_gemm(row, phase, cross, d);
      const unsigned groups = gm.N / kUnitRows, units = groups * gm.slices;
      const unsigned first = unsigned((unsigned long long)cta * units / ctas);
      const unsigned end = unsigned((unsigned long long)(cta + 1) * units / ctas);
      const unsigned windows = gm.span / 32;
      for (unsigned u = first; u < end; ++u) {
        const unsigned slice = u / groups, row0 = (u % groups) * kUnitRows;
        const unsigned mat = row0 / gm.rows_per_mat, local = row0 % gm.rows_per_mat;
        const uint8_t* w_mat = mat == 0 ? gm.w[0] : mat == 1 ? gm.w[1] : gm.w[2];
        const uint8_t* src = w_mat + (size_t(local + (lane & 15u)) * gm.K + size_t(slice) * gm.span) * 2;
        for (unsigned c = 0; c * kChunkWindows < windows; ++c) {
          const unsigned count = min(kChunkWindows, windows - c * kChunkWindows), bytes = count * 64;
          const unsigned bar = stream::smem_u32(&full_bar[slot]);
          if (round > 0 && !wait_slot(stream::smem_u32(&empty_bar[slot]), (round - 1) & 1, status, kTimeoutEmpty | slot))
            return;
          if (lane == 0) stream::expect_bytes(bar, bytes * kUnitRows);
          __syncwarp();
          if (lane < kUnitRows)
            stream::bulk_copy(ring_base + slot * kSlotBytes + lane * kRingPitch, src + size_t(c) * kChunkWindows * 64, bytes, bar);
          if (++slot == d.slots) { slot = 0; ++round; }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Consumer side.
// ---------------------------------------------------------------------------------------------------------
struct Consumer {
  const Dims& d;
  unsigned* status;
  unsigned* grid_counter;
  unsigned char* smem;          // dynamic shared memory (header first)
  unsigned long long* full_bar;
  unsigned long long* empty_bar;
  volatile unsigned* flags;     // [0] = this CTA gave up, [1] = "last arriver" broadcast, [2] = [0] as of the last boundary
  unsigned char* x_tile;        // activations of the phase: T rows, pitch x_pitch bytes
  float* part_tile;             // [warp][16][T | 1] partial sums of the consumer warps
  unsigned x_pitch, ring_base;
  unsigned slot, round;         // position in the ring (same walk as the producer)
  unsigned barriers_passed;
  unsigned lane, warp, g, t;

  __device__ __forceinline__ bool failed() const { return flags[0] != 0; }
  __device__ __forceinline__ void fail() { flags[0] = 1; }

  // Grid-wide phase boundary.  Everything this CTA wrote is ordered before its arrival; everything other CTAs
  // wrote before theirs is visible (through L2: readers use ld.cg / cp.async.cg) after the wait.  Returns false,
  // to every consumer thread alike, once this CTA or any other has given up.
  __device__ __forceinline__ bool grid_barrier() {
    ++barriers_passed;
    consumer_sync();
    if (threadIdx.x == 0) {
      if (!failed()) {
        __threadfence();
        atomicAdd(grid_counter, 1u);
        const unsigned target = barriers_passed * gridDim.x;
        const unsigned long long t0 = global_ns();
        unsigned spin = 0;
        while (load_acquire(grid_counter) < target) {
          if ((++spin & 63u) == 0) {
            if (load_relaxed(status) != 0) { fail(); break; }
            if (global_ns() - t0 > kGridWaitNs) {
              atomicCAS(status, 0u, kTimeoutGrid | (barriers_passed & 0xffu));
              fail();
              break;
            }
          }
        }
        __threadfence();
      }
      flags[2] = flags[0];   // the verdict every thread acts on: written only between this barrier's two syncs
    }
    consumer_sync();
    return flags[2] == 0;
  }

  // ---- activations into shared memory: rows warp, warp + 8, ... ; 16-byte vectors lane, lane + 32, ... ----
  // mode 0: copy;  mode 1: LayerNorm without affine;  mode 2: LayerNorm, then * (1 + scale) + shift (AdaLN).
  __device__ __noinline__ void load_activations(const bf16* src, unsigned ld, unsigned k0, unsigned cols, unsigned mode,
                                                   const bf16* scale, const bf16* shift) {
    const unsigned vecs = cols / 8;
    constexpr int kRowsPerWarp = 3, kVecsPerLane = kMaxSpan / 8 / 32;   // 24 tokens at most; 6 vectors per lane
    Bf16x8 raw[kRowsPerWarp][kVecsPerLane];
#pragma unroll
    for (int rr = 0; rr < kRowsPerWarp; ++rr) {
      const unsigned m = warp + rr * kConsumerWarps;
      if (m < d.T) {
        const uint4* row = reinterpret_cast<const uint4*>(src + size_t(m) * ld + k0);
#pragma unroll
        for (int q = 0; q < kVecsPerLane; ++q) {
          const unsigned i = lane + 32 * q;
          if (i < vecs) {
            const uint4 v = __ldcg(row + i);
            raw[rr][q] = *reinterpret_cast<const Bf16x8*>(&v);
          }
        }
      }
    }
#pragma unroll
    for (int rr = 0; rr < kRowsPerWarp; ++rr) {
      const unsigned m = warp + rr * kConsumerWarps;
      if (m >= d.T) continue;
      Bf16x8* dst = reinterpret_cast<Bf16x8*>(x_tile + size_t(m) * x_pitch);
      if (mode == 0) {
#pragma unroll
        for (int q = 0; q < kVecsPerLane; ++q)
          if (lane + 32 * q < vecs) dst[lane + 32 * q] = raw[rr][q];
        continue;
      }
      float sum = 0.f;
#pragma unroll
      for (int q = 0; q < kVecsPerLane; ++q)
        if (lane + 32 * q < vecs) {
          float f[8];
          unpack8(raw[rr][q], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) sum += f[j];
        }
      const float mean = warp_sum(sum) / float(cols);
      float var = 0.f;
#pragma unroll
      for (int q = 0; q < kVecsPerLane; ++q)
        if (lane + 32 * q < vecs) {
          float f[8];
          unpack8(raw[rr][q], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) var += (f[j] - mean) * (f[j] - mean);
        }
      const float rstd = rsqrtf(warp_sum(var) / float(cols) + d.eps);
#pragma unroll
      for (int q = 0; q < kVecsPerLane; ++q) {
        const unsigned i = lane + 32 * q;
        if (i < vecs) {
          float f[8];
          unpack8(raw[rr][q], f);
          if (mode == 2) {
            float a[8], b[8];
            unpack8(*reinterpret_cast<const Bf16x8*>(scale + 8 * i), a);
            unpack8(*reinterpret_cast<const Bf16x8*>(shift + 8 * i), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd * (1.f + a[j]) + b[j];
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = (f[j] - mean) * rstd;
          }
          dst[i] = pack8(f);
        }
      }
    }
  }

  // ---- one matrix-product phase ----
  // kind 0: y = bf16(acc + bias)            (queries / keys / values)
  // kind 1: y = bf16(acc + bias + y)        (output projection onto the residual stream)
  // kind 2: y = bf16(gelu(acc + bias))      (MLP up)
  // kind 3: K spans: partial sums to `partial`, the last arriver of a feature group adds them, + bias + y
  template <int NT>
  __device__ __noinline__ void gemm_phase(const Gemm& gm, unsigned kind, const bf16* x, unsigned ldx, unsigned x_mode,
                                             const bf16* ln_scale, const bf16* ln_shift, bf16* y, unsigned ldy,
                                             float* partial, unsigned* group_counters) {
    const unsigned cta = blockIdx.x, ctas = gridDim.x;
    const unsigned groups = gm.N / kUnitRows, units = groups * gm.slices;
    const unsigned first = unsigned((unsigned long long)cta * units / ctas);
    const unsigned end = unsigned((unsigned long long)(cta + 1) * units / ctas);
    const unsigned windows = gm.span / 32;
    const unsigned T = d.T, mp = T | 1u, slots = d.slots, ring = ring_base, pitch_x = x_pitch;
    unsigned char* const tile_x = x_tile;
    unsigned slot_now = slot, round_now = round;   // the ring walk lives in registers while the phase runs
    uint4 bfrag[kMaxChunks][2][NT];
    unsigned have_slice = 0xffffffffu;
    for (unsigned u = first; u < end; ++u) {
      const unsigned slice = u / groups, row0 = (u % groups) * kUnitRows;
      if (slice != have_slice) {
        // the phase's activations (this K span of them), then this warp's windows of them as B fragments
        load_activations(x, ldx, slice * gm.span, gm.span, x_mode, ln_scale, ln_shift);
        consumer_sync();
#pragma unroll
        for (unsigned c = 0; c < kMaxChunks; ++c)
#pragma unroll
          for (unsigned j = 0; j < 2; ++j) {
            const unsigned win = c * kChunkWindows + warp + j * kConsumerWarps;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const unsigned m = min(unsigned(nt * 8) + g, T - 1);
              bfrag[c][j][nt] = win < windows
                  ? *reinterpret_cast<const uint4*>(tile_x + size_t(m) * pitch_x + size_t(win) * 64 + t * 16)
                  : make_uint4(0, 0, 0, 0);
            }
          }
        have_slice = slice;
      }
      float acc[2][NT][4];
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[h2][nt][i] = 0.f;
#pragma unroll
      for (unsigned c = 0; c < kMaxChunks; ++c) {
        if (c * kChunkWindows >= windows) continue;
        const unsigned count = min(kChunkWindows, windows - c * kChunkWindows);
        if (!failed() && !wait_slot(stream::smem_u32(&full_bar[slot_now]), round_now & 1, status, kTimeoutFull | slot_now)) fail();
        const unsigned base = ring + slot_now * kSlotBytes + g * kRingPitch + t * 16;
#pragma unroll
        for (unsigned j = 0; j < 2; ++j) {
          const unsigned win = warp + j * kConsumerWarps;
          if (win < count) {
            const uint4 lo = stream::lds128(base + win * 64), hi = stream::lds128(base + 8 * kRingPitch + win * 64);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              skinny::mma16n8<false>(acc[0][nt], lo.x, hi.x, lo.y, hi.y, bfrag[c][j][nt].x, bfrag[c][j][nt].y);
              skinny::mma16n8<false>(acc[1][nt], lo.z, hi.z, lo.w, hi.w, bfrag[c][j][nt].z, bfrag[c][j][nt].w);
            }
          }
        }
        __syncwarp();
        if (lane == 0) stream::arrive(stream::smem_u32(&empty_bar[slot_now]));
        if (++slot_now == slots) { slot_now = 0; ++round_now; }
      }
      // the warps' partial tiles: c0, c1 = feature g, tokens 2t, 2t + 1 of the tile; c2, c3 = feature g + 8
      float* tile = part_tile + size_t(warp) * 16 * mp;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const unsigned col = nt * 8 + 2 * t;
        if (col < T) {
          tile[g * mp + col] = acc[0][nt][0] + acc[1][nt][0];
          tile[(g + 8) * mp + col] = acc[0][nt][2] + acc[1][nt][2];
        }
        if (col + 1 < T) {
          tile[g * mp + col + 1] = acc[0][nt][1] + acc[1][nt][1];
          tile[(g + 8) * mp + col + 1] = acc[0][nt][3] + acc[1][nt][3];
        }
      }
      consumer_sync();
      const unsigned mat = row0 / gm.rows_per_mat, local = row0 % gm.rows_per_mat;
      for (unsigned i = threadIdx.x; i < kUnitRows * T; i += kConsumers) {
        const unsigned r = i % kUnitRows, m = i / kUnitRows;
        float total = 0.f;
#pragma unroll
        for (int wq = 0; wq < kConsumerWarps; ++wq) total += part_tile[(wq * 16 + r) * mp + m];
        const unsigned n = row0 + r;
        if (kind == 3 && gm.slices > 1) {
          partial[(size_t(slice) * T + m) * gm.N + n] = total;
          continue;
        }
        const bf16* bias = mat == 0 ? gm.bias[0] : mat == 1 ? gm.bias[1] : gm.bias[2];
        float v = total + __bfloat162float(bias[local + r]);
        if (kind == 2) v = gelu_tanh(v);
        bf16* out = y + size_t(m) * ldy + n;
        if (kind == 1 || kind == 3) v += __bfloat162float(__ldcg(out));
        *out = __float2bfloat16_rn(v);
      }
      if (kind == 3 && gm.slices > 1) {
        // arrival of this K span for the feature group; the last one to arrive adds the spans in order
        consumer_sync();
        if (threadIdx.x == 0) {
          __threadfence();
          const unsigned before = atomicAdd(&group_counters[row0 / kUnitRows], 1u);
          flags[1] = before == gm.slices - 1 ? 1u : 0u;
          if (before == gm.slices - 1) __threadfence();
        }
        consumer_sync();
        if (flags[1] != 0) {
          for (unsigned i = threadIdx.x; i < kUnitRows * T; i += kConsumers) {
            const unsigned r = i % kUnitRows, m = i / kUnitRows, n = row0 + r;
            float total = 0.f;
            for (unsigned s = 0; s < gm.slices; ++s) total += __ldcg(partial + (size_t(s) * T + m) * gm.N + n);
            bf16* out = y + size_t(m) * ldy + n;
            const float v = total + __bfloat162float(gm.bias[0][n]) + __bfloat162float(__ldcg(out));
            *out = __float2bfloat16_rn(v);
          }
          if (threadIdx.x == 0) group_counters[row0 / kUnitRows] = 0;
        }
      }
      consumer_sync();   // partial tiles (and the activation tile) may be overwritten from here on
    }
    slot = slot_now;
    round = round_now;
  }

  // ---- attention of one (head, 16-query tile): tensor-core scores and P.V, warps split the keys ----
  __device__ __noinline__ void attention_task(unsigned head, unsigned row_base, const bf16* q, unsigned q_stride,
                                                 const bf16* k, const bf16* v, unsigned kv_stride, unsigned kv_rows,
                                                 bf16* o, unsigned o_stride) {
    const unsigned head_dim = d.head_dim, q_rows = d.T;
    const unsigned kv16 = (kv_rows + 15) & ~15u;
    const unsigned pitch = head_dim + 8;
    bf16* k_tile = reinterpret_cast<bf16*>(x_tile);          // the activation tile is idle during this phase
    bf16* v_tile = k_tile + size_t(kv16) * pitch;
    float* merge = reinterpret_cast<float*>(x_tile);         // written after every warp has finished with the keys
    const unsigned vec_per_row = head_dim / 8;
    for (unsigned i = threadIdx.x; i < kv16 * vec_per_row; i += kConsumers) {
      const unsigned j = i / vec_per_row, dd = (i % vec_per_row) * 8;
      const unsigned src_row = min(j, kv_rows - 1), bytes = j < kv_rows ? 16u : 0u;
      const unsigned kd = stream::smem_u32(k_tile + j * pitch + dd), vd = stream::smem_u32(v_tile + j * pitch + dd);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd),
                   "l"(k + size_t(src_row) * kv_stride + head * head_dim + dd), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd),
                   "l"(v + size_t(src_row) * kv_stride + head * head_dim + dd), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const unsigned ksteps = head_dim / 16;   // <= 4
    unsigned qa[4][4];
#pragma unroll
    for (int ks = 0; ks < 4; ++ks)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        qa[ks][r] = 0;
        const unsigned row = row_base + g + (r & 1) * 8, col = ks * 16 + 2 * t + (r >> 1) * 8;
        if (unsigned(ks) < ksteps && row < q_rows) {
          const unsigned bits = __ldcg(reinterpret_cast<const unsigned*>(q + size_t(row) * q_stride + head * head_dim + col));
          const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&bits));
          const bf162 scaled = __floats2bfloat162_rn(f.x * d.attn_scale, f.y * d.attn_scale);
          qa[ks][r] = *reinterpret_cast<const unsigned*>(&scaled);
        }
      }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    consumer_sync();

    float row_max[2] = {-3.0e38f, -3.0e38f}, row_sum[2] = {0.f, 0.f}, out[8][4];
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) out[nt][i] = 0.f;
    const unsigned dtiles = head_dim / 8;    // <= 8
    for (unsigned key0 = warp * 16; key0 < kv16; key0 += 16 * kConsumerWarps) {
      unsigned kb[2][4][2];
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          if (unsigned(ks) < ksteps) {
            const bf16* row = k_tile + (key0 + half * 8 + g) * pitch + ks * 16 + 2 * t;
            kb[half][ks][0] = *reinterpret_cast<const unsigned*>(row);
            kb[half][ks][1] = *reinterpret_cast<const unsigned*>(row + 8);
          }
      float s[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        s[half][0] = s[half][1] = s[half][2] = s[half][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          if (unsigned(ks) < ksteps)
            skinny::mma16n8<false>(s[half], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[half][ks][0], kb[half][ks][1]);
      }
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (key0 + half * 8 + 2 * t + (i & 1) >= kv_rows) s[half][i] = -3.0e38f;
      unsigned pa[4];
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {  // hr 0: row g (c0, c1), hr 1: row g + 8 (c2, c3)
        float tile_max = fmaxf(fmaxf(s[0][2 * hr], s[0][2 * hr + 1]), fmaxf(s[1][2 * hr], s[1][2 * hr + 1]));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float new_max = fmaxf(row_max[hr], tile_max);
        const float rescale = new_max > -1.0e38f ? __expf(row_max[hr] - new_max) : 1.f;
        float p[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float sc = s[j >> 1][2 * hr + (j & 1)];
          p[j] = sc > -1.0e38f ? __expf(sc - new_max) : 0.f;
        }
        float tile_sum = (p[0] + p[1]) + (p[2] + p[3]);
        tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, 1);
        tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, 2);
        row_sum[hr] = row_sum[hr] * rescale + tile_sum;
        row_max[hr] = new_max;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          out[nt][2 * hr] *= rescale;
          out[nt][2 * hr + 1] *= rescale;
        }
        const bf162 lo = __floats2bfloat162_rn(p[0], p[1]), hi = __floats2bfloat162_rn(p[2], p[3]);
        pa[hr] = *reinterpret_cast<const unsigned*>(&lo);
        pa[2 + hr] = *reinterpret_cast<const unsigned*>(&hi);
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
        if (unsigned(nt) < dtiles) {
          const unsigned addr = stream::smem_u32(v_tile + (key0 + (lane & 15)) * pitch + nt * 8);
          unsigned b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
          skinny::mma16n8<false>(out[nt], pa[0], pa[1], pa[2], pa[3], b0, b1);
        }
    }
    consumer_sync();   // every warp is done with the key and value tiles: the merge area may overwrite them
    const unsigned mp = head_dim + 2;
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
      float* dst = merge + (size_t(warp) * 16 + g + hr * 8) * mp;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
        if (unsigned(nt) < dtiles) {
          dst[nt * 8 + 2 * t] = out[nt][2 * hr];
          dst[nt * 8 + 2 * t + 1] = out[nt][2 * hr + 1];
        }
      if (t == 0) {
        dst[head_dim] = row_max[hr];
        dst[head_dim + 1] = row_sum[hr];
      }
    }
    consumer_sync();
    const unsigned my_rows = min(16u, q_rows - row_base);
    for (unsigned i = threadIdx.x; i < my_rows * head_dim; i += kConsumers) {
      const unsigned r = i / head_dim, dd = i % head_dim;
      float best = -3.0e38f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) best = fmaxf(best, merge[(w * 16 + r) * mp + head_dim]);
      float num = 0.f, den = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) {
        const float* src = merge + (w * 16 + r) * mp;
        const float f = src[head_dim] > -1.0e38f ? __expf(src[head_dim] - best) : 0.f;
        num += f * src[dd];
        den += f * src[head_dim + 1];
      }
      o[size_t(row_base + r) * o_stride + head * head_dim + dd] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    }
    consumer_sync();   // the merge area is the next task's key tile
  }
};

// Dynamic shared memory of the kernel for a given shape (the recipe builder mirrors this formula).
__host__ __device__ constexpr unsigned round_up(unsigned v, unsigned to) { return (v + to - 1) / to * to; }
__host__ __device__ inline unsigned activation_pitch(unsigned D, unsigned mlp_span) { return (D > mlp_span ? D : mlp_span) * 2 + 64; }
__host__ __device__ inline unsigned phase_region_bytes(unsigned T, unsigned D, unsigned mlp_span, unsigned head_dim, unsigned ctx) {
  const unsigned gemm_bytes = T * activation_pitch(D, mlp_span) + kConsumerWarps * 16 * (T | 1u) * 4;
  const unsigned keys = round_up(ctx > T ? ctx : T, 16);
  const unsigned kv_bytes = 2 * keys * (head_dim + 8) * 2, merge_bytes = kConsumerWarps * 16 * (head_dim + 2) * 4;
  const unsigned attn_bytes = kv_bytes > merge_bytes ? kv_bytes : merge_bytes;
  return round_up(gemm_bytes > attn_bytes ? gemm_bytes : attn_bytes, 128);
}

template <int NT>
__device__ __forceinline__ void run(const unsigned long long* table, bf16* seq, bf16* qkv, bf16* attn, bf16* ff, float* partial,
                                    unsigned* group_counters, unsigned* grid_counter, unsigned* status, const Dims& d) {
  extern __shared__ __align__(128) unsigned char dit_smem[];
  unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(dit_smem);
  unsigned long long* empty_bar = full_bar + kMaxSlots;
  volatile unsigned* flags = reinterpret_cast<volatile unsigned*>(empty_bar + kMaxSlots);
  const unsigned region = phase_region_bytes(d.T, d.D, d.mlp_span, d.head_dim, d.ctx);
  const unsigned warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    for (unsigned s = 0; s < kMaxSlots; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(stream::smem_u32(&full_bar[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(stream::smem_u32(&empty_bar[s])), "n"(kConsumerWarps));
    }
    flags[0] = flags[1] = flags[2] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  grid_dependency_wait();   // the table and the residual stream come from earlier launches
  __syncthreads();
  const unsigned ring_base = stream::smem_u32(dit_smem + kHeaderBytes + region);

  if (warp == kConsumerWarps) {
    produce(table, d, status, ring_base, full_bar, empty_bar);
    return;
  }

  Consumer c{d, status, grid_counter, dit_smem, full_bar, empty_bar, flags,
             dit_smem + kHeaderBytes, nullptr, activation_pitch(d.D, d.mlp_span), ring_base, 0, 0, 0,
             threadIdx.x & 31, warp, (threadIdx.x & 31) >> 2, threadIdx.x & 3};
  c.part_tile = reinterpret_cast<float*>(c.x_tile + size_t(d.T) * c.x_pitch);
  const unsigned D = d.D, T = d.T;
  const unsigned q_tiles = (T + 15) / 16, tasks = d.heads * q_tiles;
  for (unsigned layer = 0; layer < d.layers; ++layer) {
    const unsigned long long* row = table + size_t(layer) * kTableStride;
    const bool cross = (d.cross_mask >> layer) & 1u;
    const bf16* mod = reinterpret_cast<const bf16*>(row[kMod]) + d.mod_offset;   // (scale | shift) of this step
    // queries (| keys | values) of the modulated, normalised residual stream
    c.template gemm_phase<NT>(phase_gemm(row, 0, cross, d), 0, seq, D, 2, mod, mod + D, qkv, 3 * D, partial, group_counters);
    if (!c.grid_barrier()) return;
    const bf16* keys = cross ? reinterpret_cast<const bf16*>(row[kCtxK]) : qkv + D;
    const bf16* values = cross ? reinterpret_cast<const bf16*>(row[kCtxV]) : qkv + 2 * D;
    for (unsigned task = blockIdx.x; task < tasks; task += gridDim.x)
      c.attention_task(task / q_tiles, (task % q_tiles) * 16, qkv, 3 * D, keys, values, cross ? D : 3 * D,
                       cross ? d.ctx : T, attn, D);
    if (!c.grid_barrier()) return;
    c.template gemm_phase<NT>(phase_gemm(row, 1, cross, d), 1, attn, D, 0, nullptr, nullptr, seq, D, partial, group_counters);
    if (!c.grid_barrier()) return;
    c.template gemm_phase<NT>(phase_gemm(row, 2, cross, d), 2, seq, D, 1, nullptr, nullptr, ff, d.mlp, partial, group_counters);
    if (!c.grid_barrier()) return;
    c.template gemm_phase<NT>(phase_gemm(row, 3, cross, d), 3, ff, d.mlp, 0, nullptr, nullptr, seq, D, partial, group_counters);
    // the last block's results are ordered by the end of the kernel
    if (layer + 1 < d.layers && !c.grid_barrier()) return;
  }
}

}  // namespace ditb

// Stores up to 16 device addresses into consecutive 8-byte slots of a table in the arena: how a recipe hands a
// persistent kernel more pointers than a parameter list should carry (the loader resolves each argument).
// grid = 1, block = 32.
extern "C" __global__ void agi_store_pointers16(unsigned long long* table, unsigned first, unsigned count,
                                                const void* p0, const void* p1, const void* p2, const void* p3,
                                                const void* p4, const void* p5, const void* p6, const void* p7,
                                                const void* p8, const void* p9, const void* p10, const void* p11,
                                                const void* p12, const void* p13, const void* p14, const void* p15) {
  grid_dependency_wait();
  const void* all[16] = {p0, p1, p2, p3, p4, p5, p6, p7, p8, p9, p10, p11, p12, p13, p14, p15};
  if (threadIdx.x < count && threadIdx.x < 16)
    table[first + threadIdx.x] = reinterpret_cast<unsigned long long>(all[threadIdx.x]);
}

// A stack of DiT blocks in one launch.  grid = (number of SMs, 1, 1), one CTA per SM, block = 288 threads
// (8 consumer warps + 1 producer warp); dynamic shared memory = 256 + phase_region_bytes(...) + slots * 17408.
// `table`: 16 pointers per block (weights and biases of to_q, to_k, to_v, to_out, fc1, fc2; the block's AdaLN
// (scale | shift) rows; keys and values of the context tokens for cross-attention blocks).  `seq` [T, D] is
// the residual stream, updated in place; `qkv` [T, 3D], `attn` [T, D], `ff` [T, mlp] and `partial`
// [mlp / mlp_span, T, D] fp32 are scratch; `group_counters` (D / 16 words) must be zero and are left zero;
// `grid_counter` must be zero at launch.  bit l of `cross_mask`: block l attends to the context tokens.
// `mod_offset`: elements from a block's AdaLN pointer to this denoising step's (scale | shift) row.
// Shape limits: T <= 8 * (the kernel's _t suffix); D and mlp_span multiples of 32, at most 1536; D, mlp multiples of 16; mlp a multiple
// of mlp_span; head_dim a multiple of 16, at most 64; layers <= 32.
#define AGI_DIT_BLOCKS_KERNEL(NAME, NT)                                                                              \
  extern "C" __global__ void __launch_bounds__(ditb::kThreads, 1)                                                    \
  NAME(const unsigned long long* table, bf16* seq, bf16* qkv, bf16* attn, bf16* ff, float* partial,                 \
       unsigned* group_counters, unsigned* grid_counter, unsigned* status, unsigned layers, unsigned T, unsigned D,  \
       unsigned heads, unsigned head_dim, unsigned mlp, unsigned mlp_span, unsigned ctx, unsigned cross_mask,        \
       unsigned mod_offset, unsigned slots, float eps, float attn_scale) {                                           \
    const ditb::Dims d{layers, T, D, heads, head_dim, mlp, mlp_span, ctx, cross_mask, mod_offset, slots, eps,        \
                       attn_scale};                                                                                  \
    ditb::run<NT>(table, seq, qkv, attn, ff, partial, group_counters, grid_counter, status, d);                      \
  }
AGI_DIT_BLOCKS_KERNEL(agi_coop_dit_blocks_bf16_t2, 2)   // up to 16 tokens
AGI_DIT_BLOCKS_KERNEL(agi_coop_dit_blocks_bf16_t3, 3)   // up to 24 tokens
#undef AGI_DIT_BLOCKS_KERNEL

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
//   * eight consumer warps load the activations of the phase (17 x 1536 bf16, normalised on the way in)
//     straight into registers, each warp its own K windows of them as MMA B fragments for the whole phase, and
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
//
// Measured on B200 (16 blocks x 1536, 17 tokens; SM-clock stamps of two CTAs): about 57 us per block, 3.9 ms per
// action chunk, against 2.9 ms for the same blocks as 27 separate launches chained by programmatic dependent
// launch - so recipes use it only on request.  Where a block's 57 us go, on the CTA with the most work:
//   * warp-level MMA: an m16n8k16 keeps a sub-core's tensor pipe ~30 cycles on this part, so the nine 16-row
//     units a CTA owns per block cost ~1.1 us each in the pipe alone (1.7 us with ring waits): 16 us;
//   * every CTA reads the whole 17 x 1536 activation matrix of a phase from L2 (148 readers of the same
//     52 KB): 1.3 us per phase; LayerNorm on top of it, redundantly in every CTA: 3-4 us per normalised phase;
//   * five phase boundaries at 1.6 us; the K-span arrival round of the MLP down projection: 4 us;
//   * attention of 32 heads on 64 of the 148 CTAs while the others wait: 6 us.
// Two things mattered on the way there and are kept: with nine or more warps a thread is capped at 168
// registers and the spills went to L2 (the L1 is a few KB under a 223 KB shared-memory carve-out), so the
// producer's warp group hands registers to the consumers (setmaxnreg: 40 / 232); and a load whose result feeds
// a select or a conversion straight away stalls the warp for the whole trip, so operands are fetched
// unconditionally from clamped addresses, as raw bits, and looked at only after everything is in flight.
#pragma once

#include "common.cuh"
#include "gemm_skinny.cuh"  // mma16n8
#include "gemm_stream.cuh"  // bulk copy and mbarrier helpers

namespace ditb {

constexpr int kConsumerWarps = 8;
constexpr unsigned kConsumers = kConsumerWarps * 32;
constexpr unsigned kThreads = kConsumers + 128;  // + the producer's warp group (one warp of it issues the copies)
// Registers per thread after the warp groups have traded (setmaxnreg): the launch gives each of the 12 warps
// 168; the producer's group keeps 40 and each consumer thread takes 232, which holds the B fragments of a
// phase, the accumulators and the epilogue operands without spilling.
constexpr unsigned kProducerRegs = 40, kConsumerRegs = 232;
constexpr unsigned kMaxSlots = 12;
constexpr unsigned kChunkWindows = 16;           // 64-byte K windows per ring slot row: 1 KB
constexpr unsigned kUnitRows = 16;               // output features per unit = rows of one MMA tile
constexpr unsigned kRingPitch = kChunkWindows * 64 + 64;   // +64: rows g, g+1 of a fragment fall into different bank halves
constexpr unsigned kSlotBytes = kUnitRows * kRingPitch;
constexpr unsigned kMaxSpan = 1536;              // K elements a consumer warp can keep as B fragments (6 windows x 8 warps)
constexpr unsigned kMaxChunks = kMaxSpan / 32 / kChunkWindows;   // 3
constexpr unsigned kHeaderBytes = 256;           // mbarriers and flags in front of the dynamic shared memory
constexpr unsigned kTableStride = 16;            // pointers per block in the table
constexpr unsigned kMaxLayers = 32;
constexpr unsigned kTableBytes = kMaxLayers * kTableStride * 8;   // the table's copy in shared memory
constexpr unsigned kTimeoutFull = 0x700, kTimeoutEmpty = 0x800, kTimeoutGrid = 0x900;
constexpr unsigned long long kGridWaitNs = 200ull * 1000 * 1000;

// Entries of a block's row in the pointer table.
enum : unsigned { kWq = 0, kBq, kWk, kBk, kWv, kBv, kWo, kBo, kW1, kB1, kW2, kB2, kMod, kCtxK, kCtxV };

struct Dims {
  unsigned layers, T, D, heads, head_dim, mlp, mlp_span, ctx, cross_mask, mod_offset, slots;
  float eps, attn_scale;
};

// One matrix-product phase of a block.  Phase 0 of a self-attention block has three weight matrices side by
// side along the output features (queries | keys | values); their pointers sit two table entries apart.
struct Gemm {
  unsigned w_entry, b_entry;            // table entries of the first weight matrix and its bias
  unsigned rows_per_mat, N, K, span, slices;
};

// phase: 0 queries (| keys | values), 1 attention output projection, 2 MLP up, 3 MLP down.
__device__ __forceinline__ Gemm phase_gemm(unsigned phase, bool cross, const Dims& d) {
  Gemm g;
  g.rows_per_mat = d.D;
  g.K = g.span = d.D;
  g.slices = 1;
  g.N = d.D;
  if (phase == 0) {
    g.w_entry = kWq; g.b_entry = kBq;
    if (!cross) g.N = 3 * d.D;
  } else if (phase == 1) {
    g.w_entry = kWo; g.b_entry = kBo;
  } else if (phase == 2) {
    g.w_entry = kW1; g.b_entry = kB1;
    g.N = g.rows_per_mat = d.mlp;
  } else {                   // K = mlp in spans
    g.w_entry = kW2; g.b_entry = kB2;
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
      const Gemm gm = phase_gemm(phase, cross, d);
      const unsigned groups = gm.N / kUnitRows, units = groups * gm.slices;
      const unsigned first = unsigned((unsigned long long)cta * units / ctas);
      const unsigned end = unsigned((unsigned long long)(cta + 1) * units / ctas);
      const unsigned windows = gm.span / 32;
      for (unsigned u = first; u < end; ++u) {
        const unsigned slice = u / groups, row0 = (u % groups) * kUnitRows;
        const unsigned mat = row0 / gm.rows_per_mat, local = row0 % gm.rows_per_mat;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(row[gm.w_entry + 2 * mat]) +
                             (size_t(local + (lane & 15u)) * gm.K + size_t(slice) * gm.span) * 2;
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
// Consumer side.  Everything below is inlined once into the kernel: what is the same for every thread of the
// CTA comes straight from the kernel parameters, what a thread owns stays in its registers.
// ---------------------------------------------------------------------------------------------------------

// Activations of a phase, straight from global memory into this thread's MMA B fragments: for token tile nt the
// lane (g, t) owns token nt * 8 + g and, of each K window its warp multiplies, the 16 bytes t (eight elements).
// mode 0: as they are;  mode 1: LayerNorm without affine;  mode 2: LayerNorm, then * (1 + scale) + shift (AdaLN).
// Row statistics: every lane sums its own elements, the four lanes of a quad add up, lane t == 0 leaves the warp's
// share in shared memory, and after a barrier every lane adds the eight shares of its tokens in warp order (two
// passes: mean, then the centred squares, as the stand-alone kernel does).  All loads are issued before the first
// reduction, so a phase pays one trip to L2 for its inputs.
template <int NT>
__device__ __forceinline__ void load_fragments(uint4 (&frag)[kMaxChunks][2][NT], float* stats, unsigned char* mod_tile,
                                               const bf16* src, unsigned ld, unsigned k0, unsigned cols, unsigned T,
                                               unsigned mode, const bf16* scale, const bf16* shift, float eps) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned windows = cols / 32;
  if (mode == 2) {
    // AdaLN (scale | shift) of the step: staged in shared memory by asynchronous copies that land under the two
    // statistics passes (no registers held meanwhile).  Committed as a group of its own, in front of any
    // key / value prefetch of this phase, so that waiting for it does not wait for that.
    for (unsigned i = threadIdx.x; i < cols / 4; i += kConsumers) {   // 16-byte pieces of scale, then of shift
      const unsigned piece = i % (cols / 8);
      const bf16* from = (i < cols / 8 ? scale : shift) + piece * 8;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(stream::smem_u32(mod_tile + size_t(i) * 16)), "l"(from)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  // Every load is unconditional (addresses clamped into the matrix) and issued before anything looks at a value.
#pragma unroll
  for (unsigned c = 0; c < kMaxChunks; ++c)
#pragma unroll
    for (unsigned j = 0; j < 2; ++j) {
      const unsigned win = min(c * kChunkWindows + warp + j * kConsumerWarps, windows - 1);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const unsigned m = min(unsigned(nt * 8) + g, T - 1);
        frag[c][j][nt] = __ldcg(reinterpret_cast<const uint4*>(src + size_t(m) * ld + k0 + win * 32 + t * 8));
      }
    }
  const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
  for (unsigned c = 0; c < kMaxChunks; ++c)
#pragma unroll
    for (unsigned j = 0; j < 2; ++j)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        if (c * kChunkWindows + warp + j * kConsumerWarps >= windows || unsigned(nt * 8) + g >= T) frag[c][j][nt] = zero;
  if (mode == 0) return;

  // The fragments stay packed between the passes: the compiler is told they may have changed, so that it
  // unpacks them again (two shifts per pair) instead of keeping 144 floats per thread alive across the barriers.
  auto repack = [&]() {
#pragma unroll
    for (unsigned c = 0; c < kMaxChunks; ++c)
#pragma unroll
      for (unsigned j = 0; j < 2; ++j)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
          asm volatile("" : "+r"(frag[c][j][nt].x), "+r"(frag[c][j][nt].y), "+r"(frag[c][j][nt].z), "+r"(frag[c][j][nt].w));
  };
  float mean[NT], rstd[NT];
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    repack();
    float part[NT];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float lanes[4] = {0.f, 0.f, 0.f, 0.f};   // four running sums keep the additions independent
#pragma unroll
      for (unsigned c = 0; c < kMaxChunks; ++c)
#pragma unroll
        for (unsigned j = 0; j < 2; ++j) {
          float f[8];
          unpack8(*reinterpret_cast<const Bf16x8*>(&frag[c][j][nt]), f);
          // windows past the span hold zeros: they add nothing in pass 0 and must not add mean^2 in pass 1
          const bool live = c * kChunkWindows + warp + j * kConsumerWarps < windows;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float dv = f[e] - mean[nt];
            lanes[e & 3] += pass == 0 ? f[e] : (live ? dv * dv : 0.f);
          }
        }
      part[nt] = (lanes[0] + lanes[1]) + (lanes[2] + lanes[3]);
      part[nt] += __shfl_xor_sync(0xffffffffu, part[nt], 1);
      part[nt] += __shfl_xor_sync(0xffffffffu, part[nt], 2);
    }
    float* share = stats + pass * kConsumerWarps * 8 * NT;   // [pass][warp][token]
    if (t == 0) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) share[warp * 8 * NT + nt * 8 + g] = part[nt];
    }
    if (pass == 1 && mode == 2) asm volatile("cp.async.wait_group 1;" ::: "memory");   // scale | shift have landed
    consumer_sync();
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float total = 0.f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) total += share[w * 8 * NT + nt * 8 + g];
      if (pass == 0) mean[nt] = total / float(cols);
      else rstd[nt] = rsqrtf(total / float(cols) + eps);
    }
  }
  repack();
#pragma unroll
  for (unsigned c = 0; c < kMaxChunks; ++c)
#pragma unroll
    for (unsigned j = 0; j < 2; ++j) {
      const unsigned win = c * kChunkWindows + warp + j * kConsumerWarps;
      if (win >= windows) continue;
      float a[8], b[8];
      if (mode == 2) {
        unpack8(*reinterpret_cast<const Bf16x8*>(mod_tile + (size_t(win) * 4 + t) * 16), a);
        unpack8(*reinterpret_cast<const Bf16x8*>(mod_tile + (size_t(cols / 8) + win * 4 + t) * 16), b);
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float f[8];
        unpack8(*reinterpret_cast<const Bf16x8*>(&frag[c][j][nt]), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          f[e] = (f[e] - mean[nt]) * rstd[nt];
          if (mode == 2) f[e] = f[e] * (1.f + a[e]) + b[e];
        }
        const Bf16x8 packed = pack8(f);
        frag[c][j][nt] = unsigned(nt * 8) + g < T ? *reinterpret_cast<const uint4*>(&packed) : zero;
      }
    }
}

// Keys and values of one head into the shared-memory tile (16-byte asynchronous copies through L2, one group);
// rows past kv_rows are zero-filled.  The caller waits for the group and synchronises before reading.
__device__ __forceinline__ void fetch_keys_values(unsigned char* tile, unsigned head, unsigned head_dim, const bf16* k,
                                                  const bf16* v, unsigned kv_stride, unsigned kv_rows) {
  const unsigned kv16 = (kv_rows + 15) & ~15u, pitch = head_dim + 8, vec_per_row = head_dim / 8;
  bf16* k_tile = reinterpret_cast<bf16*>(tile);
  bf16* v_tile = k_tile + size_t(kv16) * pitch;
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
}

// Attention of one (head, 16-query tile): tensor-core scores and P.V, the eight warps split the keys.
// `tile` holds the keys and values (fetch_keys_values, possibly still in flight), then the warps' partial results.
__device__ __forceinline__ void attention_task(unsigned char* tile, unsigned head, unsigned row_base, unsigned head_dim,
                                               unsigned q_rows, float scale, const bf16* q, unsigned q_stride,
                                               unsigned kv_rows, bf16* o, unsigned o_stride) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned kv16 = (kv_rows + 15) & ~15u;
  const unsigned pitch = head_dim + 8;
  bf16* k_tile = reinterpret_cast<bf16*>(tile);
  bf16* v_tile = k_tile + size_t(kv16) * pitch;
  float* merge = reinterpret_cast<float*>(tile);         // written after every warp has finished with the keys
  const unsigned ksteps = head_dim / 16;   // <= 4
  unsigned qa[4][4];
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      // unconditional, clamped into the head: every load is in flight before the first value is used
      const unsigned row = row_base + g + (r & 1) * 8, col = min(unsigned(ks), ksteps - 1) * 16 + 2 * t + (r >> 1) * 8;
      qa[ks][r] = __ldcg(reinterpret_cast<const unsigned*>(q + size_t(min(row, q_rows - 1)) * q_stride + head * head_dim + col));
    }
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const bf162*>(&qa[ks][r]));
      const bf162 scaled = __floats2bfloat162_rn(f.x * scale, f.y * scale);
      qa[ks][r] = unsigned(ks) < ksteps && row_base + g + (r & 1) * 8 < q_rows ? *reinterpret_cast<const unsigned*>(&scaled) : 0u;
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

// Dynamic shared memory of the kernel for a given shape (the recipe builder mirrors these formulas): header,
// then the consumers' exchange area (partial tiles of the warps, row statistics, arrival flags), then the
// attention tile (keys and values of one head, later the warps' partial results), then the weight ring.
__host__ __device__ constexpr unsigned round_up(unsigned v, unsigned to) { return (v + to - 1) / to * to; }
__host__ __device__ constexpr unsigned exchange_bytes(unsigned T) {
  return kTableBytes + round_up(kConsumerWarps * 16 * (T | 1u) * 4 + 2 * kConsumerWarps * 24 * 4 + 64, 128) + 4 * kMaxSpan;
}
__host__ __device__ constexpr unsigned attention_bytes(unsigned T, unsigned head_dim, unsigned ctx) {
  const unsigned keys = round_up(ctx > T ? ctx : T, 16);
  const unsigned kv_bytes = 2 * keys * (head_dim + 8) * 2, merge_bytes = kConsumerWarps * 16 * (head_dim + 2) * 4;
  return round_up(kv_bytes > merge_bytes ? kv_bytes : merge_bytes, 128);
}

template <int NT>
__device__ __forceinline__ void run(const unsigned long long* table, bf16* seq, bf16* qkv, bf16* attn, bf16* ff, float* partial,
                                    unsigned* group_counters, unsigned* grid_counter, unsigned* status, const Dims& d) {
  extern __shared__ __align__(128) unsigned char dit_smem[];
  unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(dit_smem);
  unsigned long long* empty_bar = full_bar + kMaxSlots;
  // [0] = this CTA gave up, [2] = [0] as of the last phase boundary, [4..11] = "last arriver" per unit of a phase
  volatile unsigned* flags = reinterpret_cast<volatile unsigned*>(empty_bar + kMaxSlots);
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned D = d.D, T = d.T, mp = T | 1u;

  if (threadIdx.x == 0) {
    for (unsigned s = 0; s < kMaxSlots; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(stream::smem_u32(&full_bar[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(stream::smem_u32(&empty_bar[s])), "n"(kConsumerWarps));
    }
    for (unsigned i = 0; i < 12; ++i) flags[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  grid_dependency_wait();   // the table and the residual stream come from earlier launches
  // the blocks' pointers: read many times by both roles, so they are copied next to the header once
  unsigned long long* const table_s = reinterpret_cast<unsigned long long*>(dit_smem + kHeaderBytes);
  for (unsigned i = threadIdx.x; i < d.layers * kTableStride; i += kThreads) table_s[i] = table[i];
  __syncthreads();
  table = table_s;
  float* const part_tile = reinterpret_cast<float*>(dit_smem + kHeaderBytes + kTableBytes);    // [warp][16][T | 1]
  float* const stats = part_tile + kConsumerWarps * 16 * mp;                     // [pass][warp][token]
  unsigned char* const mod_tile = dit_smem + kHeaderBytes + exchange_bytes(T) - 4 * kMaxSpan;   // AdaLN scale | shift
  unsigned char* const attn_tile = dit_smem + kHeaderBytes + exchange_bytes(T);
  const unsigned ring_base = stream::smem_u32(attn_tile + attention_bytes(T, d.head_dim, d.ctx));

  if (warp >= kConsumerWarps) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kProducerRegs));
    if (warp == kConsumerWarps) produce(table, d, status, ring_base, full_bar, empty_bar);
    return;
  }
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));

  const unsigned cta = blockIdx.x, ctas = gridDim.x;
  const unsigned q_tiles = (T + 15) / 16, tasks = d.heads * q_tiles;
  unsigned slot = 0, round = 0;          // position in the ring: the same walk as the producer's
  unsigned boundaries = 0;               // phase boundaries passed so far
  const unsigned steps = 5 * d.layers;   // five phases per block

  for (unsigned step = 0; step < steps; ++step) {
    const unsigned layer = step / 5, phase5 = step % 5;
    const unsigned long long* row = table + size_t(layer) * kTableStride;
    const bool cross = (d.cross_mask >> layer) & 1u;
    if (phase5 == 1) {
      // ---------------- attention: one (head, query tile) per CTA ----------------
      const bf16* keys = cross ? reinterpret_cast<const bf16*>(row[kCtxK]) : qkv + D;
      const bf16* values = cross ? reinterpret_cast<const bf16*>(row[kCtxV]) : qkv + 2 * D;
      const unsigned kv_stride = cross ? D : 3 * D, kv_rows = cross ? d.ctx : T;
      for (unsigned task = cta; task < tasks; task += ctas) {
        // the context tokens' keys and values of a CTA's first task were requested a phase ago
        if (!cross || task != cta) fetch_keys_values(attn_tile, task / q_tiles, d.head_dim, keys, values, kv_stride, kv_rows);
        attention_task(attn_tile, task / q_tiles, (task % q_tiles) * 16, d.head_dim, T, d.attn_scale, qkv, 3 * D, kv_rows,
                       attn, D);
      }
    } else {
      // ---------------- a matrix product ----------------
      // kind 0: y = bf16(acc + bias)            queries (| keys | values) of the modulated, normalised stream
      // kind 1: y = bf16(acc + bias + y)        output projection onto the residual stream
      // kind 2: y = bf16(gelu(acc + bias))      MLP up of the normalised stream
      // kind 3: K spans: partial sums to `partial`; the last arriver of a feature group adds them, + bias + y
      const unsigned kind = phase5 == 0 ? 0u : phase5 - 1;
      // keys and values of the context tokens for this CTA's attention task: requested in this phase (behind the
      // AdaLN group, whose wait counts on being the older one), landing while the queries are computed
      bool prefetch = kind == 0 && cross && cta < tasks;
      const Gemm gm = phase_gemm(kind, cross, d);
      const bf16* x = kind == 0 || kind == 2 ? seq : kind == 1 ? attn : ff;
      const unsigned ldx = kind == 3 ? d.mlp : D;
      const unsigned x_mode = kind == 0 ? 2u : kind == 2 ? 1u : 0u;
      bf16* y = kind == 0 ? qkv : kind == 2 ? ff : seq;
      const unsigned ldy = kind == 0 ? 3 * D : kind == 2 ? d.mlp : D;
      const bf16* mod = reinterpret_cast<const bf16*>(row[kMod]) + d.mod_offset;   // (scale | shift) of this step
      const bool spans = kind == 3 && gm.slices > 1;
      const bool residual = kind == 1 || (kind == 3 && !spans);

      const unsigned groups = gm.N / kUnitRows, units = groups * gm.slices;
      const unsigned first = unsigned((unsigned long long)cta * units / ctas);
      const unsigned end = unsigned((unsigned long long)(cta + 1) * units / ctas);
      const unsigned windows = gm.span / 32;
      // this thread's (at most two) outputs of a unit: elements e and e + 256 of the 16 x T tile, feature-major
      const unsigned e0 = threadIdx.x, e1 = threadIdx.x + kConsumers;
      const bool live0 = e0 < kUnitRows * T, live1 = e1 < kUnitRows * T;
      uint4 bfrag[kMaxChunks][2][NT];
      unsigned have_slice = 0xffffffffu;
      for (unsigned u = first; u < end; ++u) {
        const unsigned slice = u / groups, row0 = (u % groups) * kUnitRows;
        if (slice != have_slice) {
          if (x_mode == 2 && !prefetch) asm volatile("cp.async.wait_group 0;" ::: "memory");   // nothing older than AdaLN's group
          load_fragments<NT>(bfrag, stats, mod_tile, x, ldx, slice * gm.span, gm.span, T, x_mode, mod, mod + D, d.eps);
          have_slice = slice;
        }
        if (prefetch) {
          fetch_keys_values(attn_tile, cta / q_tiles, d.head_dim, reinterpret_cast<const bf16*>(row[kCtxK]),
                            reinterpret_cast<const bf16*>(row[kCtxV]), D, d.ctx);
          prefetch = false;
        }
        // what the epilogue adds is requested now and used after the multiplication
        const unsigned mat = row0 / gm.rows_per_mat, local = row0 % gm.rows_per_mat;
        const bf16* bias = reinterpret_cast<const bf16*>(row[gm.b_entry + 2 * mat]) + local;
        bf16* out0 = y + size_t(e0 / kUnitRows) * ldy + row0 + e0 % kUnitRows;
        bf16* out1 = y + size_t(e1 / kUnitRows) * ldy + row0 + e1 % kUnitRows;
        // (raw bits: nothing converts, and so waits for, a value before the multiplication has been issued;
        //  a thread without a second output re-reads its first)
        const bf16* out1_or_0 = live1 ? out1 : out0;
        const unsigned short add0_bits = *reinterpret_cast<const unsigned short*>(bias + e0 % kUnitRows);
        const unsigned short add1_bits = *reinterpret_cast<const unsigned short*>(bias + e1 % kUnitRows);
        unsigned short res0_bits = 0, res1_bits = 0;
        if (residual) {
          res0_bits = __ldcg(reinterpret_cast<const unsigned short*>(live0 ? out0 : y));
          res1_bits = __ldcg(reinterpret_cast<const unsigned short*>(out1_or_0));
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
          if (flags[0] == 0 && !wait_slot(stream::smem_u32(&full_bar[slot]), round & 1, status, kTimeoutFull | slot)) flags[0] = 1;
          const unsigned base = ring_base + slot * kSlotBytes + g * kRingPitch + t * 16;
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
          if (lane == 0) stream::arrive(stream::smem_u32(&empty_bar[slot]));
          if (++slot == d.slots) { slot = 0; ++round; }
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
        float total0 = 0.f, total1 = 0.f;
#pragma unroll
        for (int wq = 0; wq < kConsumerWarps; ++wq) {   // e1 is folded back into the tile for the threads without one
          total0 += part_tile[(wq * 16 + e0 % kUnitRows) * mp + min(e0 / kUnitRows, T - 1)];
          total1 += part_tile[(wq * 16 + e1 % kUnitRows) * mp + min(e1 / kUnitRows, T - 1)];
        }
        if (spans) {
          float* slab = partial + size_t(slice) * T * gm.N + row0;
          if (live0) slab[size_t(e0 / kUnitRows) * gm.N + e0 % kUnitRows] = total0;
          if (live1) slab[size_t(e1 / kUnitRows) * gm.N + e1 % kUnitRows] = total1;
        } else {
          const float add0 = __uint_as_float(unsigned(add0_bits) << 16), add1 = __uint_as_float(unsigned(add1_bits) << 16);
          const float res0 = __uint_as_float(unsigned(res0_bits) << 16), res1 = __uint_as_float(unsigned(res1_bits) << 16);
          float v0 = total0 + add0, v1 = total1 + add1;
          if (kind == 2) {
            v0 = gelu_tanh(v0);
            v1 = gelu_tanh(v1);
          }
          if (live0) *out0 = __float2bfloat16_rn(v0 + res0);
          if (live1) *out1 = __float2bfloat16_rn(v1 + res1);
        }
        consumer_sync();   // the partial tiles may be overwritten from here on
      }
      if (prefetch)
        fetch_keys_values(attn_tile, cta / q_tiles, d.head_dim, reinterpret_cast<const bf16*>(row[kCtxK]),
                          reinterpret_cast<const bf16*>(row[kCtxV]), D, d.ctx);
      if (spans) {
        // One arrival round for all of this CTA's units: each K span counts in for its feature group; whoever
        // completes a group adds its spans in order (bit-reproducible), with bias and residual.
        for (unsigned batch = first; batch < end; batch += 8) {
          const unsigned n = min(8u, end - batch);
          if (threadIdx.x < n) {
            const unsigned group = (batch + threadIdx.x) % groups;
            __threadfence();
            const unsigned before = atomicAdd(&group_counters[group], 1u);
            flags[4 + threadIdx.x] = before == gm.slices - 1 ? 1u : 0u;
            if (before == gm.slices - 1) {
              __threadfence();
              group_counters[group] = 0;   // every span has arrived: nobody touches the counter before the next block
            }
          }
          consumer_sync();
          for (unsigned i = 0; i < n; ++i) {
            if (flags[4 + i] == 0) continue;
            const unsigned row0 = ((batch + i) % groups) * kUnitRows;
            const bf16* bias = reinterpret_cast<const bf16*>(row[gm.b_entry]) + row0;
#pragma unroll
            for (unsigned half = 0; half < 2; ++half) {
              const unsigned e = threadIdx.x + half * kConsumers;
              if (e >= kUnitRows * T) continue;
              const unsigned r = e % kUnitRows, m = e / kUnitRows;
              bf16* out = y + size_t(m) * ldy + row0 + r;
              float parts[8];
#pragma unroll
              for (unsigned sl = 0; sl < 8; ++sl)
                parts[sl] = __ldcg(partial + (size_t(min(sl, gm.slices - 1)) * T + m) * gm.N + row0 + r);
              float total = __bfloat162float(bias[r]) + __bfloat162float(__ldcg(out));
              float sum = 0.f;
#pragma unroll
              for (unsigned sl = 0; sl < 8; ++sl) sum += sl < gm.slices ? parts[sl] : 0.f;
              for (unsigned sl = 8; sl < gm.slices; ++sl) sum += __ldcg(partial + (size_t(sl) * T + m) * gm.N + row0 + r);
              *out = __float2bfloat16_rn(sum + total);
            }
          }
          consumer_sync();   // the flags are reused by the next batch
        }
      }
    }
    if (step + 1 == steps) break;   // the last block's results are ordered by the end of the kernel

    // ---------------- grid-wide phase boundary ----------------
    // Everything this CTA wrote is ordered before its arrival; everything other CTAs wrote before theirs is
    // visible (through L2: readers use ld.cg / cp.async.cg) after the wait.
    ++boundaries;
    consumer_sync();
    if (threadIdx.x == 0) {
      if (flags[0] == 0) {
        __threadfence();
        atomicAdd(grid_counter, 1u);
        const unsigned target = boundaries * ctas;
        const unsigned long long t0 = global_ns();
        unsigned spin = 0;
        while (load_acquire(grid_counter) < target) {
          if ((++spin & 63u) == 0) {
            if (load_relaxed(status) != 0) { flags[0] = 1; break; }
            if (global_ns() - t0 > kGridWaitNs) {
              atomicCAS(status, 0u, kTimeoutGrid | (boundaries & 0xffu));
              flags[0] = 1;
              break;
            }
          }
        }
        __threadfence();
      }
      flags[2] = flags[0];   // the verdict every thread acts on: written only between this boundary's two syncs
    }
    consumer_sync();
    if (flags[2] != 0) break;   // this CTA or another one gave up: the same answer for every consumer thread
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");   // nothing of this CTA's is in flight when it leaves
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

// A stack of DiT blocks in one launch.  grid = (number of SMs, 1, 1), one CTA per SM, block = 384 threads
// (8 consumer warps + the producer's warp group); dynamic shared memory = 256 + exchange_bytes(T) +
// attention_bytes(T, head_dim, ctx) + slots * 17408.
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

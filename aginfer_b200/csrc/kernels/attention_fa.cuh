// Tensor-core attention for many query rows (prefill: 288 causal tokens with 128-wide heads; the vision
// tower: 512 patch tokens, 80-wide heads, block-diagonal windows).  Streaming-softmax formulation on
// warp-level MMAs:
//
//   * one block of 1, 2 or 4 warps per (16, 32 or 64 query rows, head): fewer rows per block when the grid
//     would otherwise leave most SMs idle; warp w owns rows 16w ... 16w + 15 and keeps its Q
//     fragments, running row maxima / sums and the output accumulators in registers;
//   * keys are visited in tiles of 64: K and V tiles are staged row-major in shared memory by 16-byte
//     asynchronous copies, double-buffered so that tile i + 1 lands while tile i is multiplied;
//   * S = Q.K^T on m16n8k16 (a K row is the "col" B operand as it lies), mask, running maximum, P = exp(S - m)
//     reused in place as the A operand of P.V, V through ldmatrix.trans;
//   * only key tiles a block of rows can see are visited: the causal prefix, or the diagonal block(s).
//
// Head width is a template parameter (16-element steps); grouped-query attention maps query head h to KV
// head h / (q_heads / kv_heads).  Pitch of the shared tiles = head_dim + 8 elements: rows stay 16-byte
// aligned and the eight rows of a fragment fall into different banks.
// grid = (ceil(q_rows / (16 * warps)), q_heads), block = 32 * warps, dynamic shared memory = 4 * 64 * (head_dim + 8) * 2.
#pragma once

#include "attention.cuh"

namespace fa {

constexpr unsigned kKeyTile = 64;

template <int HD16>
__device__ __forceinline__ void attention_body(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows,
                                               unsigned kv_rows, unsigned q_heads, unsigned kv_heads, unsigned q_stride,
                                               unsigned k_stride, unsigned v_stride, unsigned o_stride, float scale,
                                               unsigned mask_mode, unsigned mask_arg, unsigned* amax_bits = nullptr) {
  constexpr unsigned head_dim = HD16 * 16, pitch = head_dim + 8, vec_per_row = head_dim / 8;
  extern __shared__ __align__(16) unsigned char attn_smem[];
  bf16* tiles = reinterpret_cast<bf16*>(attn_smem);   // [2 buffers][K | V][64][pitch]
  grid_dependency_wait();
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const unsigned head = blockIdx.y, kv_head = head / (q_heads / kv_heads);
  const unsigned rows_per_block = (blockDim.x >> 5) * 16;   // one 16-row MMA tile per warp; 1, 2 or 4 warps
  const unsigned row_base = blockIdx.x * rows_per_block, warp_row = row_base + warp * 16;
  const unsigned last_row = min(row_base + rows_per_block, q_rows) - 1;

  // keys this block of rows can see
  unsigned key_begin = 0, key_end = kv_rows;
  if (mask_mode == 1) key_end = min(kv_rows, last_row + mask_arg + 1);
  if (mask_mode == 2) {
    key_begin = (row_base / mask_arg) * mask_arg;
    key_end = min(kv_rows, (last_row / mask_arg + 1) * mask_arg);
  }
  const unsigned tiles_total = key_end > key_begin ? (key_end - key_begin + kKeyTile - 1) / kKeyTile : 0;

  auto stage = [&](unsigned tile, unsigned buffer) {
    bf16* k_tile = tiles + size_t(buffer) * 2 * kKeyTile * pitch;
    bf16* v_tile = k_tile + kKeyTile * pitch;
    const unsigned key0 = key_begin + tile * kKeyTile;
    for (unsigned i = threadIdx.x; i < kKeyTile * vec_per_row; i += blockDim.x) {
      const unsigned j = i / vec_per_row, d = (i % vec_per_row) * 8;
      const unsigned key = key0 + j, src_row = min(key, kv_rows - 1), bytes = key < kv_rows ? 16u : 0u;  // zero-fill past the end
      const unsigned kd = static_cast<unsigned>(__cvta_generic_to_shared(k_tile + j * pitch + d));
      const unsigned vd = static_cast<unsigned>(__cvta_generic_to_shared(v_tile + j * pitch + d));
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(kd),
                   "l"(k + size_t(src_row) * k_stride + kv_head * head_dim + d), "r"(bytes) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vd),
                   "l"(v + size_t(src_row) * v_stride + kv_head * head_dim + d), "r"(bytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  if (tiles_total > 0) stage(0, 0);

  // Q fragments (A operand) as stored: rows g and g + 8 of this warp's 16; zero past q_rows.  The softmax
  // scale is applied to the fp32 scores, so no second rounding of Q.
  unsigned qa[HD16][4];
#pragma unroll
  for (int ks = 0; ks < HD16; ++ks)
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      qa[ks][r] = 0;
      const unsigned row = warp_row + g + (r & 1) * 8, col = ks * 16 + 2 * t + (r >> 1) * 8;
      if (row < q_rows) {
        qa[ks][r] = *reinterpret_cast<const unsigned*>(q + size_t(row) * q_stride + head * head_dim + col);
      }
    }

  float row_max[2] = {-3.0e38f, -3.0e38f}, row_sum[2] = {0.f, 0.f}, out[2 * HD16][4];
#pragma unroll
  for (int nt = 0; nt < 2 * HD16; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) out[nt][i] = 0.f;

  for (unsigned tile = 0; tile < tiles_total; ++tile) {
    const unsigned buffer = tile & 1;
    if (tile + 1 < tiles_total) {
      stage(tile + 1, buffer ^ 1);                       // that buffer was released by the barrier below
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const bf16* k_tile = tiles + size_t(buffer) * 2 * kKeyTile * pitch;
    const bf16* v_tile = k_tile + kKeyTile * pitch;
    const unsigned key0 = key_begin + tile * kKeyTile;
    // a warp whose rows see nothing of this tile skips the arithmetic (but not the barriers)
    const unsigned warp_last = min(warp_row + 15, q_rows - 1);
    bool any = warp_row < q_rows;
    if (mask_mode == 1) any = any && key0 <= warp_last + mask_arg;
    if (mask_mode == 2) any = any && key0 < (warp_last / mask_arg + 1) * mask_arg && key0 + kKeyTile > (warp_row / mask_arg) * mask_arg;
    if (any) {
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
        const bf16* row = k_tile + (nt * 8 + g) * pitch + 2 * t;
#pragma unroll
        for (int ks = 0; ks < HD16; ++ks) {
          const unsigned b0 = *reinterpret_cast<const unsigned*>(row + ks * 16);
          const unsigned b1 = *reinterpret_cast<const unsigned*>(row + ks * 16 + 8);
          skinny_mma_bf16(s[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        }
      }
      // mask: c0,c1 belong to row g (keys 2t, 2t+1 of the 8-key tile), c2,c3 to row g + 8
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const unsigned key = key0 + nt * 8 + 2 * t + (i & 1), row = warp_row + g + (i >> 1) * 8;
          bool visible = key < kv_rows;
          if (mask_mode == 1) visible = visible && key <= row + mask_arg;
          if (mask_mode == 2) visible = visible && key / mask_arg == row / mask_arg;
          s[nt][i] = visible ? s[nt][i] * scale : -3.0e38f;
        }
      unsigned pa[4][4];   // [16-key step][a0..a3]
#pragma unroll
      for (int hr = 0; hr < 2; ++hr) {   // hr 0: row g, hr 1: row g + 8
        float tile_max = -3.0e38f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) tile_max = fmaxf(tile_max, fmaxf(s[nt][2 * hr], s[nt][2 * hr + 1]));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 1));
        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 2));
        const float new_max = fmaxf(row_max[hr], tile_max);
        const float rescale = new_max > -1.0e38f ? __expf(row_max[hr] - new_max) : 1.f;
        float tile_sum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          const float s0 = s[nt][2 * hr], s1 = s[nt][2 * hr + 1];
          const float p0 = s0 > -1.0e38f ? __expf(s0 - new_max) : 0.f;
          const float p1 = s1 > -1.0e38f ? __expf(s1 - new_max) : 0.f;
          tile_sum += p0 + p1;
          const bf162 pair = __floats2bfloat162_rn(p0, p1);
          // A operand of P.V for 16-key step nt / 2: a0/a1 = rows g / g + 8 of the first 8 keys, a2/a3 of the second
          pa[nt >> 1][(nt & 1) * 2 + hr] = *reinterpret_cast<const unsigned*>(&pair);
        }
        tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, 1);
        tile_sum += __shfl_xor_sync(0xffffffffu, tile_sum, 2);
        row_sum[hr] = row_sum[hr] * rescale + tile_sum;
        row_max[hr] = new_max;
#pragma unroll
        for (int nt = 0; nt < 2 * HD16; ++nt) {
          out[nt][2 * hr] *= rescale;
          out[nt][2 * hr + 1] *= rescale;
        }
      }
      // O += P (16 x 64 keys) . V (64 keys x head_dim): per 16 keys and 8 dims one MMA; ldmatrix with transpose
      // turns two 8 x 8 blocks of row-major V into the B fragment
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int nt = 0; nt < 2 * HD16; ++nt) {
          const unsigned addr = static_cast<unsigned>(__cvta_generic_to_shared(v_tile + (kk * 16 + (lane & 15)) * pitch + nt * 8));
          unsigned b0, b1;
          asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
          skinny_mma_bf16(out[nt], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
        }
    }
    __syncthreads();   // everyone is done with this buffer before it is refilled
  }

  float best = 0.f;   // max |o| over this thread's outputs, for a following dynamic quantisation
#pragma unroll
  for (int hr = 0; hr < 2; ++hr) {
    const unsigned row = warp_row + g + hr * 8;
    if (row >= q_rows) continue;
    const float inv = row_sum[hr] > 0.f ? 1.f / row_sum[hr] : 0.f;
    bf16* dst = o + size_t(row) * o_stride + head * head_dim + 2 * t;
#pragma unroll
    for (int nt = 0; nt < 2 * HD16; ++nt) {
      const float a = out[nt][2 * hr] * inv, b = out[nt][2 * hr + 1] * inv;
      best = fmaxf(best, fmaxf(fabsf(a), fabsf(b)));
      *reinterpret_cast<bf162*>(dst + nt * 8) = __floats2bfloat162_rn(a, b);
    }
  }
  if (amax_bits != nullptr) {   // rounding is monotonic: the rounded maximum is the maximum of the rounded outputs
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) best = fmaxf(best, __shfl_xor_sync(0xffffffffu, best, offset));
    if (lane == 0) atomicMax(amax_bits, __float_as_uint(__bfloat162float(__float2bfloat16_rn(best))));
  }
}

}  // namespace fa

#define AGI_ATTENTION_FA(NAME, HD16)                                                                                 \
  extern "C" __global__ void __launch_bounds__(128)                                                                  \
  NAME(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows, unsigned q_heads,    \
       unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride, unsigned v_stride,               \
       unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg) {                                      \
    fa::attention_body<HD16>(q, k, v, o, q_rows, kv_rows, q_heads, kv_heads, q_stride, k_stride, v_stride, o_stride, \
                             scale, mask_mode, mask_arg);                                                            \
  }
// the same, also folding max |o| into *amax_bits (a zero-initialised word)
#define AGI_ATTENTION_FA_AMAX(NAME, HD16)                                                                            \
  extern "C" __global__ void __launch_bounds__(128)                                                                  \
  NAME(const bf16* q, const bf16* k, const bf16* v, bf16* o, unsigned q_rows, unsigned kv_rows, unsigned q_heads,    \
       unsigned kv_heads, unsigned head_dim, unsigned q_stride, unsigned k_stride, unsigned v_stride,               \
       unsigned o_stride, float scale, unsigned mask_mode, unsigned mask_arg, unsigned* amax_bits) {                 \
    fa::attention_body<HD16>(q, k, v, o, q_rows, kv_rows, q_heads, kv_heads, q_stride, k_stride, v_stride, o_stride, \
                             scale, mask_mode, mask_arg, amax_bits);                                                 \
  }
AGI_ATTENTION_FA_AMAX(agi_attention_fa_amax_bf16_d80, 5)
AGI_ATTENTION_FA_AMAX(agi_attention_fa_amax_bf16_d128, 8)
#undef AGI_ATTENTION_FA_AMAX
AGI_ATTENTION_FA(agi_attention_fa_bf16_d48, 3)
AGI_ATTENTION_FA(agi_attention_fa_bf16_d64, 4)
AGI_ATTENTION_FA(agi_attention_fa_bf16_d80, 5)
AGI_ATTENTION_FA(agi_attention_fa_bf16_d128, 8)
#undef AGI_ATTENTION_FA

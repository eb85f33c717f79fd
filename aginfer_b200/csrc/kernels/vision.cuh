// Indexing kernels of the vision tower (bit-exact tier: pure data movement plus one bf16 rounding).
//
// Token order.  The tower works on patch tokens in WINDOW ORDER so that every attention window is a run
// of consecutive rows (block-diagonal mask) and every 2 x 2 merge group is four consecutive rows (the
// merger's concatenation is then a reshape):
//     token = image * P*P + window * W*W + group * m*m + sub
// with P patches per image side, W patches per window side, m = merge size; window = wy * (P/W) + wx,
// group = gy * (W/m) + gx, sub = sy * m + sx, and the patch sits at
//     (py, px) = (wy * W + gy * m + sy, wx * W + gx * m + sx).
// agi_patchify_f32_bf16 builds that order directly from the pixels (the window permutation is fused into
// the patch gather); agi_unwindow_rows_bf16 puts merged tokens back into raster order, which is where the
// language model expects them.
#pragma once

#include "common.cuh"

// pixels [images, channels, size, size] fp32 -> out [images * P * P, out_stride] bf16, row = token in window
// order, column e = ((c * temporal + t) * patch + iy) * patch + ix (the still image repeated for each of the
// `temporal` frames), columns past channels * temporal * patch^2 zero-filled up to `cols`;
// pos [3, tokens] int32 = (py, px, 0): the 2-D rotary positions of each token.
extern "C" __global__ void agi_patchify_f32_bf16(const float* pixels, bf16* out, int* pos, unsigned images,
                                                 unsigned channels, unsigned size, unsigned patch, unsigned temporal,
                                                 unsigned window, unsigned merge, unsigned cols, unsigned out_stride) {
  grid_dependency_wait();
  const unsigned P = size / patch, per_image = P * P, tokens = images * per_image;
  const unsigned wins = P / window, groups = window / merge;
  const unsigned patch_elems = channels * temporal * patch * patch;
  const size_t total = size_t(tokens) * cols;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
    const unsigned token = unsigned(i / cols), e = unsigned(i % cols);
    const unsigned image = token / per_image, in_image = token % per_image;
    const unsigned win = in_image / (window * window), in_win = in_image % (window * window);
    const unsigned group = in_win / (merge * merge), sub = in_win % (merge * merge);
    const unsigned py = (win / wins) * window + (group / groups) * merge + sub / merge;
    const unsigned px = (win % wins) * window + (group % groups) * merge + sub % merge;
    if (e == 0) {
      pos[token] = int(py);
      pos[tokens + token] = int(px);
      pos[2 * tokens + token] = 0;
    }
    float value = 0.f;
    if (e < patch_elems) {
      const unsigned ix = e % patch, iy = (e / patch) % patch, c = e / (patch * patch * temporal);
      value = pixels[((size_t(image) * channels + c) * size + py * patch + iy) * size + px * patch + ix];
    }
    out[size_t(token) * out_stride + e] = __float2bfloat16_rn(value);
  }
}

// in [images * G * G, in_stride] merged tokens in window order (G merged tokens per image side, w per window
// side) -> out rows in raster order: out[image * G*G + y * G + x].  cols % 8 == 0.
extern "C" __global__ void agi_unwindow_rows_bf16(const bf16* in, bf16* out, unsigned images, unsigned G, unsigned w,
                                                  unsigned cols, unsigned in_stride, unsigned out_stride) {
  grid_dependency_wait();
  const unsigned per_row = cols / 8, per_image = G * G, wins = G / w;
  const unsigned total = images * per_image * per_row;
  for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const unsigned row = i / per_row, c = (i % per_row) * 8;
    const unsigned image = row / per_image, in_image = row % per_image;
    const unsigned win = in_image / (w * w), group = in_image % (w * w);
    const unsigned y = (win / wins) * w + group / w, x = (win % wins) * w + group % w;
    const uint4 v = *reinterpret_cast<const uint4*>(in + size_t(row) * in_stride + c);
    *reinterpret_cast<uint4*>(out + size_t(image * per_image + y * G + x) * out_stride + c) = v;
  }
}

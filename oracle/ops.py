"""Per-kernel oracles (fp32 math on CPU; results rounded to the storage type the kernel writes)."""
from __future__ import annotations

import math

import torch

E4M3_MAX = 448.0


def bf16_round(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16)


def quantize_e4m3(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-tensor dynamic E4M3 quantisation: ``scale = amax / 448`` (1 when amax == 0, so an
    all-zero tensor stays finite), ``q = e4m3(x / scale)`` with IEEE fp32 division,
    round-to-nearest-even and saturation to +-448.  Returns (q as float8_e4m3fn, scale fp32)."""
    xf = x.float()
    amax = xf.abs().max()
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = (xf / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale.reshape(())


def gelu_tanh(x: torch.Tensor) -> torch.Tensor:
    return 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))


def gemm(x: torch.Tensor, w: torch.Tensor, *, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
         act: str | None = None, scale_a: torch.Tensor | None = None, scale_w: torch.Tensor | None = None,
         out_f32: bool = False) -> torch.Tensor:
    """Y = epilogue(X . W^T) with X [M, K], W [N, K] (bf16 or float8_e4m3fn), fp32 accumulation.
    Epilogue order: * (scale_a * scale_w), + bias, activation, + residual, round."""
    acc = x.float() @ w.float().t()
    if scale_a is not None:
        acc = acc * (scale_a.float() * scale_w.float())
    if bias is not None:
        acc = acc + bias.float()
    if act == "gelu_tanh":
        acc = gelu_tanh(acc)
    elif act == "silu":
        acc = acc * torch.sigmoid(acc)
    elif act == "relu":
        acc = torch.relu(acc)
    if residual is not None:
        acc = acc + residual.float()
    return acc if out_f32 else bf16_round(acc)


def rmsnorm(x: torch.Tensor, gain: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    return bf16_round(xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gain.float())


def layernorm(x: torch.Tensor, eps: float = 1e-5, scale: torch.Tensor | None = None,
              shift: torch.Tensor | None = None) -> torch.Tensor:
    """LayerNorm without affine parameters; with ``scale``/``shift``: AdaLN ``LN(x) * (1 + scale) + shift``."""
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = (xf - mean).pow(2).mean(-1, keepdim=True)
    y = (xf - mean) * torch.rsqrt(var + eps)
    if scale is not None:
        y = y * (1.0 + scale.float()) + shift.float()
    return bf16_round(y)


def _rotate(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x [rows, heads, head_dim], angles [rows, head_dim / 2]; half-split pairing (i, i + d/2)."""
    half = x.shape[-1] // 2
    a, b = x[..., :half].float(), x[..., half:].float()
    c, s = angles.cos()[:, None, :], angles.sin()[:, None, :]
    return bf16_round(torch.cat([a * c - b * s, b * c + a * s], dim=-1))


def rope(x: torch.Tensor, theta: float, pos_offset: int = 0) -> torch.Tensor:
    """1-D rotary embedding over x [rows, heads, head_dim], positions row + pos_offset."""
    rows, _, d = x.shape
    inv_freq = theta ** (-torch.arange(0, d, 2, dtype=torch.float32) / d)
    pos = torch.arange(rows, dtype=torch.float32) + pos_offset
    return _rotate(x, pos[:, None] * inv_freq[None, :])


def mrope(x: torch.Tensor, positions: torch.Tensor, theta: float, sections: tuple[int, int, int],
          ladder: int | None = None) -> torch.Tensor:
    """Multimodal rotary embedding: positions [3, rows] (temporal, height, width); rotary pair i uses
    stream 0 for i < s0, stream 1 for i < s0 + s1, else stream 2, and turns at theta^(-(i mod ladder) / ladder).
    ``ladder`` defaults to d / 2 (one frequency ladder over all pairs, as in a language model); a vision tower's
    2-D rotary has d / 4: the same ladder for the row half and for the column half of the pairs."""
    rows, _, d = x.shape
    ladder = ladder or d // 2
    inv_freq = theta ** (-(torch.arange(d // 2, dtype=torch.float32) % ladder) / ladder)
    stream = torch.repeat_interleave(torch.arange(3), torch.tensor(sections))
    pos = positions.float()[stream, :].t()  # [rows, d/2]
    return _rotate(x, pos * inv_freq[None, :])


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, mask: str = "none", mask_arg: int = 0,
              scale: float | None = None) -> torch.Tensor:
    """q [Sq, Hq, D], k/v [Skv, Hkv, D] -> [Sq, Hq, D].  GQA: query head h reads kv head h // (Hq / Hkv).
    mask: "none", "causal" (key j visible when j <= i + mask_arg), "block" (j // mask_arg == i // mask_arg)."""
    sq, hq, d = q.shape
    skv, hkv, _ = k.shape
    rep = hq // hkv
    kf = k.float().repeat_interleave(rep, dim=1)
    vf = v.float().repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q.float() * (scale if scale is not None else d ** -0.5), kf)
    i = torch.arange(sq)[:, None]
    j = torch.arange(skv)[None, :]
    if mask == "causal":
        scores = scores.masked_fill(~(j <= i + mask_arg), float("-inf"))
    elif mask == "block":
        scores = scores.masked_fill(~(j // mask_arg == i // mask_arg), float("-inf"))
    p = torch.softmax(scores, dim=-1)
    return bf16_round(torch.einsum("hij,jhd->ihd", p, vf))


def timestep_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """[cos(t f_i) | sin(t f_i)], f_i = exp(-ln(10000) i / (dim/2)); t is a 1-D tensor of times."""
    half = dim // 2
    freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)
    arg = t.float()[:, None] * freq[None, :]
    return bf16_round(torch.cat([arg.cos(), arg.sin()], dim=-1))


def silu(x: torch.Tensor) -> torch.Tensor:
    xf = x.float()
    return bf16_round(xf * torch.sigmoid(xf))


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    g = gate.float()
    return bf16_round(g * torch.sigmoid(g) * up.float())


# Block-level tolerance for stacks whose GEMM inputs are quantised per tensor on the fly (scale = amax / 448).
# A last-bit change of the largest activation moves the scale of the whole tensor, and with it the E4M3 code of
# several percent of its elements, so two correct implementations that differ in one bf16 rounding upstream
# differ by 3-4% of the output range after one block (measured on the oracle itself: see
# tests/test_qwen_vl_cpu.py).  Kernels fed identical inputs are held to 1e-2; BF16 blocks to 2e-2.
FP8_BLOCK_TOL = 5e-2


def ulp_noise(x: torch.Tensor, frac: float, seed: int) -> torch.Tensor:
    """Move a fraction ``frac`` of the bf16 elements of ``x`` by one unit in the last place, up or down."""
    g = torch.Generator().manual_seed(seed)
    bits = x.contiguous().view(torch.int16).clone()
    pick = (torch.rand(x.shape, generator=g) < frac).to(torch.int16)
    sign = torch.randint(0, 2, x.shape, generator=g).to(torch.int16) * 2 - 1
    return (bits + pick * sign).view(torch.bfloat16)


def max_rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    """max |got - want| / max |want|: the relative-error measure the parity tests use."""
    got, want = got.float(), want.float()
    return float((got - want).abs().max() / want.abs().max().clamp_min(1e-30))


def cosine(got: torch.Tensor, want: torch.Tensor) -> float:
    return float(torch.nn.functional.cosine_similarity(got.float().reshape(-1), want.float().reshape(-1), dim=0))

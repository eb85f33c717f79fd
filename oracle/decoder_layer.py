"""CPU oracle of one Qwen2.5-VL-style decoder layer (TEST INFRASTRUCTURE; see oracle/__init__.py).

Arithmetic of ``aginfer_b200/recipes/decoder_layer.py``, restated in fp32 from the published shape of the
architecture (pre-norm, biased Q/K/V projections, half-split rotary embedding on Q and K, grouped-query
causal attention, SwiGLU MLP); the reference project contains no implementation of it.  Tensors the GPU
recipe stores in bf16 are rounded at the same points.  FP8 layers dequantise the same E4M3 bytes and fp32
scales, and quantise each GEMM input per tensor exactly as the kernels do.
"""
from __future__ import annotations

import torch

from . import ops

L = "model.layers.0"


def _linear(cfg, w, name, x, **kw):
    weight = w[f"{L}.{name}.weight"]
    if cfg.fp8:
        xq, xs = ops.quantize_e4m3(x)
        return ops.gemm(xq, weight, scale_a=xs, scale_w=w[f"{L}.{name}.weight_scale"], **kw)
    return ops.gemm(x, weight, **kw)


def forward(cfg, w: dict, hidden: torch.Tensor) -> torch.Tensor:
    S, D = cfg.tokens, cfg.head_dim
    h = ops.rmsnorm(hidden, w[f"{L}.input_layernorm.weight"], cfg.eps)
    q = _linear(cfg, w, "self_attn.q_proj", h, bias=w[f"{L}.self_attn.q_proj.bias"]).view(S, cfg.heads, D)
    k = _linear(cfg, w, "self_attn.k_proj", h, bias=w[f"{L}.self_attn.k_proj.bias"]).view(S, cfg.kv_heads, D)
    v = _linear(cfg, w, "self_attn.v_proj", h, bias=w[f"{L}.self_attn.v_proj.bias"]).view(S, cfg.kv_heads, D)
    q, k = ops.rope(q, cfg.theta), ops.rope(k, cfg.theta)
    att = ops.attention(q, k, v, mask="causal").reshape(S, cfg.q_dim)
    x = _linear(cfg, w, "self_attn.o_proj", att, residual=hidden)
    h = ops.rmsnorm(x, w[f"{L}.post_attention_layernorm.weight"], cfg.eps)
    act = ops.swiglu(_linear(cfg, w, "mlp.gate_proj", h), _linear(cfg, w, "mlp.up_proj", h))
    return _linear(cfg, w, "mlp.down_proj", act, residual=x)

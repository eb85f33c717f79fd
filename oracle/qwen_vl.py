"""CPU oracle of the Qwen2.5-VL-shaped backbone prefill (TEST INFRASTRUCTURE; see oracle/__init__.py).

Arithmetic of ``aginfer_b200/recipes/qwen_vl.py`` restated in fp32 from the published shape of the
architecture; the reference project contains no implementation, test or golden vector of it (parity
unpinned).  Everything the shape description leaves open (token order, vision rotary layout, biases, merger,
prefix layout, padding of 3420 and 1176) is fixed in that recipe's header and followed here.  Tensors the GPU
recipe stores in bf16 are rounded at the same points; every FP8 GEMM input is quantised per tensor
(amax / 448) exactly as the kernels do, and the same E4M3 weight bytes and fp32 scales are dequantised.
"""
from __future__ import annotations

import torch

from . import ops


def window_order(cfg) -> torch.Tensor:
    """(py, px) of every token of ONE image in window order: [P*P, 2]."""
    P, W, m = cfg.grid, cfg.window, cfg.merge
    out = []
    for wy in range(P // W):
        for wx in range(P // W):
            for gy in range(W // m):
                for gx in range(W // m):
                    for sy in range(m):
                        for sx in range(m):
                            out.append((wy * W + gy * m + sy, wx * W + gx * m + sx))
    return torch.tensor(out, dtype=torch.long)


def patchify(cfg, pixels: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """pixels [images, C, S, S] fp32 -> ([tokens, patch_k] bf16 in window order, positions [3, tokens] int32)."""
    order = window_order(cfg)
    p = cfg.patch
    rows, pos = [], []
    for image in range(cfg.images):
        for py, px in order.tolist():
            tile = pixels[image, :, py * p:(py + 1) * p, px * p:(px + 1) * p]            # [C, p, p]
            vec = tile[:, None].expand(-1, cfg.temporal, -1, -1).reshape(-1)            # (c, t, iy, ix)
            rows.append(torch.nn.functional.pad(vec, (0, cfg.patch_k - vec.numel())))
            pos.append((py, px, 0))
    return ops.bf16_round(torch.stack(rows)), torch.tensor(pos, dtype=torch.int32).t().contiguous()


def unwindow(cfg, merged: torch.Tensor) -> torch.Tensor:
    """Merged tokens [images * G * G, cols] from window order to raster order."""
    G, w = cfg.grid // cfg.merge, cfg.window // cfg.merge
    out = torch.empty_like(merged)
    row = 0
    for image in range(cfg.images):
        for wy in range(G // w):
            for wx in range(G // w):
                for gy in range(w):
                    for gx in range(w):
                        out[image * G * G + (wy * w + gy) * G + wx * w + gx] = merged[row]
                        row += 1
    return out


def _fp8_linear(w: dict, name: str, xq, xs, **kw) -> torch.Tensor:
    return ops.gemm(xq, w[f"{name}.weight"], scale_a=xs, scale_w=w[f"{name}.weight_scale"], bias=w.get(f"{name}.bias"),
                    **kw)


def vision_block(cfg, w: dict, i: int, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
    """Block i of the vision tower over patch tokens x [patches, 1280] in window order."""
    P, VH, VD = cfg.patches, cfg.v_hidden, cfg.v_head_dim
    half = VD // 2
    sections = (half // 2, half - half // 2, 0)
    b = f"visual.blocks.{i}"
    xq, xs = ops.quantize_e4m3(ops.rmsnorm(x, w[f"{b}.norm1.weight"], cfg.eps))
    qkv = _fp8_linear(w, f"{b}.attn.qkv", xq, xs)
    qk = ops.mrope(qkv[:, :2 * VH].reshape(P, 2 * cfg.v_heads, VD), pos, cfg.v_theta, sections, ladder=half // 2)
    q, k = qk[:, :cfg.v_heads], qk[:, cfg.v_heads:]
    v = qkv[:, 2 * VH:].reshape(P, cfg.v_heads, VD)
    span = cfg.grid * cfg.grid if i in cfg.v_full_layers else cfg.window * cfg.window
    att = ops.attention(q, k, v, mask="block", mask_arg=span).reshape(P, VH)
    aq, as_ = ops.quantize_e4m3(att)
    x2 = _fp8_linear(w, f"{b}.attn.proj", aq, as_, residual=x)
    xq, xs = ops.quantize_e4m3(ops.rmsnorm(x2, w[f"{b}.norm2.weight"], cfg.eps))
    act = ops.swiglu(_fp8_linear(w, f"{b}.mlp.gate_proj", xq, xs), _fp8_linear(w, f"{b}.mlp.up_proj", xq, xs))
    aq, as_ = ops.quantize_e4m3(act)
    return _fp8_linear(w, f"{b}.mlp.down_proj", aq, as_, residual=x2)


def vision_block_forced(cfg, w: dict, i: int, x: torch.Tensor, pos: torch.Tensor, operands):
    """``vision_block`` with every GEMM fed the quantised operands a device run used: ``operands`` = four
    (E4M3 tensor [rows, K], fp32 scale) in the order they are produced.  Returns (block output, the oracle's own
    tensors at the four quantisation points, each computed from the forced operands upstream of it).  Two correct
    implementations then differ only by accumulation order and the bf16 rounding of the output, which is what
    the 2e-2 tier is for; the per-tensor scale jitter of free-running FP8 is taken out."""
    P, VH, VD = cfg.patches, cfg.v_hidden, cfg.v_head_dim
    half = VD // 2
    b = f"visual.blocks.{i}"
    refs = [ops.rmsnorm(x, w[f"{b}.norm1.weight"], cfg.eps)]
    qkv = _fp8_linear(w, f"{b}.attn.qkv", *operands[0])
    qk = ops.mrope(qkv[:, :2 * VH].reshape(P, 2 * cfg.v_heads, VD), pos, cfg.v_theta, (half // 2, half - half // 2, 0),
                   ladder=half // 2)
    span = cfg.grid * cfg.grid if i in cfg.v_full_layers else cfg.window * cfg.window
    refs.append(ops.attention(qk[:, :cfg.v_heads], qk[:, cfg.v_heads:], qkv[:, 2 * VH:].reshape(P, cfg.v_heads, VD),
                              mask="block", mask_arg=span).reshape(P, VH))
    x2 = _fp8_linear(w, f"{b}.attn.proj", *operands[1], residual=x)
    refs.append(ops.rmsnorm(x2, w[f"{b}.norm2.weight"], cfg.eps))
    refs.append(ops.swiglu(_fp8_linear(w, f"{b}.mlp.gate_proj", *operands[2]), _fp8_linear(w, f"{b}.mlp.up_proj", *operands[2])))
    return _fp8_linear(w, f"{b}.mlp.down_proj", *operands[3], residual=x2), refs


def merger(cfg, w: dict, x: torch.Tensor) -> torch.Tensor:
    """Patch tokens [patches, 1280] (window order) -> merged tokens [patches / 4, hidden] (window order)."""
    normed = ops.rmsnorm(x, w["visual.merger.ln_q.weight"], cfg.eps).reshape(cfg.merged, cfg.merged_dim)
    xq, xs = ops.quantize_e4m3(normed)
    mid = _fp8_linear(w, "visual.merger.mlp.0", xq, xs, act="gelu_tanh")
    xq, xs = ops.quantize_e4m3(mid)
    return _fp8_linear(w, "visual.merger.mlp.2", xq, xs)


def vision_tower(cfg, w: dict, pixels: torch.Tensor) -> torch.Tensor:
    """Merged image tokens [images * G * G, hidden] in window order."""
    patches, pos = patchify(cfg, pixels)
    x = ops.gemm(patches, w["visual.patch_embed.proj.weight"])
    for i in range(cfg.v_layers):
        x = vision_block(cfg, w, i, x, pos)
    return merger(cfg, w, x)


def decoder_layer(cfg, w: dict, i: int, h: torch.Tensor, positions: torch.Tensor, attn_hook=None):
    """Layer i of the language model: (next hidden states, rotated K [tokens, kv_dim], V [tokens, kv_dim]).
    ``attn_hook`` (tests only) maps the attention output before it is quantised, e.g. to add last-bit noise."""
    S, D = cfg.tokens, cfg.head_dim
    l = f"model.layers.{i}"
    xq, xs = ops.quantize_e4m3(ops.rmsnorm(h, w[f"{l}.input_layernorm.weight"], cfg.eps))
    q = _fp8_linear(w, f"{l}.self_attn.q_proj", xq, xs).view(S, cfg.heads, D)
    k = _fp8_linear(w, f"{l}.self_attn.k_proj", xq, xs).view(S, cfg.kv_heads, D)
    v = _fp8_linear(w, f"{l}.self_attn.v_proj", xq, xs).view(S, cfg.kv_heads, D)
    q, k = ops.mrope(q, positions, cfg.theta, cfg.sections), ops.mrope(k, positions, cfg.theta, cfg.sections)
    att = ops.attention(q, k, v, mask="causal").reshape(S, cfg.q_dim)
    if attn_hook is not None:
        att = attn_hook(att)
    aq, as_ = ops.quantize_e4m3(att)
    h2 = _fp8_linear(w, f"{l}.self_attn.o_proj", aq, as_, residual=h)
    xq, xs = ops.quantize_e4m3(ops.rmsnorm(h2, w[f"{l}.post_attention_layernorm.weight"], cfg.eps))
    act = ops.swiglu(_fp8_linear(w, f"{l}.mlp.gate_proj", xq, xs), _fp8_linear(w, f"{l}.mlp.up_proj", xq, xs))
    aq, as_ = ops.quantize_e4m3(act)
    return _fp8_linear(w, f"{l}.mlp.down_proj", aq, as_, residual=h2), k.reshape(S, cfg.kv_dim), v.reshape(S, cfg.kv_dim)


def decoder_layer_forced(cfg, w: dict, i: int, h: torch.Tensor, positions: torch.Tensor, operands):
    """``decoder_layer`` with every GEMM fed the quantised operands a device run used (see ``vision_block_forced``).
    Returns (next hidden states, the oracle's own tensors at the four quantisation points)."""
    S, D = cfg.tokens, cfg.head_dim
    l = f"model.layers.{i}"
    refs = [ops.rmsnorm(h, w[f"{l}.input_layernorm.weight"], cfg.eps)]
    q = _fp8_linear(w, f"{l}.self_attn.q_proj", *operands[0]).view(S, cfg.heads, D)
    k = _fp8_linear(w, f"{l}.self_attn.k_proj", *operands[0]).view(S, cfg.kv_heads, D)
    v = _fp8_linear(w, f"{l}.self_attn.v_proj", *operands[0]).view(S, cfg.kv_heads, D)
    q, k = ops.mrope(q, positions, cfg.theta, cfg.sections), ops.mrope(k, positions, cfg.theta, cfg.sections)
    refs.append(ops.attention(q, k, v, mask="causal").reshape(S, cfg.q_dim))
    h2 = _fp8_linear(w, f"{l}.self_attn.o_proj", *operands[1], residual=h)
    refs.append(ops.rmsnorm(h2, w[f"{l}.post_attention_layernorm.weight"], cfg.eps))
    refs.append(ops.swiglu(_fp8_linear(w, f"{l}.mlp.gate_proj", *operands[2]), _fp8_linear(w, f"{l}.mlp.up_proj", *operands[2])))
    return _fp8_linear(w, f"{l}.mlp.down_proj", *operands[3], residual=h2), refs


def language_model(cfg, w: dict, h: torch.Tensor, positions: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """Hidden states [tokens, hidden] -> (final-norm hidden states, K/V cache [layers, 2, tokens, kv_dim])."""
    cache = torch.empty(cfg.layers, 2, cfg.tokens, cfg.kv_dim, dtype=torch.bfloat16)
    for i in range(cfg.layers):
        h, cache[i, 0], cache[i, 1] = decoder_layer(cfg, w, i, h, positions)
    return ops.rmsnorm(h, w["model.norm.weight"], cfg.eps), cache


def embed_prefix(cfg, w: dict, merged_window_order: torch.Tensor, input_ids: torch.Tensor) -> torch.Tensor:
    """[image tokens in raster order | text embeddings] -> [tokens, hidden] bf16."""
    text = w["model.embed_tokens.weight"][input_ids.long()]
    return torch.cat([unwindow(cfg, merged_window_order), text], dim=0)


def forward(cfg, w: dict, pixels: torch.Tensor, input_ids: torch.Tensor, positions: torch.Tensor):
    """Returns (hidden_out [tokens, hidden] bf16, kv_cache [layers, 2, tokens, kv_dim] bf16)."""
    merged = vision_tower(cfg, w, pixels)
    return language_model(cfg, w, embed_prefix(cfg, w, merged, input_ids), positions)

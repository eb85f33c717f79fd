"""CPU oracle of the LingBot-VLA-shaped episode (TEST INFRASTRUCTURE; see oracle/__init__.py).

Arithmetic of ``aginfer_b200/recipes/lingbot.py`` restated in fp32: the FP8 backbone prefill of
``oracle/qwen_vl.py`` followed by the BF16 flow-matching action expert.  The reference project contains no
implementation, test or golden vector of it (parity unpinned); every open choice is listed in the recipe's
header and followed here.  Tensors the GPU recipe stores in bf16 are rounded at the same points.
"""
from __future__ import annotations

import torch

from . import ops
from . import qwen_vl as backbone

E = "expert"
PAD = 32


def _lin(w: dict, name: str, x: torch.Tensor, **kw) -> torch.Tensor:
    return ops.gemm(x, w[f"{name}.weight"], bias=w.get(f"{name}.bias"), **kw)


def _pad(x: torch.Tensor) -> torch.Tensor:
    return torch.nn.functional.pad(x, (0, PAD - x.shape[-1]))


def expert_layer(cfg, w: dict, j: int, seq: torch.Tensor, prefix_k: torch.Tensor, prefix_v: torch.Tensor, pos0: int):
    """Layer j over action tokens seq [horizon, 1024]; prefix_k / prefix_v [prefix, kv_dim] are the backbone's."""
    T, D = cfg.horizon, cfg.head_dim
    l = f"{E}.layers.{j}"
    bb = cfg.backbone
    hn = ops.rmsnorm(seq, w[f"{l}.input_layernorm.weight"], bb.eps)
    q = ops.rope(_lin(w, f"{l}.self_attn.q_proj", hn).view(T, cfg.e_heads, D), bb.theta, pos0)
    k = ops.rope(_lin(w, f"{l}.self_attn.k_proj", hn).view(T, cfg.e_kv_heads, D), bb.theta, pos0)
    v = _lin(w, f"{l}.self_attn.v_proj", hn).view(T, cfg.e_kv_heads, D)
    keys = torch.cat([prefix_k.view(-1, cfg.e_kv_heads, D), k], dim=0)
    values = torch.cat([prefix_v.view(-1, cfg.e_kv_heads, D), v], dim=0)
    att = ops.attention(q, keys, values).reshape(T, cfg.e_hidden)
    seq2 = _lin(w, f"{l}.self_attn.o_proj", att, residual=seq)
    hn = ops.rmsnorm(seq2, w[f"{l}.post_attention_layernorm.weight"], bb.eps)
    act = ops.swiglu(_lin(w, f"{l}.mlp.gate_proj", hn), _lin(w, f"{l}.mlp.up_proj", hn))
    return _lin(w, f"{l}.mlp.down_proj", act, residual=seq2)


def action_expert(cfg, w: dict, cache: torch.Tensor, state: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """cache [layers, 2, prefix, kv_dim] (bf16, as the prefill exports it) -> actions [horizon, action_dim] fp32."""
    S, T = cfg.steps, cfg.horizon
    times = torch.arange(S, dtype=torch.float32) / S
    t_hid = _lin(w, f"{E}.time_mlp.0", ops.timestep_embedding(times, cfg.time_dim), act="silu")
    cond = _lin(w, f"{E}.time_mlp.2", t_hid)
    s_emb = _lin(w, f"{E}.state_in", _pad(state))
    cond = ops.bf16_round(cond.float() + s_emb.float())
    pos0 = cfg.first_action_position()
    x_bf = _pad(noise)
    x = x_bf.float().clone()
    for step in range(S):
        seq = _lin(w, f"{E}.action_in", x_bf)
        seq = ops.bf16_round(seq.float() + cond[step].float())
        for j in range(cfg.e_layers):
            src = cfg.backbone_layer_of(j)
            seq = expert_layer(cfg, w, j, seq, cache[src, 0], cache[src, 1], pos0)
        vel = _lin(w, f"{E}.action_out", ops.rmsnorm(seq, w[f"{E}.norm.weight"], cfg.backbone.eps))
        x = x + vel.float() / S
        x_bf = ops.bf16_round(x)
    return x[:, :cfg.action_dim].contiguous()


def forward(cfg, w: dict, pixels, input_ids, positions, state, noise):
    """Returns (actions [horizon, action_dim] fp32, hidden_out, kv_cache)."""
    hidden, cache = backbone.forward(cfg.backbone, w, pixels, input_ids, positions)
    return action_expert(cfg, w, cache, state, noise), hidden, cache

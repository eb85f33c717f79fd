"""CPU oracle of the flow-matching DiT action head (TEST INFRASTRUCTURE; see oracle/__init__.py).

Defines the arithmetic of ``aginfer_b200/recipes/dit.py``.  The reference (wenhuiNi/AgInfer)
has no implementation of this model; the structure below follows the public description of
NVIDIA's GR00T-N1.5 action head, restated from its shape, with these choices made here:

* state encoder and action decoder are two-layer MLPs with ReLU; the action encoder is
  ``W3(silu(W2([W1 a | sinusoid(t)])))`` with a learned position embedding added to the 16
  action tokens; the state token is prepended (17 tokens);
* flow time t = i / steps is discretised to ``floor(t * 1000)`` before either sinusoid;
* every block: ``h = LN(x) * (1 + scale) + shift`` with ``(scale | shift) = Linear(silu(temb))``;
  attention (even blocks: queries from h, keys/values from the backbone tokens; odd blocks:
  self attention), ``x += to_out(attn)``; ``x += fc2(gelu_tanh(fc1(LN(x))))``; LayerNorms have no
  affine parameters, eps 1e-5; all Linear layers have biases;
* output: ``LN(x)`` modulated by ``norm_out``, ``proj_out`` to 1024, action decoder on the 16
  action tokens gives the velocity; Euler update ``x += v / steps`` on an fp32 latent.

Arithmetic is fp32 on the bf16 weights; every tensor the GPU recipe stores in bf16 is
rounded to bf16 at the same point (the per-op oracles in ``ops.py`` do that rounding).
"""
from __future__ import annotations

import torch

from . import ops

P = "action_head"


def _lin(w, name, x, **kw):
    return ops.gemm(x, w[f"{name}.weight"], bias=w[f"{name}.bias"], **kw)


def forward(cfg, w: dict, backbone: torch.Tensor, state: torch.Tensor, noise: torch.Tensor) -> torch.Tensor:
    """Returns the action chunk [horizon, action_dim] in fp32."""
    D, T, H, S = cfg.hidden, cfg.tokens, cfg.horizon, cfg.steps
    heads, hd = cfg.heads, cfg.head_dim
    times = torch.tensor(cfg.step_times())

    # once per chunk
    state_tok = _lin(w, f"{P}.state_encoder.fc2", _lin(w, f"{P}.state_encoder.fc1", state, act="relu"))
    kv = {}
    for l in range(cfg.layers):
        if cfg.is_cross(l):
            b = f"{P}.dit.blocks.{l}.attn"
            kv[l] = (_lin(w, f"{b}.to_k", backbone), _lin(w, f"{b}.to_v", backbone))
    t_hid = _lin(w, f"{P}.dit.timestep_embedder.linear_1", ops.timestep_embedding(times, cfg.time_dim), act="silu")
    temb_act = ops.silu(_lin(w, f"{P}.dit.timestep_embedder.linear_2", t_hid))
    mods = [_lin(w, f"{P}.dit.blocks.{l}.norm1.linear", temb_act) for l in range(cfg.layers)]
    mods.append(_lin(w, f"{P}.dit.norm_out.linear", temb_act))

    x = noise.float().clone()
    x_bf = noise.clone()
    for step in range(S):
        a = _lin(w, f"{P}.action_encoder.W1", x_bf)
        tau = ops.timestep_embedding(times[step].repeat(H), D)
        enc = _lin(w, f"{P}.action_encoder.W3", _lin(w, f"{P}.action_encoder.W2", torch.cat([a, tau], dim=-1), act="silu"))
        enc = ops.bf16_round(enc.float() + w[f"{P}.position_embedding.weight"].float())
        seq = torch.cat([state_tok, enc], dim=0)
        for l in range(cfg.layers):
            b = f"{P}.dit.blocks.{l}"
            scale, shift = mods[l][step, :D], mods[l][step, D:]
            h = ops.layernorm(seq, cfg.ln_eps, scale, shift)
            q = _lin(w, f"{b}.attn.to_q", h)
            if cfg.is_cross(l):
                k, v = kv[l]
            else:
                k, v = _lin(w, f"{b}.attn.to_k", h), _lin(w, f"{b}.attn.to_v", h)
            att = ops.attention(q.view(T, heads, hd), k.view(-1, heads, hd), v.view(-1, heads, hd)).reshape(T, D)
            seq = _lin(w, f"{b}.attn.to_out", att, residual=seq)
            h = ops.layernorm(seq, cfg.ln_eps)
            seq = _lin(w, f"{b}.ff.fc2", _lin(w, f"{b}.ff.fc1", h, act="gelu_tanh"), residual=seq)
        scale, shift = mods[cfg.layers][step, :D], mods[cfg.layers][step, D:]
        h = ops.layernorm(seq, cfg.ln_eps, scale, shift)
        out = _lin(w, f"{P}.dit.proj_out", h)
        vel = _lin(w, f"{P}.action_decoder.fc2", _lin(w, f"{P}.action_decoder.fc1", out[1:], act="relu"))
        x = x + vel.float() / S
        x_bf = ops.bf16_round(x)
    return x

"""Launch recipe of a LingBot-VLA-shaped episode: FP8 vision-language prefill + BF16 flow-matching action expert.

Backbone: the Qwen2.5-VL-7B-shaped prefill of ``qwen_vl.py`` (28 layers x 3584, 28 query / 4 KV heads of 128,
SwiGLU 18944, 3 images -> 192 merged tokens + 64 text tokens = 256).  Action expert: 18 layers x 1024, 8 query /
4 KV heads of 128, SwiGLU 4096, 50 action tokens x 14 dims, 10 Euler steps of the learned velocity field, all in
ONE graph-safe profile (steps unrolled, the step time baked into the launches).

What the shape description leaves open is fixed here and mirrored by ``oracle/lingbot.py``:
  * expert layer j attends over [K/V of backbone layer (j * layers) // e_layers | its own 50 action tokens]
    (306 keys, no mask inside: every action token sees the whole prefix and every action token);
  * rotary embedding on the expert's Q and K: 1-D, same theta as the backbone, action token i at position
    (largest prefix position + 1 + i); the prefix keys keep the M-RoPE rotation the backbone gave them;
  * action tokens enter as  action_in(x_t) + [time_mlp(sinusoidal(t)) + state_in(state)]  (the bracket depends
    on the step only, so all steps' conditioning vectors are computed once before the loop); there is no
    separate state token; t runs from 0 to 1 - 1/steps and x <- x + v / steps;
  * expert linears carry no bias except the input / output / conditioning projections; RMSNorm gains 1;
  * the 14-wide action and state vectors are held padded to 32 columns (zero weights and bias there), which
    keeps every GEMM's K a whole number of 64-byte windows.
Outputs: ``actions`` [50, 14] fp32, plus the prefill's outputs.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from . import qwen_vl
from .builder import F32, RecipeBuilder, Tensor, U32, Weight, grid_for, io

BACKBONE_7B = qwen_vl.VlConfig(images=3, hidden=3584, heads=28, kv_heads=4, intermediate=18944, layers=28,
                               text_tokens=64)
PAD = 32      # columns the 14-wide action / state vectors are padded to
E = "expert"


@dataclass(frozen=True)
class EpisodeConfig:
    backbone: qwen_vl.VlConfig = BACKBONE_7B
    e_layers: int = 18
    e_hidden: int = 1024
    e_heads: int = 8
    e_kv_heads: int = 4
    e_mlp: int = 4096
    horizon: int = 50
    action_dim: int = 14
    state_dim: int = 14
    time_dim: int = 256
    steps: int = 10

    @property
    def head_dim(self) -> int:
        return self.backbone.head_dim

    @property
    def e_kv_dim(self) -> int:
        return self.e_kv_heads * self.head_dim

    def backbone_layer_of(self, j: int) -> int:
        return (j * self.backbone.layers) // self.e_layers

    def first_action_position(self) -> int:
        return int(qwen_vl.rope_positions(self.backbone).max()) + 1


def expert_shapes(cfg: EpisodeConfig) -> dict[str, tuple[int, ...]]:
    H, I, KV = cfg.e_hidden, cfg.e_mlp, cfg.e_kv_dim
    assert KV == cfg.backbone.kv_dim, "the expert shares the backbone's K/V width"
    s = {f"{E}.action_in.weight": (H, PAD), f"{E}.action_in.bias": (H,), f"{E}.state_in.weight": (H, PAD),
         f"{E}.state_in.bias": (H,), f"{E}.time_mlp.0.weight": (H, cfg.time_dim), f"{E}.time_mlp.0.bias": (H,),
         f"{E}.time_mlp.2.weight": (H, H), f"{E}.time_mlp.2.bias": (H,), f"{E}.norm.weight": (H,),
         f"{E}.action_out.weight": (PAD, H), f"{E}.action_out.bias": (PAD,)}
    for j in range(cfg.e_layers):
        l = f"{E}.layers.{j}"
        s.update({f"{l}.input_layernorm.weight": (H,), f"{l}.post_attention_layernorm.weight": (H,),
                  f"{l}.self_attn.q_proj.weight": (H, H), f"{l}.self_attn.k_proj.weight": (KV, H),
                  f"{l}.self_attn.v_proj.weight": (KV, H), f"{l}.self_attn.o_proj.weight": (H, H),
                  f"{l}.mlp.gate_proj.weight": (I, H), f"{l}.mlp.up_proj.weight": (I, H), f"{l}.mlp.down_proj.weight": (H, I)})
    return s


def synthetic_weights(cfg: EpisodeConfig, seed: int = 4, std: float = 0.02) -> dict:
    """Backbone checkpoint (FP8 linears, ``qwen_vl.synthetic_weights``) plus BF16 expert weights ~ N(0, std)."""
    import torch
    out = qwen_vl.synthetic_weights(cfg.backbone, seed=seed, std=std)
    g = torch.Generator().manual_seed(seed + 77)
    for name, shape in expert_shapes(cfg).items():
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            t = torch.ones(shape)
        else:
            t = torch.randn(shape, generator=g) * std
        if name.startswith((f"{E}.action_in.weight", f"{E}.state_in.weight")):
            t[:, cfg.action_dim:] = 0          # padding columns of the 14-wide inputs
        if name.startswith(f"{E}.action_out"):
            t[cfg.action_dim:] = 0             # padding rows of the 14-wide output (weight and bias)
        out[name] = t.to(torch.bfloat16)
    return out


def synthetic_inputs(cfg: EpisodeConfig, seed: int = 4) -> dict:
    import torch
    x = qwen_vl.synthetic_inputs(cfg.backbone, seed=seed)
    g = torch.Generator().manual_seed(seed + 2000)
    x["state"] = torch.randn(1, cfg.state_dim, generator=g).to(torch.bfloat16)
    x["noise"] = torch.randn(cfg.horizon, cfg.action_dim, generator=g).to(torch.bfloat16)
    return x


def build_recipe(cfg: EpisodeConfig, weights, packed: bool = False, trace: bool = False) -> RecipeBuilder:
    """``weights``: name -> (dtype, shape) as from ``package.describe``."""
    bb = cfg.backbone
    BF, H, I, KV, D, T, S = 2, cfg.e_hidden, cfg.e_mlp, cfg.e_kv_dim, cfg.head_dim, cfg.horizon, cfg.steps
    prefix = bb.tokens
    keys = prefix + T

    def expert(r: RecipeBuilder, cache, _hidden) -> None:
        def elementwise(kernel, args, work, op):
            r.launch(kernel, (grid_for(work), 1, 1), (256, 1, 1), args, op=op)

        def lin(x, name, y, M, N, K, **kw):
            bias = Weight(f"{name}.bias") if f"{name}.bias" in weights else None
            r.gemm(x, Weight(f"{name}.weight"), y, M, N, K, bias=bias, **kw)

        def group(x, parts, M, K):
            """Projections that share their input as one launch: ``parts`` = (name, y, N, ldy)."""
            biased = {f"{name}.bias" in weights for name, *_ in parts}
            if len(biased) != 1 or K % 64:          # mixed bias / odd K: one launch each
                for name, y, N, ldy in parts:
                    lin(x, name, y, M, N, K, ldy=ldy)
                return
            r.gemm_group(x, [(Weight(f"{name}.weight"), Weight(f"{name}.bias") if True in biased else None, None, y, N, ldy)
                             for name, y, N, ldy in parts], M, K)

        # ---- once per episode: conditioning vectors of every step, latent, K/V of the prefix ----
        t_sin, t_hid, cond, s_pad, s_emb = (r.alloc(S * cfg.time_dim * BF), r.alloc(S * H * BF), r.alloc(S * H * BF),
                                            r.alloc(PAD * BF), r.alloc(H * BF))
        x_f32, x_bf, vel = r.alloc(T * PAD * 4), r.alloc(T * PAD * BF), r.alloc(T * PAD * BF)
        kcat, vcat = r.alloc(cfg.e_layers * keys * KV * BF), r.alloc(cfg.e_layers * keys * KV * BF)
        elementwise("agi_timestep_embedding", [t_sin, U32(S), U32(cfg.time_dim), U32(cfg.time_dim), F32(0.0), F32(1.0 / S)],
                    S * cfg.time_dim // 2, "timestep_embedding")
        lin(t_sin, f"{E}.time_mlp.0", t_hid, S, H, cfg.time_dim, act="silu")
        lin(t_hid, f"{E}.time_mlp.2", cond, S, H, H)
        elementwise("agi_fill_u32", [s_pad, U32(0), U32(PAD * BF // 4)], PAD, "zero")
        elementwise("agi_copy_rows_bf16", [Tensor("state"), s_pad, U32(1), U32(cfg.state_dim), U32(cfg.state_dim), U32(PAD)],
                    cfg.state_dim, "copy")
        lin(s_pad, f"{E}.state_in", s_emb, 1, H, PAD)
        elementwise("agi_add_rows_bf16", [cond, s_emb, U32(S), U32(H), U32(H), U32(1)], S * H, "add_rows")
        elementwise("agi_fill_u32", [x_bf, U32(0), U32(T * PAD * BF // 4)], T * PAD, "zero")
        elementwise("agi_copy_rows_bf16", [Tensor("noise"), x_bf, U32(T), U32(cfg.action_dim), U32(cfg.action_dim), U32(PAD)],
                    T * cfg.action_dim, "copy")
        elementwise("agi_bf16_to_f32", [x_bf, x_f32, U32(T * PAD)], T * PAD, "cast")
        for j in range(cfg.e_layers):
            src = cfg.backbone_layer_of(j)
            for which, cat in ((0, kcat), (1, vcat)):
                elementwise("agi_copy_u32", [cache + (2 * src + which) * prefix * KV * BF, cat + j * keys * KV * BF,
                                             U32(prefix * KV * BF // 4)], prefix * KV // 2, "prefix_kv")

        # ---- per step ----
        seq, seq2, hn = r.alloc(T * H * BF), r.alloc(T * H * BF), r.alloc(T * H * BF)
        q_buf, att, gu, act = r.alloc(T * H * BF), r.alloc(T * H * BF), r.alloc(T * 2 * I * BF), r.alloc(T * I * BF)
        pos0 = cfg.first_action_position()
        for step in range(S):
            lin(x_bf, f"{E}.action_in", seq, T, H, PAD)
            elementwise("agi_add_rows_bf16", [seq, cond + step * H * BF, U32(T), U32(H), U32(H), U32(1)], T * H, "add_rows")
            for j in range(cfg.e_layers):
                l = f"{E}.layers.{j}"
                k_rows = kcat + (j * keys + prefix) * KV * BF
                v_rows = vcat + (j * keys + prefix) * KV * BF
                r.rmsnorm(seq, Weight(f"{l}.input_layernorm.weight"), hn, T, H, bb.eps)
                group(hn, [(f"{l}.self_attn.q_proj", q_buf, H, H), (f"{l}.self_attn.k_proj", k_rows, KV, KV),
                           (f"{l}.self_attn.v_proj", v_rows, KV, KV)], T, H)
                r.rope_pair(q_buf, cfg.e_heads, H, k_rows, cfg.e_kv_heads, KV, T, D, bb.theta, pos_offset=pos0)
                r.attention(q_buf, kcat + j * keys * KV * BF, vcat + j * keys * KV * BF, att, q_rows=T, kv_rows=keys,
                            q_heads=cfg.e_heads, kv_heads=cfg.e_kv_heads, head_dim=D, q_stride=H, k_stride=KV,
                            v_stride=KV, o_stride=H, mask="none",
                            # the prefix rows were copied in once per episode, before this step's conditioning add (a
                            # launch that releases its successors only after its own wait); the tail is this layer's
                            kv_static=True, kv_static_rows=prefix)
                lin(att, f"{l}.self_attn.o_proj", seq2, T, H, H, residual=seq)
                r.rmsnorm(seq2, Weight(f"{l}.post_attention_layernorm.weight"), hn, T, H, bb.eps)
                group(hn, [(f"{l}.mlp.gate_proj", gu, I, 2 * I), (f"{l}.mlp.up_proj", gu + I * BF, I, 2 * I)], T, H)
                r.swiglu(gu, gu + I * BF, act, T, I, 2 * I)
                lin(act, f"{l}.mlp.down_proj", seq, T, H, I, residual=seq2)
            r.rmsnorm(seq, Weight(f"{E}.norm.weight"), hn, T, H, bb.eps)
            lin(hn, f"{E}.action_out", vel, T, PAD, H)
            elementwise("agi_euler_step", [x_f32, vel, x_bf, F32(1.0 / S), U32(T * PAD)], T * PAD, "euler_step")
        elementwise("agi_copy_rows_u32", [x_f32, Tensor("actions"), U32(T), U32(cfg.action_dim), U32(PAD), U32(cfg.action_dim)],
                    T * cfg.action_dim, "export_actions")

    return qwen_vl.build_recipe(bb, weights, packed=packed, trace=trace,
                                extra_inputs=[io("state", "BF16", [1, cfg.state_dim]),
                                              io("noise", "BF16", [cfg.horizon, cfg.action_dim])],
                                extra_outputs=[io("actions", "F32", [cfg.horizon, cfg.action_dim])], tail=expert)


def algorithmic(cfg: EpisodeConfig) -> dict[str, int]:
    bb = qwen_vl.algorithmic(cfg.backbone)
    per_layer = 2 * cfg.e_hidden ** 2 + 2 * cfg.e_kv_dim * cfg.e_hidden + 3 * cfg.e_mlp * cfg.e_hidden
    expert = cfg.e_layers * per_layer
    return {"backbone_fp8_weight_bytes": bb["fp8_weight_bytes"], "backbone_flops": bb["flops"], "expert_params": expert,
            "expert_weight_bytes_per_episode": 2 * expert * cfg.steps,
            "expert_flops": 2 * cfg.horizon * expert * cfg.steps}

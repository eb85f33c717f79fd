"""Launch recipe of a GR00T-N1.5-shaped flow-matching action head (DiT) at batch 1.

Shape (``DitConfig`` defaults): 16 blocks, hidden 1536, 32 heads x 48, GELU MLP 6144, AdaLN
conditioning on the flow time; blocks alternate cross-attention to the 300 backbone tokens
(dim 2048; even blocks) and self-attention over 1 state token + 16 action tokens (odd
blocks); action dim 32, state dim 64; 4 Euler steps from caller-provided noise.

The whole denoising loop is ONE profile: the steps are unrolled into the launch list with
the time of each step baked in as a scalar, so the loader replays one CUDA graph per action
chunk.  Work that does not depend on the evolving action latent is hoisted in front of the
loop and done once per chunk:
  * the state token (state encoder MLP);
  * K and V of the backbone tokens for the eight cross-attention blocks;
  * the time embedding and every block's AdaLN (scale, shift) for all steps at once
    (one skinny GEMM with M = steps per block instead of ``steps`` GEMVs).
What remains per step streams each block's Q/K/V/O and MLP weights exactly once.

Tensor names follow Hugging Face conventions (``<module>.weight`` / ``.bias``, weights
``[out, in]``) so the packed blob is ordered by the reference's name sort.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Mapping, Sequence

from .builder import Arena, F32, RecipeBuilder, Tensor, U32, Weight, dit_block_geometry, io, grid_for


@dataclass(frozen=True)
class DitConfig:
    layers: int = 16
    hidden: int = 1536
    heads: int = 32
    head_dim: int = 48
    mlp: int = 6144
    action_dim: int = 32
    state_dim: int = 64
    horizon: int = 16
    backbone_tokens: int = 300
    backbone_dim: int = 2048
    steps: int = 4
    encoder_hidden: int = 1024     # width of the state-encoder / action-decoder MLPs
    out_dim: int = 1024            # DiT output width in front of the action decoder
    time_dim: int = 256            # sinusoidal width of the flow-time embedding
    time_buckets: int = 1000       # flow time t in [0, 1) is discretised to floor(t * buckets)
    ln_eps: float = 1e-5

    @property
    def tokens(self) -> int:
        return 1 + self.horizon

    def is_cross(self, layer: int) -> bool:
        return layer % 2 == 0

    def step_times(self) -> list[float]:
        """Discretised flow time fed to the embeddings at each Euler step (t = i / steps)."""
        return [float(int(i / self.steps * self.time_buckets)) for i in range(self.steps)]


P = "action_head"


def weight_shapes(cfg: DitConfig) -> dict[str, tuple[int, ...]]:
    """Every checkpoint tensor of the action head: name -> shape (all BF16)."""
    D, s = cfg.hidden, {}

    def linear(name: str, out: int, inp: int) -> None:
        s[f"{name}.weight"] = (out, inp)
        s[f"{name}.bias"] = (out,)

    linear(f"{P}.state_encoder.fc1", cfg.encoder_hidden, cfg.state_dim)
    linear(f"{P}.state_encoder.fc2", D, cfg.encoder_hidden)
    linear(f"{P}.action_encoder.W1", D, cfg.action_dim)
    linear(f"{P}.action_encoder.W2", D, 2 * D)
    linear(f"{P}.action_encoder.W3", D, D)
    s[f"{P}.position_embedding.weight"] = (cfg.horizon, D)
    linear(f"{P}.dit.timestep_embedder.linear_1", D, cfg.time_dim)
    linear(f"{P}.dit.timestep_embedder.linear_2", D, D)
    for l in range(cfg.layers):
        b = f"{P}.dit.blocks.{l}"
        kv_in = cfg.backbone_dim if cfg.is_cross(l) else D
        linear(f"{b}.norm1.linear", 2 * D, D)
        linear(f"{b}.attn.to_q", D, D)
        linear(f"{b}.attn.to_k", D, kv_in)
        linear(f"{b}.attn.to_v", D, kv_in)
        linear(f"{b}.attn.to_out", D, D)
        linear(f"{b}.ff.fc1", cfg.mlp, D)
        linear(f"{b}.ff.fc2", D, cfg.mlp)
    linear(f"{P}.dit.norm_out.linear", 2 * D, D)
    linear(f"{P}.dit.proj_out", cfg.out_dim, D)
    linear(f"{P}.action_decoder.fc1", cfg.encoder_hidden, cfg.out_dim)
    linear(f"{P}.action_decoder.fc2", cfg.action_dim, cfg.encoder_hidden)
    return s


def synthetic_weights(cfg: DitConfig, seed: int = 2, std: float = 0.02) -> dict:
    """Random-init BF16 weights ~ N(0, std), one generator stream in name-sorted order."""
    import torch
    g = torch.Generator().manual_seed(seed)
    return {name: (torch.randn(shape, generator=g) * std).to(torch.bfloat16)
            for name, shape in sorted(weight_shapes(cfg).items())}


def packed_names(cfg: DitConfig) -> list[str]:
    """The block matrices that are multiplied with the 17-token sequence once per denoising step: queries (and keys,
    values of the self-attention blocks), attention output, MLP up and down.  The cross-attention key / value
    projections run once per chunk over the context tokens and stay row-major."""
    names = []
    for l in range(cfg.layers):
        b = f"{P}.dit.blocks.{l}"
        names += [f"{b}.attn.to_q.weight", f"{b}.attn.to_out.weight", f"{b}.ff.fc1.weight", f"{b}.ff.fc2.weight"]
        if not cfg.is_cross(l):
            names += [f"{b}.attn.to_k.weight", f"{b}.attn.to_v.weight"]
    return names


def pack_checkpoint(cfg: DitConfig, weights: dict) -> dict:
    """Packaging-time layout pass: the matrices of ``packed_names`` are replaced (same name) by their packed form
    [K / 64, N, 64] for the weight-streaming tensor-core GEMM (see ``layout.py``).  Values are untouched, so the
    oracle keeps using the row-major checkpoint.  Needs hidden and MLP widths in whole 128-row tiles."""
    from .layout import pack_kblock_swizzled
    chosen = set(packed_names(cfg))
    return {k: pack_kblock_swizzled(v) if k in chosen and v.dim() == 2 and v.shape[0] % 128 == 0 and v.shape[1] % 64 == 0
            else v for k, v in weights.items()}


def synthetic_inputs(cfg: DitConfig, seed: int = 2) -> dict:
    """Backbone tokens, state and initial noise ~ N(0, 1), BF16 (noise is an explicit input: the
    loader ignores RunOptions.seed just as the reference does)."""
    import torch
    g = torch.Generator().manual_seed(seed + 1000)
    return {"backbone_features": torch.randn(cfg.backbone_tokens, cfg.backbone_dim, generator=g).to(torch.bfloat16),
            "state": torch.randn(1, cfg.state_dim, generator=g).to(torch.bfloat16),
            "noise": torch.randn(cfg.horizon, cfg.action_dim, generator=g).to(torch.bfloat16)}


def build_recipe(cfg: DitConfig = DitConfig(), weights: Mapping[str, tuple[str, tuple[int, ...]]] | None = None,
                 gemm_tactic: str = "auto", profile: str = "default", stream_profile: bool = False,
                 fuse: bool = True, batch_kv: bool = True, block_kernel: bool | None = None,
                 step_profiles: Sequence[int] = ()) -> RecipeBuilder:
    """``block_kernel``: run each denoising step's blocks as one launch of the persistent block kernel
    (78 launches per chunk instead of 506).  Off by default: measured on B200 it is the slower of the two
    (3.9 ms per chunk against 2.9 ms), see the kernel's header for where its time goes.
    ``step_profiles``: further numbers of Euler steps to package as sibling profiles ``<profile>/steps=<n>``
    (same tensors; the loader runs one of them when the caller's RunOptions ask for n denoising steps).
    ``stream_profile``: also emit the measurement profiles of the dominant kernel."""
    D, T = cfg.hidden, cfg.tokens
    fits = dit_block_geometry(T, D, cfg.heads, cfg.head_dim, cfg.mlp, cfg.backbone_tokens, cfg.layers) is not None
    if block_kernel is None:
        block_kernel = False
    if block_kernel and not fits:
        raise ValueError("this shape is outside what the persistent block kernel covers")
    r = RecipeBuilder(weights or {k: ("BF16", v) for k, v in weight_shapes(cfg).items()})
    if block_kernel and any(r.is_packed(Weight(n)) for n in packed_names(cfg)):
        raise ValueError("the persistent block kernel reads row-major weights; package the checkpoint unpacked")
    if block_kernel:
        r.dit_scratch(T, D, cfg.mlp)      # outlives every profile: allocated before the first mark
    variants = [(profile, cfg.steps)] + [(f"{profile}/steps={n}", n) for n in step_profiles]
    for i, (name, steps) in enumerate(variants):
        mark = r.mark()                   # profiles never run concurrently: they share the arena above the mark
        _emit_chunk(r, replace(cfg, steps=steps), name, gemm_tactic, fuse, batch_kv, block_kernel,
                    measure=stream_profile and i == 0)
        r.release(mark)
    return r


def head_inputs(cfg: DitConfig) -> list[dict]:
    """The profile inputs the action head reads besides the context tokens."""
    return [io("state", "BF16", [1, cfg.state_dim]), io("noise", "BF16", [cfg.horizon, cfg.action_dim])]


def emit_action_head(r: RecipeBuilder, cfg: DitConfig, context, *, gemm_tactic: str = "auto", fuse: bool = True,
                     batch_kv: bool = True, block_kernel: bool = False) -> None:
    """Append the whole action chunk to the profile being built: ``context`` ([backbone_tokens, backbone_dim] bf16,
    any pointer: a profile input, or what an earlier part of the same profile wrote) conditions the head, which
    reads the profile tensors ``state`` and ``noise`` and writes ``actions``."""
    _emit_chunk(r, cfg, None, gemm_tactic, fuse, batch_kv, block_kernel, measure=False, context=context)


def _emit_chunk(r: RecipeBuilder, cfg: DitConfig, profile: str | None, gemm_tactic: str, fuse: bool, batch_kv: bool,
                block_kernel: bool, measure: bool, context=None) -> None:
    """One profile: the whole action chunk of ``cfg.steps`` Euler steps (``profile`` None: appended to the
    profile that is already open, without a status export of its own)."""
    D, T, H, S = cfg.hidden, cfg.tokens, cfg.horizon, cfg.steps
    if profile is not None:
        r.begin_profile(profile, [io("backbone_features", "BF16", [cfg.backbone_tokens, cfg.backbone_dim]),
                                  *head_inputs(cfg)],
                        [io("actions", "F32", [H, cfg.action_dim]), io("status", "I32", [1])])
    context = context if context is not None else Tensor("backbone_features")
    BF = 2

    def lin(x, name, y, M, N, K, **kw):
        r.gemm(x, Weight(f"{name}.weight"), y, M, N, K, bias=Weight(f"{name}.bias"), tactic=gemm_tactic, **kw)

    def elementwise(kernel, args, count, op):
        r.launch(kernel, (grid_for(count), 1, 1), (256, 1, 1), args, op=op)

    # ---- persistent buffers ----------------------------------------------------------------
    x_f32 = r.alloc(H * cfg.action_dim * 4)          # action latent, fp32 across the Euler steps
    x_bf = r.alloc(H * cfg.action_dim * BF)          # its bf16 copy, input of the action encoder
    seq = r.alloc(T * D * BF)                        # residual stream [state token; action tokens]
    state_tok = r.alloc(D * BF)
    mods = [r.alloc(S * 2 * D * BF) for _ in range(cfg.layers + 1)]   # AdaLN (scale | shift) per step
    cross = [l for l in range(cfg.layers) if cfg.is_cross(l)]
    kv_bytes = cfg.backbone_tokens * D * BF
    kv_all = r.alloc(2 * len(cross) * kv_bytes)      # K then V of every cross-attention block, back to back
    kv = {l: (kv_all + 2 * i * kv_bytes, kv_all + (2 * i + 1) * kv_bytes) for i, l in enumerate(cross)}

    # ---- once per chunk --------------------------------------------------------------------
    mark = r.mark()
    h_state = r.alloc(cfg.encoder_hidden * BF)
    lin(Tensor("state"), f"{P}.state_encoder.fc1", h_state, 1, cfg.encoder_hidden, cfg.state_dim, act="relu")
    lin(h_state, f"{P}.state_encoder.fc2", state_tok, 1, D, cfg.encoder_hidden)
    if batch_kv and (cfg.backbone_dim * BF) % 128 == 0:
        # every block's K and V projection of the context tokens, 16 at a time, as one tensor-core launch
        jobs = [(Weight(f"{P}.dit.blocks.{l}.attn.{n}.weight"), Weight(f"{P}.dit.blocks.{l}.attn.{n}.bias"))
                for l in cross for n in ("to_k", "to_v")]
        for i in range(0, len(jobs), 16):
            r.gemm_batch(context, jobs[i:i + 16], kv_all + i * kv_bytes, cfg.backbone_tokens, D,
                         cfg.backbone_dim, seg_stride=cfg.backbone_tokens * D)
    else:
        for l, (k_buf, v_buf) in kv.items():
            b = f"{P}.dit.blocks.{l}.attn"
            lin(context, f"{b}.to_k", k_buf, cfg.backbone_tokens, D, cfg.backbone_dim)
            lin(context, f"{b}.to_v", v_buf, cfg.backbone_tokens, D, cfg.backbone_dim)
    t_sin, t_hid, temb, temb_act = (r.alloc(S * cfg.time_dim * BF), r.alloc(S * D * BF), r.alloc(S * D * BF),
                                    r.alloc(S * D * BF))
    times = cfg.step_times()
    dt_bucket = times[1] - times[0] if S > 1 else 0.0
    elementwise("agi_timestep_embedding", [t_sin, U32(S), U32(cfg.time_dim), U32(cfg.time_dim), F32(times[0]),
                                           F32(dt_bucket)], S * cfg.time_dim // 2, "timestep_embedding")
    lin(t_sin, f"{P}.dit.timestep_embedder.linear_1", t_hid, S, D, cfg.time_dim, act="silu")
    lin(t_hid, f"{P}.dit.timestep_embedder.linear_2", temb, S, D, D)
    elementwise("agi_silu_bf16", [temb, temb_act, U32(S * D)], S * D, "silu")
    mod_jobs = [(Weight(f"{P}.dit.blocks.{l}.norm1.linear.weight"), Weight(f"{P}.dit.blocks.{l}.norm1.linear.bias"))
                for l in range(cfg.layers)]
    if batch_kv and (D * BF) % 128 == 0:
        # the blocks' AdaLN projections share their input: 16 at a time as one tensor-core launch
        # (mods[l] are equal-sized consecutive buffers, so block l's output starts l * S * 2D elements in)
        for i in range(0, len(mod_jobs), 16):
            r.gemm_batch(temb_act, mod_jobs[i:i + 16], mods[i], S, 2 * D, D, seg_stride=S * 2 * D)
    else:
        for l in range(cfg.layers):
            lin(temb_act, f"{P}.dit.blocks.{l}.norm1.linear", mods[l], S, 2 * D, D)
    lin(temb_act, f"{P}.dit.norm_out.linear", mods[cfg.layers], S, 2 * D, D)
    elementwise("agi_bf16_to_f32", [Tensor("noise"), x_f32, U32(H * cfg.action_dim)], H * cfg.action_dim, "cast")
    elementwise("agi_copy_rows_bf16", [Tensor("noise"), x_bf, U32(H), U32(cfg.action_dim), U32(cfg.action_dim),
                                       U32(cfg.action_dim)], H * cfg.action_dim, "copy")
    r.release(mark)

    # ---- per-step scratch ------------------------------------------------------------------
    enc_cat = r.alloc(H * 2 * D * BF)     # [W1 x_t | tau(t)]
    enc_hid = r.alloc(H * D * BF)
    h = r.alloc(T * D * BF)               # normalised / modulated activations
    qkv = r.alloc(T * 3 * D * BF)         # [Q | K | V] column blocks (cross-attention blocks use the Q block only)
    attn = r.alloc(T * D * BF)
    ff = r.alloc(T * cfg.mlp * BF)
    out_hid = r.alloc(T * cfg.out_dim * BF)
    dec_hid = r.alloc(H * cfg.encoder_hidden * BF)
    velocity = r.alloc(H * cfg.action_dim * BF)

    if block_kernel:
        # the blocks' pointers, once per chunk: 16 slots per block in the order the kernel reads them
        table = r.alloc(cfg.layers * 16 * 8)
        for l in range(cfg.layers):
            b = f"{P}.dit.blocks.{l}"
            names = ["attn.to_q", "attn.to_k", "attn.to_v", "attn.to_out", "ff.fc1", "ff.fc2"]
            row = [Weight(f"{b}.{n}.{kind}") for n in names for kind in ("weight", "bias")]
            row += [mods[l], *(kv[l] if cfg.is_cross(l) else (mods[l], mods[l]))]
            r.store_pointers(table, l * 16, row)
        cross_mask = sum(1 << l for l in range(cfg.layers) if cfg.is_cross(l))

    for step in range(S):
        mod_row = step * 2 * D * BF       # this step's (scale | shift) row inside each mods[l]
        # action encoder: tokens 1..H of the sequence
        lin(x_bf, f"{P}.action_encoder.W1", enc_cat, H, D, cfg.action_dim, ldy=2 * D)
        elementwise("agi_timestep_embedding", [enc_cat + D * BF, U32(H), U32(D), U32(2 * D), F32(times[step]), F32(0.0)],
                    H * D // 2, "timestep_embedding")
        lin(enc_cat, f"{P}.action_encoder.W2", enc_hid, H, D, 2 * D, act="silu")
        lin(enc_hid, f"{P}.action_encoder.W3", seq + D * BF, H, D, D)
        elementwise("agi_add_rows_bf16", [seq + D * BF, Weight(f"{P}.position_embedding.weight"), U32(H), U32(D), U32(D),
                                          U32(H)], H * D, "add_position_embedding")
        elementwise("agi_copy_rows_bf16", [state_tok, seq, U32(1), U32(D), U32(D), U32(D)], D, "copy")

        if block_kernel:
            r.dit_blocks(table, seq, qkv, attn, ff, layers=cfg.layers, T=T, D=D, heads=cfg.heads, head_dim=cfg.head_dim,
                         mlp=cfg.mlp, ctx=cfg.backbone_tokens, cross_mask=cross_mask, mod_offset=step * 2 * D,
                         eps=cfg.ln_eps)
        for l in range(0 if block_kernel else cfg.layers):
            b = f"{P}.dit.blocks.{l}"
            adaln = {"eps": cfg.ln_eps, "scale": mods[l] + mod_row, "shift": mods[l] + (mod_row + D * BF)}
            part = lambda name, n: (Weight(f"{b}.{name}.weight"), Weight(f"{b}.{name}.bias"), n)
            if cfg.is_cross(l):
                r.fused_linear(seq, [part("attn.to_q", D)], qkv, T, D, ln=adaln, ln_scratch=h, ldy=3 * D, fuse=fuse)
                k_buf, v_buf, kv_rows, kv_stride = (*kv[l], cfg.backbone_tokens, D)
            else:
                r.fused_linear(seq, [part("attn.to_q", D), part("attn.to_k", D), part("attn.to_v", D)], qkv, T, D,
                               ln=adaln, ln_scratch=h, ldy=3 * D, fuse=fuse)
                k_buf, v_buf, kv_rows, kv_stride = qkv + D * BF, qkv + 2 * D * BF, T, 3 * D
            # the context keys / values were projected before this step's position-embedding add (a launch that
            # releases its successors only after its own wait): safe to request ahead of the dependency wait
            r.attention(qkv, k_buf, v_buf, attn, q_rows=T, kv_rows=kv_rows, q_heads=cfg.heads, kv_heads=cfg.heads,
                        head_dim=cfg.head_dim, q_stride=3 * D, k_stride=kv_stride, v_stride=kv_stride, o_stride=D,
                        kv_static=cfg.is_cross(l))
            lin(attn, f"{b}.attn.to_out", seq, T, D, D, residual=seq)
            r.fused_linear(seq, [part("ff.fc1", cfg.mlp)], ff, T, D, ln={"eps": cfg.ln_eps}, ln_scratch=h,
                           act="gelu_tanh", fuse=fuse)
            lin(ff, f"{b}.ff.fc2", seq, T, D, cfg.mlp, residual=seq)

        r.fused_linear(seq, [(Weight(f"{P}.dit.proj_out.weight"), Weight(f"{P}.dit.proj_out.bias"), cfg.out_dim)],
                       out_hid, T, D, ln={"eps": cfg.ln_eps, "scale": mods[cfg.layers] + mod_row,
                                          "shift": mods[cfg.layers] + (mod_row + D * BF)}, ln_scratch=h, fuse=fuse)
        lin(out_hid + cfg.out_dim * BF, f"{P}.action_decoder.fc1", dec_hid, H, cfg.encoder_hidden, cfg.out_dim, act="relu")
        lin(dec_hid, f"{P}.action_decoder.fc2", velocity, H, cfg.action_dim, cfg.encoder_hidden)
        elementwise("agi_euler_step", [x_f32, velocity, x_bf, F32(1.0 / S), U32(H * cfg.action_dim)],
                    H * cfg.action_dim, "euler_step")

    r.launch("agi_copy_u32", (1, 1, 1), (256, 1, 1), [x_f32, Tensor("actions"), U32(H * cfg.action_dim)],
             op="copy_out")
    if profile is not None:
        r.export_status(Tensor("status"))   # 0 = every bounded wait of the chunk was satisfied

    if measure and block_kernel:
        # Measurement profiles of the persistent block kernel: the pointer table plus 1 resp. 5 launches of one
        # denoising step's blocks and nothing else (same kernel, geometry and weights as above; the residual stream
        # starts from zeros).  (time of "blocks_5" - time of "blocks_1") / 4 is the duration of one launch.
        for count in (1, 5):
            r.begin_profile(f"blocks_{count}", [io("token", "I32", [1])], [io("status", "I32", [1])])
            r.launch("agi_fill_u32", (4, 1, 1), (256, 1, 1), [seq, U32(0), U32(T * D * BF // 4)], op="clear")
            for l in range(cfg.layers):
                b = f"{P}.dit.blocks.{l}"
                names = ["attn.to_q", "attn.to_k", "attn.to_v", "attn.to_out", "ff.fc1", "ff.fc2"]
                row = [Weight(f"{b}.{n}.{kind}") for n in names for kind in ("weight", "bias")]
                r.store_pointers(table, l * 16, row + [mods[l], *(kv[l] if cfg.is_cross(l) else (mods[l], mods[l]))])
            for _ in range(count):
                r.dit_blocks(table, seq, qkv, attn, ff, layers=cfg.layers, T=T, D=D, heads=cfg.heads,
                             head_dim=cfg.head_dim, mlp=cfg.mlp, ctx=cfg.backbone_tokens, cross_mask=cross_mask,
                             mod_offset=0, eps=cfg.ln_eps)
            r.export_status(Tensor("status"))
    elif measure:
        # Measurement profile: the weight-streaming GEMM launches of ONE denoising step, back to back and
        # nothing else (same kernels, tilings and weights as above; the LayerNorm launches between them are
        # left out; activations are whatever the arena holds).  Timing it gives the
        # weight-streaming rate of the dominant kernel in isolation.
        r.begin_profile("gemm_stream", [io("token", "I32", [1])], [io("status", "I32", [1])])
        for l in range(cfg.layers):
            b = f"{P}.dit.blocks.{l}"
            part = lambda name, n: (Weight(f"{b}.{name}.weight"), Weight(f"{b}.{name}.bias"), n)
            names = ["attn.to_q"] if cfg.is_cross(l) else ["attn.to_q", "attn.to_k", "attn.to_v"]
            first = r.launch_count()
            r.fused_linear(seq, [part(n, D) for n in names], qkv, T, D, ln={"eps": cfg.ln_eps}, ln_scratch=h,
                           ldy=3 * D, fuse=fuse)
            lin(attn, f"{b}.attn.to_out", seq, T, D, D, residual=seq)
            r.fused_linear(seq, [part("ff.fc1", cfg.mlp)], ff, T, D, ln={"eps": cfg.ln_eps}, ln_scratch=h,
                           act="gelu_tanh", fuse=fuse)
            lin(ff, f"{b}.ff.fc2", seq, T, D, cfg.mlp, residual=seq)
            r.drop_launches(first, "agi_layernorm_bf16")   # emitted exactly as in the chunk, minus the norms
        r.export_status(Tensor("status"))


def stream_profile_bytes(cfg: DitConfig = DitConfig()) -> tuple[int, int]:
    """(algorithmic bytes, GEMM launches) of the ``gemm_stream`` profile: per launch
    N*K*2 (weights) + M*K*2 (activations in) + M*N*2 (out) + N*2 (bias), residual reads included."""
    D, T, total, count = cfg.hidden, cfg.tokens, 0, 0
    for l in range(cfg.layers):
        shapes = [(D if cfg.is_cross(l) else 3 * D, D, False), (D, D, True), (cfg.mlp, D, False), (D, cfg.mlp, True)]
        for N, K, residual in shapes:
            total += N * K * 2 + T * K * 2 + T * N * 2 + N * 2 + (T * N * 2 if residual else 0)
            count += 1
    return total, count


def algorithmic_bytes(cfg: DitConfig = DitConfig()) -> dict[str, int]:
    """Weight bytes one action chunk must stream from HBM, by the accounting of the recipe above."""
    shapes = weight_shapes(cfg)
    size = {k: 2 * int(__import__("math").prod(v)) for k, v in shapes.items()}
    once = sum(v for k, v in size.items() if any(t in k for t in (
        "state_encoder", "timestep_embedder", "norm1.linear", "norm_out.linear")))
    once += sum(v for k, v in size.items() if (".attn.to_k" in k or ".attn.to_v" in k)
                and cfg.is_cross(int(k.split(".blocks.")[1].split(".")[0])))
    per_step = sum(size.values()) - once
    return {"once": once, "per_step": per_step, "per_chunk": once + cfg.steps * per_step, "total_weights": sum(size.values())}

"""Launch recipe of a Qwen2.5-VL-shaped backbone prefill (vision tower -> merger -> language model), FP8.

Default shape (the 3B model's): vision encoder of 32 blocks x 1280 (16 heads of 80, SwiGLU 3420, RMSNorm),
patches of 14 x 14 x 2 frames, attention inside 112-pixel windows (8 x 8 patches = 64 tokens) except blocks
7/15/23/31 which attend over the whole image (256 tokens), 2 x 2 patch merger 5120 -> 5120 -> 2048; language
model of 36 layers x 2048 (16 query / 2 KV heads of 128, SwiGLU 11008), M-RoPE sections (16, 24, 24); prefix
= 2 images x 64 merged tokens + 160 text tokens = 288.  Linear weights are E4M3 with per-tensor fp32 scales
(``<name>.weight_scale``); every GEMM input is quantised per tensor on the device (amax / 448).

What the shape description leaves open is fixed here and mirrored by the CPU oracle:
  * tokens run in window order from the patch gather on (see csrc/kernels/vision.cuh); merged tokens return to
    raster order when they are written into the language model's hidden states;
  * vision rotary embedding: half-split pairs over the 80-wide head, the first 20 pairs turn with the patch
    row, the last 20 with the patch column, each group over the same frequency ladder theta^(-j/20), j = 0..19,
    theta = 10000 (the published Qwen2.5-VL vision rotary);
  * all vision linears carry a bias; in the language model only q/k/v do;
  * merger = RMSNorm(1280) -> concat of the 4 patches of a group -> Linear + GELU(tanh) -> Linear;
  * image tokens come first in the prefix (image 0, image 1), then the text tokens; M-RoPE positions are an
    input tensor [3, 288] (``synthetic_inputs`` builds them: an image's tokens share the temporal position and
    count rows / columns of the merged grid from it; text continues after the largest position so far);
  * the SwiGLU width 3420 is stored padded to 3456 (zero rows / columns, numerically inert) so that K is a
    whole number of 128-byte blocks; the patch embedding's K = 1176 is padded to 1216 the same way.
Outputs: the final-norm hidden states [288, 2048], the rotated K / V of every layer [36, 2, 288, 256] and the
status word (0 = every bounded wait in every kernel succeeded).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Sequence

from .builder import RecipeBuilder, Tensor, U32, Weight, ceil_div, grid_for, io
from .layout import pack_kblock_swizzled, padded_token_rows


@dataclass(frozen=True)
class VlConfig:
    # vision tower
    images: int = 2
    image_size: int = 224
    channels: int = 3
    patch: int = 14
    temporal: int = 2
    window: int = 8                     # patches per window side (112 px)
    merge: int = 2
    v_layers: int = 32
    v_hidden: int = 1280
    v_heads: int = 16
    v_mlp: int = 3420
    v_full_layers: tuple[int, ...] = (7, 15, 23, 31)
    v_theta: float = 10000.0
    # language model
    layers: int = 36
    hidden: int = 2048
    heads: int = 16
    kv_heads: int = 2
    head_dim: int = 128
    intermediate: int = 11008
    vocab: int = 151936
    text_tokens: int = 160
    theta: float = 1e6
    sections: tuple[int, int, int] = (16, 24, 24)
    eps: float = 1e-6

    @property
    def grid(self) -> int:               # patches per image side
        return self.image_size // self.patch

    @property
    def patches(self) -> int:
        return self.images * self.grid * self.grid

    @property
    def patch_elems(self) -> int:
        return self.channels * self.temporal * self.patch * self.patch

    @property
    def patch_k(self) -> int:            # padded to whole 128-byte bf16 blocks
        return ceil_div(self.patch_elems, 64) * 64

    @property
    def v_mlp_padded(self) -> int:
        return ceil_div(self.v_mlp, 128) * 128

    @property
    def v_head_dim(self) -> int:
        return self.v_hidden // self.v_heads

    @property
    def merged(self) -> int:             # image tokens the language model sees
        return self.patches // (self.merge * self.merge)

    @property
    def merged_dim(self) -> int:
        return self.v_hidden * self.merge * self.merge

    @property
    def tokens(self) -> int:
        return self.merged + self.text_tokens

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim


def vision_linears(cfg: VlConfig, i: int) -> dict[str, tuple[int, int, int, int]]:
    """name -> (N stored, K stored, N real, K real) of block i's FP8 linears."""
    H, I, Ip = cfg.v_hidden, cfg.v_mlp, cfg.v_mlp_padded
    b = f"visual.blocks.{i}"
    return {f"{b}.attn.qkv": (3 * H, H, 3 * H, H), f"{b}.attn.proj": (H, H, H, H),
            f"{b}.mlp.gate_proj": (Ip, H, I, H), f"{b}.mlp.up_proj": (Ip, H, I, H), f"{b}.mlp.down_proj": (H, Ip, H, I)}


def llm_linears(cfg: VlConfig, i: int) -> dict[str, tuple[int, int]]:
    H, I = cfg.hidden, cfg.intermediate
    l = f"model.layers.{i}"
    return {f"{l}.self_attn.q_proj": (cfg.q_dim, H), f"{l}.self_attn.k_proj": (cfg.kv_dim, H),
            f"{l}.self_attn.v_proj": (cfg.kv_dim, H), f"{l}.self_attn.o_proj": (H, cfg.q_dim),
            f"{l}.mlp.gate_proj": (I, H), f"{l}.mlp.up_proj": (I, H), f"{l}.mlp.down_proj": (H, I)}


def synthetic_weights(cfg: VlConfig, seed: int = 3, std: float = 0.02) -> dict:
    """Random-init checkpoint: linears ~ N(0, std) quantised per tensor to E4M3 (scale = amax / 448), biases
    ~ N(0, std) bf16, norm gains 1, embedding table and patch embedding bf16."""
    import torch
    g = torch.Generator().manual_seed(seed)
    out: dict = {}

    def fp8(name: str, n: int, k: int, n_real: int | None = None, k_real: int | None = None) -> None:
        n_real, k_real = n_real or n, k_real or k
        w = torch.zeros(n, k)
        w[:n_real, :k_real] = torch.randn(n_real, k_real, generator=g) * std
        scale = w.abs().max() / 448.0
        out[f"{name}.weight"] = (w / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
        out[f"{name}.weight_scale"] = scale.reshape(()).float()

    def bias(name: str, n: int, n_real: int | None = None) -> None:
        b = torch.zeros(n)
        b[:n_real or n] = torch.randn(n_real or n, generator=g) * std
        out[f"{name}.bias"] = b.to(torch.bfloat16)

    ones = lambda n: torch.ones(n, dtype=torch.bfloat16)
    pe = torch.zeros(cfg.v_hidden, cfg.patch_k)
    pe[:, :cfg.patch_elems] = torch.randn(cfg.v_hidden, cfg.patch_elems, generator=g) * std
    out["visual.patch_embed.proj.weight"] = pe.to(torch.bfloat16)
    for i in range(cfg.v_layers):
        for name, (n, k, n_real, k_real) in vision_linears(cfg, i).items():
            fp8(name, n, k, n_real, k_real)
            bias(name, n, n_real)
        out[f"visual.blocks.{i}.norm1.weight"] = ones(cfg.v_hidden)
        out[f"visual.blocks.{i}.norm2.weight"] = ones(cfg.v_hidden)
    out["visual.merger.ln_q.weight"] = ones(cfg.v_hidden)
    fp8("visual.merger.mlp.0", cfg.merged_dim, cfg.merged_dim)
    bias("visual.merger.mlp.0", cfg.merged_dim)
    fp8("visual.merger.mlp.2", cfg.hidden, cfg.merged_dim)
    bias("visual.merger.mlp.2", cfg.hidden)
    out["model.embed_tokens.weight"] = (torch.randn(cfg.vocab, cfg.hidden, generator=g) * std).to(torch.bfloat16)
    for i in range(cfg.layers):
        for name, (n, k) in llm_linears(cfg, i).items():
            fp8(name, n, k)
        for p in ("q_proj", "k_proj", "v_proj"):
            bias(f"model.layers.{i}.self_attn.{p}", cfg.q_dim if p == "q_proj" else cfg.kv_dim)
        out[f"model.layers.{i}.input_layernorm.weight"] = ones(cfg.hidden)
        out[f"model.layers.{i}.post_attention_layernorm.weight"] = ones(cfg.hidden)
    out["model.norm.weight"] = ones(cfg.hidden)
    return out


def pack_checkpoint(weights: dict) -> dict:
    """Packaging-time layout pass: every E4M3 linear weight [N, K] is replaced (same name) by its packed form
    [K / 128, N padded to 256, 128] for the bulk-copy tensor-core GEMM (see ``layout.py``).  The values are
    untouched, so the oracle keeps using the row-major checkpoint."""
    import torch
    return {k: pack_kblock_swizzled(v) if v.dtype == torch.float8_e4m3fn and v.dim() == 2 else v
            for k, v in weights.items()}


def rope_positions(cfg: VlConfig):
    """M-RoPE position streams [3, tokens] int32 for [image 0 | image 1 | ... | text]."""
    import torch
    G = cfg.grid // cfg.merge
    pos = torch.zeros(3, cfg.tokens, dtype=torch.int32)
    start, at = 0, 0
    for _ in range(cfg.images):
        ys, xs = torch.meshgrid(torch.arange(G), torch.arange(G), indexing="ij")
        pos[0, at:at + G * G] = start
        pos[1, at:at + G * G] = start + ys.reshape(-1).int()
        pos[2, at:at + G * G] = start + xs.reshape(-1).int()
        start, at = start + G, at + G * G
    text = torch.arange(cfg.text_tokens, dtype=torch.int32) + start
    pos[:, at:] = text
    return pos


def synthetic_inputs(cfg: VlConfig, seed: int = 3) -> dict:
    import torch
    g = torch.Generator().manual_seed(seed + 1000)
    return {"pixels": torch.rand(cfg.images, cfg.channels, cfg.image_size, cfg.image_size, generator=g),
            "input_ids": torch.randint(0, cfg.vocab, (cfg.text_tokens,), generator=g, dtype=torch.int32),
            "positions": rope_positions(cfg)}


def build_recipe(cfg: VlConfig, weights, gemm_tactic: str = "auto", trace: bool = False,
                 group: bool = True, packed: bool = False, extra_inputs=(), extra_outputs=(), tail=None,
                 extra_counters: int = 0, operand_trace: Sequence[str] = ()) -> RecipeBuilder:
    """``weights``: name -> (dtype, shape) as from ``package.describe``.  ``trace`` adds three outputs for
    block-by-block checks: ``vision_trace`` [v_layers + 1, patches, 1280] (the patch embedding, then every
    block's output), ``merged_out`` [merged, hidden] (window order) and ``hidden_trace``
    [layers + 1, tokens, hidden] (the assembled prefix, then every decoder layer's output).  ``group`` runs the
    projections that share an input (Q | K | V, gate | up) as one launch each.  ``packed``: ``weights`` describes
    a checkpoint that went through ``pack_checkpoint``; activations are quantised into the same layout and every
    FP8 GEMM fills its ring with bulk copies.  ``tail(recipe, cache, hidden)`` appends launches that consume the
    prefill inside the same profile (an action expert reading the K/V cache), with ``extra_inputs`` /
    ``extra_outputs`` added to the profile's interface.  ``operand_trace`` (row-major operands only): names of
    blocks (``visual.blocks.3``, ``model.layers.0`` ...) whose four quantised GEMM inputs are exported as they
    stand in front of the GEMM: outputs ``<block>.operand<j>`` (E4M3 bytes [rows, K]) and ``<block>.scale<j>``
    (fp32), j = 0..3 = after the first norm, after attention, after the second norm, after SwiGLU."""
    BF = 2
    P, VH, VD, VI = cfg.patches, cfg.v_hidden, cfg.v_head_dim, cfg.v_mlp_padded
    S, H, I, D = cfg.tokens, cfg.hidden, cfg.intermediate, cfg.head_dim
    G = cfg.grid // cfg.merge
    assert not (operand_trace and packed), "operands are exported in the row-major layout only"
    operand_shapes = {}
    for block in operand_trace:
        rows, ks = (P, (VH, VH, VH, VI)) if block.startswith("visual.") else (S, (H, cfg.q_dim, H, I))
        operand_shapes[block] = [(rows, k) for k in ks]
    operand_outputs = [spec for block, shapes in operand_shapes.items() for j, (rows, k) in enumerate(shapes)
                       for spec in (io(f"{block}.operand{j}", "F8_E4M3", [rows, k]), io(f"{block}.scale{j}", "F32", [1]))]
    r = RecipeBuilder(weights, counter_slots=4 * (cfg.v_layers + cfg.layers) + 8 + extra_counters)   # one per quantisation
    r.begin_profile("default",
                    [io("pixels", "F32", [cfg.images, cfg.channels, cfg.image_size, cfg.image_size]),
                     io("input_ids", "I32", [cfg.text_tokens]), io("positions", "I32", [3, S]), *extra_inputs],
                    [io("hidden_out", "BF16", [S, H]), io("kv_cache", "BF16", [cfg.layers, 2, S, cfg.kv_dim]),
                     io("status", "I32", [1]), *extra_outputs, *operand_outputs] + ([io("vision_trace", "BF16", [cfg.v_layers + 1, P, VH]),
                                                   io("merged_out", "BF16", [cfg.merged, H]),
                                                   io("hidden_trace", "BF16", [cfg.layers + 1, S, H])] if trace else []))
    rows_of = padded_token_rows if packed else (lambda m: m)
    quant = r.alloc(max(rows_of(P) * max(VH, VI), rows_of(cfg.merged) * cfg.merged_dim, rows_of(S) * max(H, I, cfg.q_dim)))
    scale = r.alloc(4)

    traces: list[tuple[object, str, int]] = []       # (arena buffer, output tensor, bytes): copied out at the end

    def snapshot(src, name: str, index: int, nbytes: int) -> None:
        """Keep a copy of ``src`` for output ``name``[index] (trace mode only)."""
        if trace:
            keep = r.alloc(nbytes)
            r.launch("agi_copy_u32", (grid_for(nbytes // 4), 1, 1), (256, 1, 1), [src, keep, U32(nbytes // 4)], op="trace")
            traces.append((keep, name, index, nbytes))

    watched: dict[str, int] = {}      # block being built -> quantisations seen so far (operand_trace only)

    def quantize(x, rows: int, K: int, amax=None):
        r.quantize_e4m3(x, quant, scale, rows * K, amax=amax, packed=(rows, K) if packed else None)
        for block in watched:
            j = watched[block]
            r.launch("agi_copy_u32", (grid_for(rows * K // 4), 1, 1), (256, 1, 1),
                     [quant, Tensor(f"{block}.operand{j}"), U32(rows * K // 4)], op="trace")
            r.launch("agi_copy_u32", (1, 1, 1), (32, 1, 1), [scale, Tensor(f"{block}.scale{j}"), U32(1)], op="trace")
            watched[block] = j + 1

    def watch(block: str) -> None:
        watched.clear()
        if block in operand_shapes:
            watched[block] = 0

    def norm_quantize(x, gain: str, y, rows: int, cols: int, q_rows: int | None = None, q_cols: int | None = None):
        """RMSNorm that also leaves max |y| behind, then the E4M3 quantisation of y (viewed [q_rows, q_cols])."""
        amax = r.counter()
        r.rmsnorm(x, Weight(gain), y, rows, cols, cfg.eps, amax=amax)
        quantize(y, q_rows or rows, q_cols or cols, amax=amax)

    def attention_amax(head_dim: int):
        """A counter for the attention kernel to leave max |o| in, for the head widths that have such a variant."""
        return r.counter() if head_dim in (80, 128) else None

    def swiglu_quantize(gate, up, out, rows: int, cols: int):
        amax = r.counter()
        r.swiglu(gate, up, out, rows, cols, 2 * cols, amax=amax)
        quantize(out, rows, cols, amax=amax)

    def group_q(parts, M: int, K: int) -> None:
        """``parts``: (name, y, N, ldy); FP8 GEMMs over ``quant`` sharing one launch when ``group`` is set."""
        # wide pairs (the decoder's gate | up: 2 x 11008) run faster as two launches of the 256-row kernel than as one
        # grouped launch of 128-row tiles (288 tokens: 2 x 13.6 us against 39.5 us); small parts (K, V) gain from sharing
        if group and gemm_tactic == "auto" and sum(p[2] for p in parts) <= 8192:
            r.gemm_group(quant, [(Weight(f"{n}.weight"), Weight(f"{n}.bias") if f"{n}.bias" in weights else None,
                                  Weight(f"{n}.weight_scale"), y, N, ldy) for n, y, N, ldy in parts], M, K,
                         dtype="e4m3", scale_a=scale, packed=packed)
        else:
            for n, y, N, ldy in parts:
                linear_q(n, y, M, N, K, ldy=ldy)

    def linear_q(name: str, y, M: int, N: int, K: int, **kw) -> None:
        """FP8 GEMM over the activations last quantised into ``quant``."""
        bias = Weight(f"{name}.bias") if f"{name}.bias" in weights else None
        r.gemm(quant, Weight(f"{name}.weight"), y, M, N, K, dtype="e4m3", scale_a=scale,
               scale_w=Weight(f"{name}.weight_scale"), bias=bias, tactic=gemm_tactic, packed=packed, **kw)

    # ---------------- vision tower ----------------
    patches, vpos = r.alloc(P * cfg.patch_k * BF), r.alloc(3 * P * 4)
    x, x2, normed = r.alloc(P * VH * BF), r.alloc(P * VH * BF), r.alloc(P * VH * BF)
    qkv, attn = r.alloc(P * 3 * VH * BF), r.alloc(P * VH * BF)
    gate_up, act = r.alloc(P * 2 * VI * BF), r.alloc(P * VI * BF)
    r.launch("agi_patchify_f32_bf16", (grid_for(P * cfg.patch_k), 1, 1), (256, 1, 1),
             [Tensor("pixels"), patches, vpos, U32(cfg.images), U32(cfg.channels), U32(cfg.image_size), U32(cfg.patch),
              U32(cfg.temporal), U32(cfg.window), U32(cfg.merge), U32(cfg.patch_k), U32(cfg.patch_k)], op="patchify")
    r.gemm(patches, Weight("visual.patch_embed.proj.weight"), x, P, VH, cfg.patch_k, tactic=gemm_tactic)
    snapshot(x, "vision_trace", 0, P * VH * BF)
    half = VD // 2
    for i in range(cfg.v_layers):
        b = f"visual.blocks.{i}"
        watch(b)
        norm_quantize(x, f"{b}.norm1.weight", normed, P, VH)
        linear_q(f"{b}.attn.qkv", qkv, P, 3 * VH, VH)
        # rows x (q heads + k heads) of width 80 sit side by side at the start of each qkv row
        r.mrope(qkv, vpos, P, 2 * cfg.v_heads, VD, 3 * VH, cfg.v_theta, (half // 2, half - half // 2, 0), ladder=half // 2)
        span = cfg.grid * cfg.grid if i in cfg.v_full_layers else cfg.window * cfg.window
        r.attention(qkv, qkv + VH * BF, qkv + 2 * VH * BF, attn, q_rows=P, kv_rows=P, q_heads=cfg.v_heads,
                    kv_heads=cfg.v_heads, head_dim=VD, q_stride=3 * VH, k_stride=3 * VH, v_stride=3 * VH, o_stride=VH,
                    mask="block", mask_arg=span, amax=(a_max := attention_amax(VD)))
        quantize(attn, P, VH, amax=a_max)
        linear_q(f"{b}.attn.proj", x2, P, VH, VH, residual=x)
        norm_quantize(x2, f"{b}.norm2.weight", normed, P, VH)
        group_q([(f"{b}.mlp.gate_proj", gate_up, VI, 2 * VI), (f"{b}.mlp.up_proj", gate_up + VI * BF, VI, 2 * VI)], P, VH)
        swiglu_quantize(gate_up, gate_up + VI * BF, act, P, VI)
        linear_q(f"{b}.mlp.down_proj", x, P, VH, VI, residual=x2)
        snapshot(x, "vision_trace", i + 1, P * VH * BF)
    watch("")
    # merger: per-patch norm; four consecutive rows of 1280 are one row of 5120
    M4, MD = cfg.merged, cfg.merged_dim
    mid, merged = r.alloc(M4 * MD * BF), r.alloc(M4 * H * BF)
    norm_quantize(x, "visual.merger.ln_q.weight", normed, P, VH, M4, MD)
    linear_q("visual.merger.mlp.0", mid, M4, MD, MD, act="gelu_tanh")
    quantize(mid, M4, MD)
    linear_q("visual.merger.mlp.2", merged, M4, H, MD)
    snapshot(merged, "merged_out", 0, M4 * H * BF)

    # ---------------- language model ----------------
    h, h2, hn = r.alloc(S * H * BF), r.alloc(S * H * BF), r.alloc(S * H * BF)
    q_buf, att = r.alloc(S * cfg.q_dim * BF), r.alloc(S * cfg.q_dim * BF)
    cache = r.alloc(cfg.layers * 2 * S * cfg.kv_dim * BF)
    gu, sw = r.alloc(S * 2 * I * BF), r.alloc(S * I * BF)
    r.launch("agi_unwindow_rows_bf16", (grid_for(M4 * H // 8), 1, 1), (256, 1, 1),
             [merged, h, U32(cfg.images), U32(G), U32(cfg.window // cfg.merge), U32(H), U32(H), U32(H)], op="unwindow")
    r.launch("agi_gather_rows_bf16", (grid_for(cfg.text_tokens * H // 8), 1, 1), (256, 1, 1),
             [Weight("model.embed_tokens.weight"), Tensor("input_ids"), h + M4 * H * BF, U32(cfg.text_tokens), U32(H),
              U32(cfg.vocab), U32(H)], op="embedding_gather")
    snapshot(h, "hidden_trace", 0, S * H * BF)
    for i in range(cfg.layers):
        l = f"model.layers.{i}"
        watch(l)
        k_cache = cache + (2 * i) * S * cfg.kv_dim * BF
        v_cache = cache + (2 * i + 1) * S * cfg.kv_dim * BF
        norm_quantize(h, f"{l}.input_layernorm.weight", hn, S, H)
        group_q([(f"{l}.self_attn.q_proj", q_buf, cfg.q_dim, cfg.q_dim), (f"{l}.self_attn.k_proj", k_cache, cfg.kv_dim,
                  cfg.kv_dim), (f"{l}.self_attn.v_proj", v_cache, cfg.kv_dim, cfg.kv_dim)], S, H)
        r.mrope(q_buf, Tensor("positions"), S, cfg.heads, D, cfg.q_dim, cfg.theta, cfg.sections)
        r.mrope(k_cache, Tensor("positions"), S, cfg.kv_heads, D, cfg.kv_dim, cfg.theta, cfg.sections)
        r.attention(q_buf, k_cache, v_cache, att, q_rows=S, kv_rows=S, q_heads=cfg.heads, kv_heads=cfg.kv_heads,
                    head_dim=D, q_stride=cfg.q_dim, k_stride=cfg.kv_dim, v_stride=cfg.kv_dim, o_stride=cfg.q_dim,
                    mask="causal", amax=(a_max := attention_amax(D)))
        quantize(att, S, cfg.q_dim, amax=a_max)
        linear_q(f"{l}.self_attn.o_proj", h2, S, H, cfg.q_dim, residual=h)
        norm_quantize(h2, f"{l}.post_attention_layernorm.weight", hn, S, H)
        group_q([(f"{l}.mlp.gate_proj", gu, I, 2 * I), (f"{l}.mlp.up_proj", gu + I * BF, I, 2 * I)], S, H)
        swiglu_quantize(gu, gu + I * BF, sw, S, I)
        linear_q(f"{l}.mlp.down_proj", h, S, H, I, residual=h2)
        snapshot(h, "hidden_trace", i + 1, S * H * BF)
    watch("")
    r.rmsnorm(h, Weight("model.norm.weight"), Tensor("hidden_out"), S, H, cfg.eps)
    words = cfg.layers * 2 * S * cfg.kv_dim * BF // 4
    r.launch("agi_copy_u32", (grid_for(words), 1, 1), (256, 1, 1), [cache, Tensor("kv_cache"), U32(words)],
             op="export_kv_cache")
    if tail is not None:
        tail(r, cache, h)
    r.export_status(Tensor("status"))
    # trace outputs are whole tensors: gather the kept copies of one output into a contiguous run, copy once
    for name in ("vision_trace", "merged_out", "hidden_trace"):
        parts = sorted((t for t in traces if t[1] == name), key=lambda t: t[2])
        if parts:
            total = sum(t[3] for t in parts)
            run = r.alloc(total)
            at = 0
            for keep, _, _, nbytes in parts:
                r.launch("agi_copy_u32", (grid_for(nbytes // 4), 1, 1), (256, 1, 1), [keep, run + at, U32(nbytes // 4)],
                         op="trace")
                at += nbytes
            r.launch("agi_copy_u32", (grid_for(total // 4), 1, 1), (256, 1, 1), [run, Tensor(name), U32(total // 4)],
                     op="trace")
    return r


def algorithmic(cfg: VlConfig) -> dict[str, int]:
    """Weight bytes streamed and flops of one prefill (real, unpadded shapes)."""
    v = cfg.v_layers * sum(n * k for _, _, n, k in vision_linears(cfg, 0).values())
    merger = cfg.merged_dim * cfg.merged_dim + cfg.hidden * cfg.merged_dim
    llm = cfg.layers * sum(n * k for n, k in llm_linears(cfg, 0).values())
    patch = cfg.v_hidden * cfg.patch_elems
    flops = 2 * (cfg.patches * (v + patch) + cfg.merged * merger + cfg.tokens * llm)
    return {"fp8_weight_bytes": v + merger + llm, "bf16_weight_bytes": 2 * patch + 2 * cfg.text_tokens * cfg.hidden,
            "flops": flops, "params": v + merger + llm + patch}

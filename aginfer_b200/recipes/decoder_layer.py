"""Launch recipe of one Qwen2.5-VL-style decoder layer (prefill): RMSNorm -> QKV (+bias) -> 1-D RoPE ->
GQA causal attention -> O projection + residual -> RMSNorm -> gate/up -> SwiGLU -> down + residual.

Default shape: hidden 2048, 16 query / 2 KV heads of 128, SwiGLU 11008, eps 1e-6, theta 1e6, 288 tokens,
BF16 weights.  ``fp8=True`` builds the same layer with E4M3 linear weights and per-tensor fp32 scales
(``<name>.weight_scale``, ModelOpt style); activations are then quantised per tensor before every GEMM.
Checkpoint names follow Hugging Face (``model.layers.0.self_attn.q_proj.weight`` ...), so q/k/v are not
adjacent in the packed blob and each projection is its own launch writing a column block of one buffer.
"""
from __future__ import annotations

from dataclasses import dataclass

from .builder import RecipeBuilder, Tensor, Weight, io


@dataclass(frozen=True)
class LayerConfig:
    hidden: int = 2048
    heads: int = 16
    kv_heads: int = 2
    head_dim: int = 128
    intermediate: int = 11008
    tokens: int = 288
    eps: float = 1e-6
    theta: float = 1e6
    fp8: bool = False

    @property
    def q_dim(self) -> int:
        return self.heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.kv_heads * self.head_dim


L = "model.layers.0"
LINEARS = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj", "mlp.gate_proj",
           "mlp.up_proj", "mlp.down_proj")


def linear_shapes(cfg: LayerConfig) -> dict[str, tuple[int, int]]:
    H, I = cfg.hidden, cfg.intermediate
    return {"self_attn.q_proj": (cfg.q_dim, H), "self_attn.k_proj": (cfg.kv_dim, H), "self_attn.v_proj": (cfg.kv_dim, H),
            "self_attn.o_proj": (H, cfg.q_dim), "mlp.gate_proj": (I, H), "mlp.up_proj": (I, H), "mlp.down_proj": (H, I)}


def synthetic_weights(cfg: LayerConfig, seed: int = 0, std: float = 0.02) -> dict:
    """BF16 ~ N(0, std) linears, RMSNorm gains 1.0, small QKV biases; with ``cfg.fp8`` the linears are
    quantised per tensor by amax / 448 to E4M3 and their fp32 scales stored beside them."""
    import torch
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in linear_shapes(cfg).items():
        w = torch.randn(shape, generator=g) * std
        if cfg.fp8:
            scale = w.abs().max() / 448.0
            out[f"{L}.{name}.weight"] = (w / scale).clamp(-448, 448).to(torch.float8_e4m3fn)
            out[f"{L}.{name}.weight_scale"] = scale.reshape(()).float()
        else:
            out[f"{L}.{name}.weight"] = w.to(torch.bfloat16)
    for name in ("q_proj", "k_proj", "v_proj"):
        out[f"{L}.self_attn.{name}.bias"] = (torch.randn(linear_shapes(cfg)[f"self_attn.{name}"][0], generator=g) * std
                                             ).to(torch.bfloat16)
    out[f"{L}.input_layernorm.weight"] = torch.ones(cfg.hidden, dtype=torch.bfloat16)
    out[f"{L}.post_attention_layernorm.weight"] = torch.ones(cfg.hidden, dtype=torch.bfloat16)
    return out


def synthetic_input(cfg: LayerConfig, seed: int = 0):
    import torch
    g = torch.Generator().manual_seed(seed + 1000)
    return torch.randn(cfg.tokens, cfg.hidden, generator=g).to(torch.bfloat16)


def build_recipe(cfg: LayerConfig, weights, gemm_tactic: str = "auto") -> RecipeBuilder:
    """``weights``: name -> (dtype, shape) as from ``package.describe``."""
    S, H, I, D = cfg.tokens, cfg.hidden, cfg.intermediate, cfg.head_dim
    qkv_dim = cfg.q_dim + 2 * cfg.kv_dim
    r = RecipeBuilder(weights)
    r.begin_profile("default", [io("hidden_in", "BF16", [S, H])], [io("hidden_out", "BF16", [S, H])])
    BF = 2
    normed, qkv, attn = r.alloc(S * H * BF), r.alloc(S * qkv_dim * BF), r.alloc(S * cfg.q_dim * BF)
    resid, gate_up, act = r.alloc(S * H * BF), r.alloc(S * 2 * I * BF), r.alloc(S * I * BF)
    quant, scale = r.alloc(S * max(H, I, cfg.q_dim)), r.alloc(4)

    def linear(x, name, y, N, K, **kw):
        """One projection; FP8 layers first quantise ``x`` per tensor (amax / 448) into ``quant``."""
        w = Weight(f"{L}.{name}.weight")
        if cfg.fp8:
            r.quantize_e4m3(x, quant, scale, S * K)
            r.gemm(quant, w, y, S, N, K, dtype="e4m3", scale_a=scale, scale_w=Weight(f"{L}.{name}.weight_scale"),
                   tactic=gemm_tactic, **kw)
        else:
            r.gemm(x, w, y, S, N, K, tactic=gemm_tactic, **kw)

    r.rmsnorm(Tensor("hidden_in"), Weight(f"{L}.input_layernorm.weight"), normed, S, H, cfg.eps)
    col = 0
    for name, width in (("q_proj", cfg.q_dim), ("k_proj", cfg.kv_dim), ("v_proj", cfg.kv_dim)):
        linear(normed, f"self_attn.{name}", qkv + col * BF, width, H, bias=Weight(f"{L}.self_attn.{name}.bias"),
               ldy=qkv_dim)
        col += width
    r.rope(qkv, S, cfg.heads + cfg.kv_heads, D, qkv_dim, cfg.theta)
    r.attention(qkv, qkv + cfg.q_dim * BF, qkv + (cfg.q_dim + cfg.kv_dim) * BF, attn, q_rows=S, kv_rows=S,
                q_heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=D, q_stride=qkv_dim, k_stride=qkv_dim,
                v_stride=qkv_dim, o_stride=cfg.q_dim, mask="causal")
    linear(attn, "self_attn.o_proj", resid, H, cfg.q_dim, residual=Tensor("hidden_in"))
    r.rmsnorm(resid, Weight(f"{L}.post_attention_layernorm.weight"), normed, S, H, cfg.eps)
    linear(normed, "mlp.gate_proj", gate_up, I, H, ldy=2 * I)
    linear(normed, "mlp.up_proj", gate_up + I * BF, I, H, ldy=2 * I)
    r.swiglu(gate_up, gate_up + I * BF, act, S, I, 2 * I)
    linear(act, "mlp.down_proj", Tensor("hidden_out"), H, I, residual=resid)
    return r


def algorithmic(cfg: LayerConfig) -> dict[str, int]:
    """Weight bytes and flops of the layer (what the roofline floors are computed from)."""
    params = sum(n * k for n, k in linear_shapes(cfg).values())
    return {"weight_bytes": params * (1 if cfg.fp8 else 2), "flops": 2 * cfg.tokens * params, "params": params}

"""Launch recipe of a GR00T-N1.5-shaped vision-language-action model end to end: ONE profile from pixels and
token ids to the action chunk.

Backbone: the Qwen2.5-VL-3B-shaped FP8 prefill of ``qwen_vl.py`` (BASELINE config 4: 2 images + 160 text tokens
= 288 tokens of width 2048).  Head: the flow-matching DiT of ``dit.py`` (BASELINE config 3: 16 blocks x 1536,
1 state + 16 action tokens, 4 Euler steps), cross-attending to the backbone's final hidden states: the head's
context is the prefill's ``hidden_out`` (after the final RMSNorm), all 288 tokens of it, so the two halves meet
inside the profile without a trip through the caller.  Inputs: ``pixels``, ``input_ids``, ``positions``,
``state``, ``noise``; outputs: ``actions`` [16, 32] fp32, plus the prefill's ``hidden_out`` and ``kv_cache``.

Checkpoint: the backbone's tensors (``visual.*``, ``model.*``; E4M3 linears with ``weight_scale``) and the
head's (``action_head.*``, BF16) in one directory.
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace

from . import dit, qwen_vl
from .builder import RecipeBuilder, Tensor, io


@dataclass(frozen=True)
class VlaConfig:
    backbone: qwen_vl.VlConfig = qwen_vl.VlConfig()
    head: dit.DitConfig = field(default_factory=lambda: dit.DitConfig(backbone_tokens=288))

    def __post_init__(self):
        if self.head.backbone_tokens != self.backbone.tokens or self.head.backbone_dim != self.backbone.hidden:
            raise ValueError("the head's context must be the backbone's prefix: "
                             f"{self.backbone.tokens} tokens of width {self.backbone.hidden}")


def synthetic_weights(cfg: VlaConfig) -> dict:
    """Backbone (seed 3) and head (seed 2) checkpoints side by side."""
    return {**qwen_vl.synthetic_weights(cfg.backbone), **dit.synthetic_weights(cfg.head, seed=2)}


def synthetic_inputs(cfg: VlaConfig) -> dict:
    head = dit.synthetic_inputs(cfg.head, seed=2)
    return {**qwen_vl.synthetic_inputs(cfg.backbone), "state": head["state"], "noise": head["noise"]}


def build_recipe(cfg: VlaConfig, weights, packed: bool = False, block_kernel: bool = False) -> RecipeBuilder:
    """``weights``: name -> (dtype, shape) of the joint checkpoint (``package.describe``)."""
    H = cfg.head

    def head(r: RecipeBuilder, _cache, _hidden) -> None:
        # the prefill's last launch wrote the normalised hidden states into the output tensor: that is the context
        dit.emit_action_head(r, H, Tensor("hidden_out"), block_kernel=block_kernel)

    return qwen_vl.build_recipe(cfg.backbone, weights, packed=packed, extra_inputs=dit.head_inputs(H),
                                extra_outputs=[io("actions", "F32", [H.horizon, H.action_dim])], tail=head,
                                extra_counters=8)


def reduced(v_layers: int = 2, layers: int = 2, head_layers: int = 4, vocab: int = 2048) -> VlaConfig:
    """Real widths and token counts at reduced depth (tests)."""
    full = tuple(i for i in (7, 15, 23, 31) if i < v_layers) or (v_layers - 1,)
    return VlaConfig(replace(qwen_vl.VlConfig(), v_layers=v_layers, v_full_layers=full, layers=layers, vocab=vocab),
                     dit.DitConfig(layers=head_layers, backbone_tokens=288))

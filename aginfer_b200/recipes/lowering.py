"""From an adapter's graph description to the sm100 artifact set: ``modelc plan``.

The reference's adapters only NAME what a lowering would do (``src/aginfer/adapters/groot.py:13-29``: passes
``fuse_qkv``, ``fuse_mlp``, ``fuse_norm`` ...; subgraphs ``vision``, ``vlm_conditioning``,
``flow_matching_dit_step``; a recipe with a once-per-episode conditioning part and a denoising loop), and its
compiler expects somebody else to have written ``<artifact-dir>/<arch>/{kernels.cubin,plan.json,tactics.json}``
(``src/aginfer/compiler.py:61-75``).  This module is that somebody for sm100: it reads the checkpoint's tensor
inventory and shape description, picks the recipe generator the adapter's subgraphs call for, turns the pass
names into the generator's fusion choices, and writes the artifact directory.

Where the model's shape comes from: ``config.json`` may carry a section ``"aginfer_recipe": {"name": ...,
"config": {...}}`` (the synthetic checkpoints of this repository write one); without it the action-head shape is
read off the tensor shapes, and the step count / horizon / state width off the shape profile.
"""
from __future__ import annotations

import dataclasses
import json
import re
from pathlib import Path
from typing import Any, Mapping, Sequence

from ..errors import ValidationError
from . import decoder_layer, dit, lingbot, qwen_vl, vla
from .builder import RecipeBuilder

Inventory = Mapping[str, tuple[str, tuple[int, ...]]]      # tensor name -> (dtype, shape)

# What each graph pass of the adapters becomes in the generators (recorded in tactics.json as op "graph_pass").
PASS_LOWERING = {
    "fuse_qkv": "Q | K | V projections of a block share one launch (grouped tensor-core GEMM / side-by-side weight "
                "matrices in the weight-streaming kernel); cross-attention K/V of all blocks in one batched launch",
    "fuse_mlp": "gate | up share one grouped launch; activation (GELU / SiLU / SwiGLU input) in the GEMM epilogue; "
                "residual add in the down projection's epilogue",
    "fuse_norm": "norms fold the amax of the dynamic FP8 quantisation that follows; AdaLN modulation inside the "
                 "LayerNorm kernel; all steps' modulation vectors computed once in front of the denoising loop",
    "constant_fold": "step times, rotary tables' arguments and shapes are literals of the launch list",
    "eliminate_view_ops": "views are byte offsets and leading dimensions of launch arguments",
    "remove_training_nodes": "nothing of the kind is emitted",
    "deduplicate_tied_weights": "one blob entry per checkpoint tensor; launches share offsets",
}


def config_from_dict(cls, values: Mapping[str, Any]):
    """A (possibly nested) frozen dataclass from plain JSON values; unknown keys are an error."""
    fields = {f.name: f for f in dataclasses.fields(cls)}
    unknown = set(values) - set(fields)
    if unknown:
        raise ValidationError(f"unknown {cls.__name__} fields: {sorted(unknown)}")
    built = {}
    for key, value in values.items():
        default = fields[key].default
        if default is dataclasses.MISSING and fields[key].default_factory is not dataclasses.MISSING:
            default = fields[key].default_factory()
        if dataclasses.is_dataclass(default) and isinstance(value, Mapping):
            value = config_from_dict(type(default), value)
        elif isinstance(default, tuple) and isinstance(value, list):
            value = tuple(value)
        built[key] = value
    return cls(**built)


def config_to_dict(cfg) -> dict[str, Any]:
    return json.loads(json.dumps(dataclasses.asdict(cfg)))


def infer_dit_config(inventory: Inventory, profile: Mapping[str, Any], heads: int | None) -> dit.DitConfig:
    """The action head's shape from its tensor shapes (names of ``dit.weight_shapes``) and the shape profile."""
    P = dit.P

    def shape(name: str) -> tuple[int, ...]:
        if name not in inventory:
            raise ValidationError(f"checkpoint has no tensor {name}: not an action-head checkpoint of the known layout")
        return inventory[name][1]

    layers = 1 + max((int(m.group(1)) for n in inventory if (m := re.match(rf"{re.escape(P)}\.dit\.blocks\.(\d+)\.", n))),
                     default=-1)
    if layers < 1:
        raise ValidationError("checkpoint has no action_head.dit.blocks.* tensors")
    hidden = shape(f"{P}.dit.blocks.0.attn.to_q.weight")[0]
    cross = next((l for l in range(layers) if shape(f"{P}.dit.blocks.{l}.attn.to_k.weight")[1] != hidden), None)
    first = profile["profiles"][0]
    if heads is None:
        heads = hidden // 48 if hidden % 48 == 0 else hidden // 64     # the two head widths the kernels are built for
    return dit.DitConfig(
        layers=layers, hidden=hidden, heads=heads, head_dim=hidden // heads,
        mlp=shape(f"{P}.dit.blocks.0.ff.fc1.weight")[0], action_dim=shape(f"{P}.action_encoder.W1.weight")[1],
        state_dim=shape(f"{P}.state_encoder.fc1.weight")[1], horizon=shape(f"{P}.position_embedding.weight")[0],
        backbone_tokens=int(first["sequence_length"]["opt"]),
        backbone_dim=shape(f"{P}.dit.blocks.{cross}.attn.to_k.weight")[1] if cross is not None else hidden,
        steps=int(profile.get("default_denoising", {}).get("steps", 4)),
        encoder_hidden=shape(f"{P}.state_encoder.fc1.weight")[0], out_dim=shape(f"{P}.dit.proj_out.weight")[0],
        time_dim=shape(f"{P}.dit.timestep_embedder.linear_1.weight")[1])


def choose_recipe(adapter: str, graph: Mapping[str, Any], inventory: Inventory, config: Mapping[str, Any]) -> str:
    """Which generator the adapter's subgraphs call for, given what the checkpoint actually contains."""
    section = config.get("aginfer_recipe")
    if isinstance(section, Mapping) and section.get("name"):
        return str(section["name"])
    subgraphs = set(graph.get("subgraphs", ()))
    has_head = any(n.startswith(dit.P + ".") for n in inventory)
    has_expert = any(n.startswith(lingbot.E + ".") for n in inventory)
    has_backbone = any(n.startswith(("visual.", "model.")) for n in inventory)
    if "pi_action_expert_step" in subgraphs and has_expert and has_backbone:
        return "lingbot_episode"
    if "flow_matching_dit_step" in subgraphs and has_head:
        return "vla" if has_backbone else "dit"       # with the backbone's tensors: pixels and ids in, actions out
    if has_backbone and not has_head and not has_expert:
        return "qwen_vl_prefill"
    raise ValidationError(f"no sm100 recipe generator for adapter {adapter} with this checkpoint's tensors")


def lower(adapter: str, graph: Mapping[str, Any], inventory: Inventory, config: Mapping[str, Any],
          profile: Mapping[str, Any], *, packed: bool = False, step_profiles: Sequence[int] = (),
          heads: int | None = None) -> tuple[RecipeBuilder, str, dict[str, Any]]:
    """Returns (recipe, generator name, shape config as a dict)."""
    passes = list(graph.get("passes", ()))
    name = choose_recipe(adapter, graph, inventory, config)
    section = config.get("aginfer_recipe") if isinstance(config.get("aginfer_recipe"), Mapping) else {}
    values = section.get("config")
    fused = "fuse_qkv" in passes and "fuse_mlp" in passes
    if name == "dit":
        cfg = config_from_dict(dit.DitConfig, values) if values else infer_dit_config(inventory, profile, heads)
        recipe = dit.build_recipe(cfg, inventory, fuse=fused, batch_kv="fuse_qkv" in passes, step_profiles=tuple(step_profiles))
    elif name == "vla":
        cfg = config_from_dict(vla.VlaConfig, values or {})
        recipe = vla.build_recipe(cfg, inventory, packed=packed)
    elif name == "qwen_vl_prefill":
        cfg = config_from_dict(qwen_vl.VlConfig, values or {})
        recipe = qwen_vl.build_recipe(cfg, inventory, packed=packed)
    elif name == "lingbot_episode":
        cfg = config_from_dict(lingbot.EpisodeConfig, values or {})
        recipe = lingbot.build_recipe(cfg, inventory, packed=packed)
    elif name == "decoder_layer":
        cfg = config_from_dict(decoder_layer.LayerConfig, values or {})
        recipe = decoder_layer.build_recipe(cfg, inventory)
    else:
        raise ValidationError(f"unknown recipe generator {name!r}")
    for p in passes:      # the adapter's pass list, and what became of each, travel in the tactic database
        recipe.tactics[("graph_pass", p)] = {"op": "graph_pass", "algorithm": p, "kernel": "-", "uses": 1,
                                             "lowered_to": PASS_LOWERING.get(p, "no effect on the launch list")}
    recipe.tactics[("recipe", name)] = {"op": "recipe", "algorithm": name, "kernel": "-", "uses": 1,
                                        "adapter": adapter, "subgraphs": list(graph.get("subgraphs", ())),
                                        "packed_operands": bool(packed)}
    return recipe, name, config_to_dict(cfg)


def write_artifact_dir(root: Path, recipe: RecipeBuilder, cubin: Path | None = None) -> Path:
    from .package import write_artifacts
    return write_artifacts(Path(root), recipe, cubin)

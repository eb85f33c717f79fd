"""From tensors + a recipe to an ``.aim`` file, through the same steps a user of ``modelc`` takes:
write a Hugging Face style checkpoint (safetensors + config.json), write the artifact directory
(``toolchain.json``, ``sm100/{kernels.cubin,plan.json,tactics.json}``), write a shape profile, run
``compile_model`` for ``--cuda-arch sm100a``.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Any, Mapping

from ..build import CUBIN, build_kernels
from ..modelc import CompileOptions, compile_model
from ..target import CudaArch, Platform
from ..weights import write_safetensors
from .builder import RecipeBuilder

# CUDA 12.8+ driver/runtime (first toolkits that target sm_100a), cuBLASLt 12, cuDNN 9.
TOOLCHAIN = {"cuda_driver_min": 12080, "cuda_runtime_min": 12080, "cuda_runtime_max": 12999, "cublaslt_abi": 12,
             "cudnn_abi": 9}
FP8_CONFIG = {"quant_method": "modelopt", "quantization_format": "fp8_e4m3", "scales": "explicit"}


def tensor_record(t) -> tuple[str, list[int], bytes]:
    """(safetensors dtype, shape, raw little-endian bytes) of a torch CPU tensor."""
    import torch
    names = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float8_e4m3fn: "F8_E4M3"}
    t = t.detach().contiguous().cpu()
    raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
    return names[t.dtype], list(t.shape), raw


def describe(tensors: Mapping[str, Any]) -> dict[str, tuple[str, tuple[int, ...]]]:
    """name -> (dtype, shape): what ``RecipeBuilder`` needs to lay out the weight blob."""
    import torch
    names = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.float8_e4m3fn: "F8_E4M3"}
    return {k: (names[v.dtype], tuple(v.shape)) for k, v in tensors.items()}


def write_checkpoint(root: Path, tensors: Mapping[str, Any], model_type: str = "groot",
                     recipe: tuple[str, Any] | None = None) -> Path:
    """``recipe``: (generator name, its config dataclass), recorded in ``config.json`` under ``aginfer_recipe`` so
    that ``modelc plan`` can rebuild the launch recipe from the checkpoint directory alone."""
    import torch
    root.mkdir(parents=True, exist_ok=True)
    config: dict[str, Any] = {"model_type": model_type, "architectures": ["SyntheticForActionPrediction"]}
    if recipe is not None:
        import dataclasses
        config["aginfer_recipe"] = {"name": recipe[0], "config": json.loads(json.dumps(dataclasses.asdict(recipe[1])))}
    if any(t.dtype == torch.float8_e4m3fn for t in tensors.values()):
        config["quantization_config"] = dict(FP8_CONFIG)
    (root / "config.json").write_text(json.dumps(config))
    write_safetensors(root / "model.safetensors", {k: tensor_record(v) for k, v in tensors.items()})
    return root


def write_artifacts(root: Path, recipe: RecipeBuilder, cubin: Path | None = None) -> Path:
    folder = root / recipe.arch
    folder.mkdir(parents=True, exist_ok=True)
    (root / "toolchain.json").write_text(json.dumps(TOOLCHAIN))
    source = Path(cubin) if cubin else (CUBIN if CUBIN.exists() else build_kernels())
    (folder / "kernels.cubin").write_bytes(source.read_bytes())
    (folder / "plan.json").write_text(json.dumps(recipe.plan()))
    (folder / "tactics.json").write_text(json.dumps(recipe.tactic_database()))
    return root


def write_profile(path: Path, name: str = "default", steps: int = 4, **ranges: int) -> Path:
    fields = ("sequence_length", "image_height", "image_width", "image_count", "state_length", "action_horizon")
    profile = {"name": name, "batch": 1}
    for f in fields:
        v = int(ranges.get(f, 1))
        profile[f] = {"min": v, "opt": v, "max": v}
    path.write_text(json.dumps({"profiles": [profile], "default_denoising": {"steps": steps}}))
    return path


def build_aim(workdir: Path, tensors: Mapping[str, Any], recipe: RecipeBuilder, *, name: str = "model.aim",
              adapter: str = "groot_n1_5", model_type: str = "groot", steps: int = 4, **ranges: int) -> Path:
    """Package ``tensors`` and ``recipe`` into ``workdir/name`` via ``compile_model``."""
    workdir = Path(workdir)
    checkpoint = write_checkpoint(workdir / "checkpoint", tensors, model_type)
    artifacts = write_artifacts(workdir / "artifacts", recipe)
    profile = write_profile(workdir / "profile.json", steps=steps, **ranges)
    out = workdir / name
    compile_model(CompileOptions(source=str(checkpoint), revision=None, adapter=adapter,
                                 platform=Platform.LINUX_X86_64_GNU, cuda_arches=(CudaArch.SM100,),
                                 profile_path=profile, artifact_dir=artifacts, output=out, offline=True))
    return out

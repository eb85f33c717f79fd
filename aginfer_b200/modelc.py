"""``modelc``: turn a checkpoint plus a per-architecture artifact directory into an ``.aim``.

Replaces the reference's ``src/aginfer/compiler.py:30-115`` (``compile_model``), the
artifact contract it reads (``<dir>/toolchain.json`` and
``<dir>/<arch>/{kernels.cubin,plan.json,tactics.json}``, ``compiler.py:61-75``), the shape
profile loader (``profiles.py:12-57``), the two metadata-only adapters
(``adapters/groot.py``, ``adapters/lingbot.py``) and the command line
(``cli.py:29-94``).  For inputs the reference accepts, the written file is byte-identical
to the reference's; the only additions are the ``sm100`` target row and the new-flavour
CUBIN check (see ``target.py``).
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
from dataclasses import dataclass, replace
from pathlib import Path
from typing import Any

from .container import AimInfo, AimReader, AimWriter, VariantPayload
from .errors import AgInferError, ValidationError
from .planfmt import compile_execution_plan
from .target import RUNTIME_ABI, CudaArch, Platform, ToolchainRange, validate_target
from .weights import Checkpoint, collect_metadata, load_checkpoint, pack_weights

_PASSES = ["constant_fold", "remove_training_nodes", "eliminate_view_ops", "fuse_qkv", "fuse_mlp", "fuse_norm",
           "deduplicate_tied_weights"]
_ONCE = {"execute": "once", "cache": True}
_LOOP = {"execute": "denoising_loop", "schedule": "profile"}

# name -> (model_family, accepted model_type tokens, subgraphs, extra recipe keys)
ADAPTERS: dict[str, tuple[str, tuple[str, ...], list[str], dict[str, Any]]] = {
    "groot_n1_5": ("groot_n1_5", ("groot", "eagle"),
                   ["vision", "vlm_conditioning", "flow_matching_dit_step"], {}),
    "lingbot_vla_1": ("lingbot_vla_1_no_depth", ("lingbot", "qwen2_5_vl", "qwen2.5-vl", "pi0"),
                      ["qwen2_5_vision", "vlm_conditioning", "pi_action_expert_step"], {"depth_input": False}),
}
ADAPTER_VERSION = 1
_IO_IN = [{"name": n, "dtype": d, "location": "device"}
          for n, d in (("input_ids", "I32"), ("pixel_values", "checkpoint"), ("state", "checkpoint"))]
_IO_OUT = [{"name": "actions", "dtype": "checkpoint", "location": "device"}]
_RANGE_FIELDS = ("sequence_length", "image_height", "image_width", "image_count", "state_length", "action_horizon")


def adapter_names() -> tuple[str, ...]:
    return tuple(sorted(ADAPTERS))


def describe_model(adapter: str, checkpoint: Checkpoint) -> tuple[str, dict[str, Any]]:
    """Model family and the static graph/recipe description an adapter contributes."""
    if adapter not in ADAPTERS:
        raise ValidationError(f"unknown adapter {adapter!r}; available: {', '.join(adapter_names())}")
    family, tokens, subgraphs, extra = ADAPTERS[adapter]
    model_type = str(checkpoint.config.get("model_type", "")).lower()
    archs = " ".join(str(a).lower() for a in checkpoint.config.get("architectures", []))
    if not any(t in model_type or t in archs for t in tokens):
        raise ValidationError(
            f"adapter {adapter} does not match checkpoint model_type={model_type!r}; expected one of {tokens}")
    graph = {"opset": 1, "passes": list(_PASSES), "subgraphs": list(subgraphs),
             "recipe": {**extra, "conditioning": dict(_ONCE), "action_head": dict(_LOOP)}}
    return family, graph


def load_profile(path: str | Path) -> dict[str, Any]:
    """Read and check a shape-profile file: JSON, or YAML when PyYAML is importable."""
    source = Path(path)
    try:
        text = source.read_text(encoding="utf-8")
    except OSError as exc:
        raise ValidationError(f"cannot read shape profile {source}: {exc}") from exc
    try:
        value = json.loads(text)
    except json.JSONDecodeError:
        try:
            import yaml
        except ImportError as exc:
            raise ValidationError("non-JSON YAML profiles require: pip install aginfer[yaml]") from exc
        try:
            value = yaml.safe_load(text)
        except Exception as exc:
            raise ValidationError(f"invalid shape profile {source}: {exc}") from exc
    if not isinstance(value, dict):
        raise ValidationError("shape profile must be an object")
    profiles = value.get("profiles")
    if not isinstance(profiles, list) or not profiles:
        raise ValidationError("shape profile requires a non-empty profiles list")
    seen: set[str] = set()
    for i, profile in enumerate(profiles):
        if not isinstance(profile, dict):
            raise ValidationError(f"profile {i} must be an object")
        name = profile.get("name")
        if not isinstance(name, str) or not name or name in seen:
            raise ValidationError(f"profile {i} needs a unique non-empty name")
        seen.add(name)
        if profile.get("batch", 1) != 1:
            raise ValidationError(f"profile {name}: only batch=1 is supported")
        for field in _RANGE_FIELDS:
            bounds = profile.get(field)
            if not isinstance(bounds, dict) or set(bounds) != {"min", "opt", "max"}:
                raise ValidationError(f"profile {name}: {field} must define min, opt, and max")
            try:
                low, mid, high = (int(bounds[k]) for k in ("min", "opt", "max"))
            except (TypeError, ValueError) as exc:
                raise ValidationError(f"profile {name}: {field} bounds must be integers") from exc
            if low <= 0 or not low <= mid <= high:
                raise ValidationError(f"profile {name}: expected 0 < min <= opt <= max for {field}")
    denoising = value.get("default_denoising", {})
    if not isinstance(denoising, dict) or int(denoising.get("steps", 1)) <= 0:
        raise ValidationError("default_denoising.steps must be positive")
    return value


@dataclass(frozen=True)
class CompileOptions:
    source: str
    revision: str | None
    adapter: str
    platform: Platform
    cuda_arches: tuple[CudaArch, ...]
    profile_path: Path
    artifact_dir: Path
    output: Path
    offline: bool = False
    backbone: str | None = None


def _json_object(path: Path, label: str) -> dict[str, Any]:
    try:
        value = json.loads(path.read_text(encoding="utf-8"))
    except (OSError, UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise ValidationError(f"cannot parse {label} {path}: {exc}") from exc
    if not isinstance(value, dict):
        raise ValidationError(f"{label} must contain a JSON object: {path}")
    return value


def read_toolchain(root: Path) -> ToolchainRange:
    value = _json_object(root / "toolchain.json", "toolchain compatibility file")
    try:
        tc = ToolchainRange.from_dict(value)
    except (KeyError, TypeError, ValueError) as exc:
        raise ValidationError(f"invalid toolchain.json: {exc}") from exc
    if tc.cuda_runtime_min <= 0 or tc.cuda_runtime_max < tc.cuda_runtime_min:
        raise ValidationError("toolchain CUDA Runtime range is invalid")
    if min(tc.cuda_driver_min, tc.cublaslt_abi, tc.cudnn_abi) <= 0:
        raise ValidationError("toolchain ABI values must be positive")
    return tc


def check_tactics(value: dict[str, Any], arch: CudaArch) -> None:
    if value.get("cuda_arch") != arch.name_string:
        raise ValidationError(f"tactic database target must be exactly {arch.name_string}")
    entries = value.get("tactics")
    if not isinstance(entries, list) or not entries:
        raise ValidationError(f"no verified tactics available for {arch.name_string}")
    for i, entry in enumerate(entries):
        if not isinstance(entry, dict) or not entry.get("op") or not entry.get("algorithm"):
            raise ValidationError(f"invalid tactic entry {i} for {arch.name_string}")


def compile_model(options: CompileOptions) -> AimInfo:
    if options.output.suffix.lower() != ".aim":
        raise ValidationError("output filename must use the .aim extension")
    try:
        validate_target(options.platform, list(options.cuda_arches))
    except ValueError as exc:
        raise ValidationError(str(exc)) from exc
    profile = load_profile(options.profile_path)
    checkpoint = load_checkpoint(options.source, options.revision, options.offline)
    family, graph = describe_model(options.adapter, checkpoint)

    tensors = list(checkpoint.tensors)
    backbone: Checkpoint | None = None
    if options.adapter == "lingbot_vla_1":
        if not options.backbone:
            raise ValidationError("lingbot_vla_1 requires --backbone so deployment has no QWEN25_PATH dependency")
        backbone = load_checkpoint(options.backbone, None, options.offline)
        taken = {t.name for t in tensors}
        tensors += [replace(t, name=f"backbone.{t.name}") if t.name in taken else t for t in backbone.tensors]

    blob, table = pack_weights(tensors)
    variants, tactic_digest = [], {}
    for arch in options.cuda_arches:
        folder = options.artifact_dir / arch.name_string
        cubin_path = folder / "kernels.cubin"
        try:
            kernels = cubin_path.read_bytes()
        except OSError as exc:
            raise ValidationError(
                f"cannot read precompiled {arch.name_string} kernel bundle {cubin_path}: {exc}") from exc
        if not kernels:
            raise ValidationError(f"empty precompiled {arch.name_string} kernel bundle: {cubin_path}")
        plan = _json_object(folder / "plan.json", "execution plan")
        tactics = _json_object(folder / "tactics.json", "tactic database")
        compiled = compile_execution_plan(plan, arch, weight_size=len(blob))
        check_tactics(tactics, arch)
        tactic_digest[arch.name_string] = {
            "database_sha256": hashlib.sha256((folder / "tactics.json").read_bytes()).hexdigest(),
            "entry_count": len(tactics["tactics"]),
        }
        variants.append(VariantPayload(arch, kernels, blob, compiled.data))

    manifest = {
        "model_family": family,
        "adapter": options.adapter,
        "adapter_version": ADAPTER_VERSION,
        "source": options.source,
        "source_revision": checkpoint.revision,
        "backbone_revision": backbone.revision if backbone else None,
        "platform": options.platform.triple,
        "cuda_arches": [a.name_string for a in options.cuda_arches],
        "runtime_abi": RUNTIME_ABI,
        "toolchain": read_toolchain(options.artifact_dir).to_dict(),
        "checkpoint_dtypes": sorted({t.dtype for t in tensors}),
        "strict_dtype_preservation": True,
        "tf32_default": False,
        "batch": 1,
        "profiles": profile["profiles"],
        "default_denoising": profile.get("default_denoising", {"steps": 1}),
        "inputs": [dict(x) for x in _IO_IN],
        "outputs": [dict(x) for x in _IO_OUT],
        "checkpoint_metadata": collect_metadata(checkpoint.root),
        "tactics": tactic_digest,
        "deployment_features": {"ptx": False, "jit": False, "autotune": False,
                                "runtime_weight_repacking": False, "cpu_fallback": False},
    }
    return AimWriter.write(options.output, platform=options.platform, manifest=manifest, graph=graph,
                           tensors={"alignment": 256, "count": len(table), "items": table}, variants=variants)


def plan_artifacts(args) -> dict[str, Any]:
    """``modelc plan``: checkpoint directory + adapter + shape profile -> ``<artifact-dir>/toolchain.json`` and
    ``<artifact-dir>/sm100/{kernels.cubin,plan.json,tactics.json}``, ready for ``modelc compile``.  The role the
    reference leaves to whoever fills ``--artifact-dir`` (``src/aginfer/compiler.py:61-75``), driven by the
    adapter's graph description (``src/aginfer/adapters/groot.py:13-29``)."""
    from .recipes import lowering
    if args.cuda_arch != CudaArch.SM100:
        raise ValidationError("modelc plan generates sm100 recipes only")
    profile = load_profile(args.profile)
    source = args.source
    if args.pack_checkpoint:
        source = str(_pack_checkpoint(Path(args.source), args.pack_checkpoint))
    checkpoint = load_checkpoint(source, None, args.offline)
    _, graph = describe_model(args.adapter, checkpoint)
    tensors = list(checkpoint.tensors)
    if args.backbone:
        taken = {t.name for t in tensors}
        tensors += [replace(t, name=f"backbone.{t.name}") if t.name in taken else t
                    for t in load_checkpoint(args.backbone, None, args.offline).tensors]
    inventory = {t.name: (t.dtype, tuple(t.shape)) for t in tensors}
    steps = tuple(int(v) for v in args.step_profiles.split(",") if v.strip())
    recipe, name, shape = lowering.lower(args.adapter, graph, inventory, checkpoint.config, profile,
                                         packed=bool(args.packed or args.pack_checkpoint), step_profiles=steps,
                                         heads=args.heads)
    lowering.write_artifact_dir(args.artifact_dir, recipe)
    plan = recipe.plan()
    return {"artifact_dir": str(args.artifact_dir), "recipe": name, "source": source, "shape": shape,
            "profiles": {p["profile"]: len(p["launches"]) for p in plan["shape_dispatch"]},
            "arena_bytes": plan["arena_bytes"], "weight_bytes": recipe.weight_bytes,
            "graph_passes": list(graph["passes"])}


def _pack_checkpoint(source: Path, target: Path) -> Path:
    """The packaging-time layout pass for FP8 prefill recipes: every E4M3 ``[N, K]`` linear weight rewritten into
    the packed tile layout of ``recipes/layout.py`` (same names; shape [K / 128, N padded to 256, 128]); everything else copied."""
    import shutil

    import torch

    from .recipes import qwen_vl
    from .recipes.package import tensor_record
    from .weights import write_safetensors
    checkpoint = load_checkpoint(str(source), None, True)
    target.mkdir(parents=True, exist_ok=True)
    for path in sorted(Path(source).iterdir()):
        if path.is_file() and path.suffix != ".safetensors":
            shutil.copy(path, target / path.name)
    dtypes = {"F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F8_E4M3": torch.float8_e4m3fn}
    by_file: dict[Path, dict[str, Any]] = {}
    for record in checkpoint.tensors:
        with open(record.source, "rb") as handle:
            handle.seek(record.source_offset)
            data = torch.frombuffer(bytearray(handle.read(record.byte_length)), dtype=torch.uint8)
        by_file.setdefault(record.source, {})[record.name] = data.view(dtypes[record.dtype]).reshape(record.shape)
    for path, tensors in by_file.items():
        packed = qwen_vl.pack_checkpoint(tensors)
        write_safetensors(target / path.name, {k: tensor_record(v) for k, v in packed.items()})
    return target


def _typed(parser):
    def convert(text: str):
        try:
            return parser(text)
        except ValueError as exc:
            raise argparse.ArgumentTypeError(str(exc)) from exc
    return convert


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="modelc", description="AgInfer target-specific AIM compiler")
    parser.add_argument("--version", action="version", version="modelc 0.1.0 (AIM schema 1.0, ABI 1)")
    sub = parser.add_subparsers(dest="command", required=True)
    c = sub.add_parser("compile", help="validate a checkpoint and build a target-specific AIM")
    c.add_argument("--source", required=True)
    c.add_argument("--revision")
    c.add_argument("--adapter", required=True, choices=adapter_names())
    c.add_argument("--platform", required=True, type=_typed(Platform.parse))
    c.add_argument("--cuda-arch", required=True, action="append", type=_typed(CudaArch.parse), dest="cuda_arches")
    c.add_argument("--profile", required=True, type=Path)
    c.add_argument("--artifact-dir", required=True, type=Path,
                   help="verified AOT outputs: toolchain.json and <arch>/{kernels.cubin,plan.json,tactics.json}")
    c.add_argument("--backbone", help="local Qwen2.5-VL checkpoint required by lingbot_vla_1")
    c.add_argument("--offline", action="store_true")
    c.add_argument("--output", required=True, type=Path)
    g = sub.add_parser("plan", help="write the sm100 artifact directory (kernel bundle, plan.json, tactics.json, "
                                    "toolchain.json) for a checkpoint: the adapter's graph passes lowered to a launch recipe")
    g.add_argument("--source", required=True)
    g.add_argument("--adapter", required=True, choices=adapter_names())
    g.add_argument("--profile", required=True, type=Path)
    g.add_argument("--cuda-arch", required=True, type=_typed(CudaArch.parse), dest="cuda_arch")
    g.add_argument("--artifact-dir", required=True, type=Path)
    g.add_argument("--backbone", help="local Qwen2.5-VL checkpoint whose tensors join the blob (lingbot_vla_1)")
    g.add_argument("--packed", action="store_true",
                   help="FP8 linear weights are in the packed tile layout (see --pack-checkpoint)")
    g.add_argument("--pack-checkpoint", type=Path, metavar="DIR",
                   help="first rewrite the checkpoint's FP8 linear weights into the packed tile layout under DIR "
                        "(same tensor names) and plan for that copy; implies --packed")
    g.add_argument("--step-profiles", default="", help="comma-separated extra Euler step counts to package as "
                                                       "sibling profiles <profile>/steps=<n>")
    g.add_argument("--heads", type=int, help="attention heads of the action head when config.json does not say")
    g.add_argument("--offline", action="store_true")
    i = sub.add_parser("inspect", help="verify and display an AIM manifest")
    i.add_argument("aim", type=Path)
    i.add_argument("--no-payload-checksums", action="store_true")
    return parser


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    try:
        if args.command == "compile":
            info = compile_model(CompileOptions(
                source=args.source, revision=args.revision, adapter=args.adapter, platform=args.platform,
                cuda_arches=tuple(args.cuda_arches), profile_path=args.profile, artifact_dir=args.artifact_dir,
                output=args.output, offline=args.offline, backbone=args.backbone))
            print(f"wrote {info.path} ({info.file_size} bytes, sha256={info.file_sha256})")
            return 0
        if args.command == "plan":
            print(json.dumps(plan_artifacts(args), sort_keys=True))
            return 0
        info = AimReader.read(args.aim, verify_payloads=not args.no_payload_checksums)
        print(json.dumps({
            "path": str(info.path), "schema": f"{info.schema_major}.{info.schema_minor}",
            "runtime_abi": info.runtime_abi, "platform": info.platform.triple,
            "cuda_arches": [v.arch.name_string for v in info.variants], "file_size": info.file_size,
            "file_sha256": info.file_sha256, "manifest": info.manifest, "graph": info.graph,
            "tensor_count": info.tensors.get("count"),
        }, indent=2, ensure_ascii=False, sort_keys=True))
        return 0
    except (AgInferError, ValueError) as exc:
        print(f"modelc: error: {exc}", file=sys.stderr)
        return 2


if __name__ == "__main__":
    raise SystemExit(main())

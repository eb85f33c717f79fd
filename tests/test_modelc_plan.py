"""``modelc plan``: from a checkpoint directory to the sm100 artifact set on the command line, then
``modelc compile`` and a load through the C ABI, with no Python API call in between.

Reference: the adapters name graph passes and subgraphs but lower nothing (``src/aginfer/adapters/groot.py:13-29``),
and ``modelc compile`` expects a filled artifact directory (``src/aginfer/compiler.py:61-75``).
"""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest

from aginfer_b200 import runtime as rt
from aginfer_b200.recipes import dit
from aginfer_b200.recipes.package import write_checkpoint, write_profile
from tests.test_dit_cpu import TINY

ROOT = Path(__file__).resolve().parent.parent
OVERRIDES = dict(cuda_driver_version_override=12080, cuda_runtime_version_override=12080, cublaslt_abi_override=12,
                 cudnn_abi_override=9)


def modelc(*args: str) -> subprocess.CompletedProcess:
    return subprocess.run([sys.executable, "-m", "aginfer_b200.modelc", *args], cwd=ROOT, capture_output=True, text=True)


@pytest.mark.parametrize("described", [True, False])
def test_checkpoint_to_plan_to_aim_on_the_command_line(tmp_path, described):
    # `described`: config.json carries the shape; otherwise it is read off the tensor shapes and the profile
    ckpt = write_checkpoint(tmp_path / "ckpt", dit.synthetic_weights(TINY), "groot", recipe=("dit", TINY) if described else None)
    profile = write_profile(tmp_path / "profile.json", steps=TINY.steps, action_horizon=TINY.horizon,
                            state_length=TINY.state_dim, sequence_length=TINY.backbone_tokens)
    artifacts = tmp_path / "artifacts"
    done = modelc("plan", "--source", str(ckpt), "--adapter", "groot_n1_5", "--profile", str(profile), "--cuda-arch", "sm100a",
                  "--artifact-dir", str(artifacts), "--step-profiles", "1,4", "--heads", str(TINY.heads), "--offline")
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    assert report["recipe"] == "dit" and report["shape"]["hidden"] == TINY.hidden and report["shape"]["mlp"] == TINY.mlp
    assert report["shape"] == json.loads(json.dumps(__import__("dataclasses").asdict(TINY)))
    assert set(report["profiles"]) == {"default", "default/steps=1", "default/steps=4"}
    assert "fuse_qkv" in report["graph_passes"]
    for name in ("toolchain.json", "sm100/kernels.cubin", "sm100/plan.json", "sm100/tactics.json"):
        assert (artifacts / name).is_file()
    # the written plan is the one the Python API generates for the same shape
    want = dit.build_recipe(TINY, step_profiles=(1, 4)).plan()
    assert json.loads((artifacts / "sm100/plan.json").read_text()) == json.loads(json.dumps(want))
    tactics = json.loads((artifacts / "sm100/tactics.json").read_text())["tactics"]
    lowered = {t["algorithm"]: t["lowered_to"] for t in tactics if t["op"] == "graph_pass"}
    assert {"fuse_qkv", "fuse_mlp", "fuse_norm"} <= set(lowered) and "one launch" in lowered["fuse_qkv"]
    assert any(t["op"] == "recipe" and t["algorithm"] == "dit" and t["adapter"] == "groot_n1_5" for t in tactics)

    aim = tmp_path / "model.aim"
    done = modelc("compile", "--source", str(ckpt), "--adapter", "groot_n1_5", "--platform", "linux-x86_64-gnu",
                  "--cuda-arch", "sm100a", "--profile", str(profile), "--artifact-dir", str(artifacts), "--offline",
                  "--output", str(aim))
    assert done.returncode == 0, done.stderr
    session = rt.Session.create(rt.Runtime.create(cuda_arch_override=100, **OVERRIDES), rt.Model.load(aim), "default/steps=1")
    assert [t.name for t in session.input_info()] == ["backbone_features", "state", "noise"]
    assert [t.name for t in session.output_info()] == ["actions", "status"]


def test_plan_refuses_what_it_cannot_lower(tmp_path):
    ckpt = write_checkpoint(tmp_path / "ckpt", {"something.else": dit.synthetic_weights(TINY)["action_head.position_embedding.weight"]})
    profile = write_profile(tmp_path / "profile.json")
    done = modelc("plan", "--source", str(ckpt), "--adapter", "groot_n1_5", "--profile", str(profile), "--cuda-arch", "sm100a",
                  "--artifact-dir", str(tmp_path / "a"), "--offline")
    assert done.returncode == 2 and "no sm100 recipe generator" in done.stderr
    done = modelc("plan", "--source", str(ckpt), "--adapter", "groot_n1_5", "--profile", str(profile), "--cuda-arch", "sm120",
                  "--artifact-dir", str(tmp_path / "a"), "--offline")
    assert done.returncode == 2 and "sm100 recipes only" in done.stderr


def test_plan_packs_an_fp8_checkpoint_and_plans_the_prefill(tmp_path):
    # the packaging-time layout pass as a modelc flag: FP8 linear weights rewritten into the packed tile layout
    # (same names), the prefill recipe planned for that copy with bulk-copy GEMM producers
    import torch

    from aginfer_b200.recipes import qwen_vl
    from aginfer_b200.weights import load_checkpoint
    cfg = qwen_vl.VlConfig(v_layers=1, v_full_layers=(0,), layers=1, vocab=256)
    weights = qwen_vl.synthetic_weights(cfg)
    ckpt = write_checkpoint(tmp_path / "ckpt", weights, "qwen2_5_vl", recipe=("qwen_vl_prefill", cfg))
    profile = write_profile(tmp_path / "profile.json", sequence_length=cfg.tokens)
    done = modelc("plan", "--source", str(ckpt), "--adapter", "lingbot_vla_1", "--profile", str(profile), "--cuda-arch",
                  "sm100a", "--artifact-dir", str(tmp_path / "artifacts"), "--pack-checkpoint", str(tmp_path / "packed"),
                  "--offline")
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    assert report["recipe"] == "qwen_vl_prefill" and report["source"] == str(tmp_path / "packed")
    plan = json.loads((tmp_path / "artifacts/sm100/plan.json").read_text())
    assert any(l["kernel"].startswith("agi_gemm_tcp") or l["kernel"].startswith("agi_gemm_tcq")
               for l in plan["shape_dispatch"][0]["launches"])
    # the packed copy holds the same tensors, byte for byte what the Python layout pass produces
    want = qwen_vl.pack_checkpoint(weights)
    got = {t.name: t for t in load_checkpoint(str(tmp_path / "packed"), None, True).tensors}
    assert set(got) == set(want)
    name = next(k for k, v in want.items() if v.dtype == torch.float8_e4m3fn and v.dim() == 3)   # a packed linear weight
    record = got[name]
    with open(record.source, "rb") as handle:
        handle.seek(record.source_offset)
        assert handle.read(record.byte_length) == want[name].contiguous().view(torch.uint8).numpy().tobytes()

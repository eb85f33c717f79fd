"""The boundary, checked against the reference's own code.

Two directions:

* the reference's caller-side tests (``tests/runtime_test.cc``, ``tests/cuda_runtime_test.cc``), compiled
  UNMODIFIED against this repository's library through ``include/aginfer_b200_compat.hpp`` (the C++ surface of
  ``include/aginfer/runtime.h:120-176`` over the C ABI), must pass;
* the reference's C++ runtime, carrying only ``oracle/ref_sm100.patch`` (target row, new CUBIN ELF flavour,
  shared-memory opt-in), must load one of this repository's sm100 packages and produce, through its own
  ``Session::Enqueue`` launch loop (``cpp/runtime.cc:333-355``), exactly the bytes this repository's loader
  produces.

The executables are built where the reference checkout is available (``make -C oracle sm100``, also run by
``__graft_entry__.build()``) into ``oracle/_ref_sm100/``; the tests skip where they are missing.
"""
from __future__ import annotations

import json
import subprocess
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
BUILT = ROOT / "oracle" / "_ref_sm100"
GOLDEN = json.loads((ROOT / "tests" / "golden" / "format_golden.json").read_text())


def need(name: str) -> Path:
    path = BUILT / name
    if not path.exists():
        pytest.skip(f"{path} is not built (needs the reference checkout: make -C oracle sm100)")
    return path


def test_reference_runtime_test_passes_against_this_library(tmp_path):
    # the reference's CPU-only integration test on the reference's own fixture package (sm89, all probes overridden)
    fixture = tmp_path / "test.aim"
    fixture.write_bytes(bytes.fromhex(GOLDEN["runtime_fixture_hex"]))
    done = subprocess.run([str(need("runtime_test_compat")), str(fixture)], capture_output=True, text=True, timeout=60)
    assert done.returncode == 0, (done.returncode, done.stderr)


@pytest.mark.gpu
def test_reference_cuda_runtime_test_passes_against_this_library(tmp_path):
    # the reference's real-GPU test: one vector_add launch through Session::Enqueue, then a shape it must refuse.
    # Its fixture (tests/make_cuda_fixture.py in the reference) is an sm89 package; this is the same package for
    # sm100, from this repository's packager and kernel bundle.
    from aginfer_b200.recipes import RecipeBuilder, Tensor, io
    from aginfer_b200.recipes.package import build_aim, describe
    weights = {"unused.pad": torch.zeros(8, dtype=torch.bfloat16)}
    recipe = RecipeBuilder(describe(weights))
    recipe.begin_profile("vector16", [io("left", "F32", [16]), io("right", "F32", [16])], [io("output", "F32", [16])])
    recipe.vector_add(Tensor("left"), Tensor("right"), Tensor("output"), 16)
    aim = build_aim(tmp_path, weights, recipe)
    done = subprocess.run([str(need("cuda_runtime_test_compat")), str(aim)], capture_output=True, text=True, timeout=120)
    assert done.returncode == 0, (done.returncode, done.stderr)


RAW_DTYPE = {"F32": (0, torch.float32), "F16": (1, torch.float16), "BF16": (2, torch.bfloat16), "I32": (4, torch.int32)}


@pytest.mark.gpu
def test_patched_reference_runtime_runs_the_action_head_package(tmp_path):
    # BASELINE config 3 (16 blocks x 1536, 4 Euler steps) through the reference's own launch loop
    from aginfer_b200 import runtime as rt
    from aginfer_b200.recipes import dit
    from aginfer_b200.recipes.package import build_aim
    from aginfer_b200.runner import Runner
    probe = need("ref_probe_gpu")
    cfg = dit.DitConfig()
    weights, inputs = dit.synthetic_weights(cfg, seed=2), dit.synthetic_inputs(cfg, seed=2)
    aim = build_aim(tmp_path, weights, dit.build_recipe(cfg), steps=cfg.steps, action_horizon=cfg.horizon,
                    state_length=cfg.state_dim)

    ours = Runner(aim, flags=rt.NO_GRAPH_REPLAY)          # plain launches, like the reference's loop
    out = ours.empty_outputs()
    ours.run({k: v.cuda() for k, v in inputs.items()}, out)
    torch.cuda.synchronize()
    assert int(out["status"].item()) == 0

    lines = []
    for info in ours.inputs:
        path = tmp_path / f"in_{info.name}.bin"
        path.write_bytes(inputs[info.name].contiguous().view(torch.uint8).numpy().tobytes())
        lines.append(f"in {info.name} {RAW_DTYPE[info.dtype][0]} {path} " + " ".join(map(str, info.shape)))
    for info in ours.outputs:
        lines.append(f"out {info.name} {RAW_DTYPE[info.dtype][0]} {tmp_path / ('out_' + info.name + '.bin')} "
                     + " ".join(map(str, info.shape)))
    manifest = tmp_path / "manifest.txt"
    manifest.write_text("\n".join(lines) + "\n")
    done = subprocess.run([str(probe), str(aim), "default", str(manifest), "20"], capture_output=True, text=True, timeout=300)
    report = dict(line.split("=", 1) for line in done.stdout.splitlines() if "=" in line)
    assert done.returncode == 0 and report.get("enqueue") == "OK|" and report.get("device") == "cudaSuccess", (done, report)
    print(f"reference launch loop (patched reference runtime): {float(report['ms_per_enqueue']):.3f} ms per action chunk")
    for info in ours.outputs:
        raw = (tmp_path / f"out_{info.name}.bin").read_bytes()
        theirs = torch.frombuffer(bytearray(raw), dtype=RAW_DTYPE[info.dtype][1]).reshape(info.shape)
        assert torch.equal(theirs, out[info.name].cpu()), f"{info.name} differs between the two loaders"

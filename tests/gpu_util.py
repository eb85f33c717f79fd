"""Helpers for the GPU parity tests: package a one-profile recipe and run it through the C ABI."""
from __future__ import annotations

from pathlib import Path

import torch

from aginfer_b200.recipes import RecipeBuilder
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner

MAX_REL = 2e-2   # tolerance of the bf16 tier: max |got - want| / max |want|
PLAN_DTYPE = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32",
              torch.float8_e4m3fn: "F8_E4M3", torch.uint8: "F8_E4M3"}


def spec(name: str, t: torch.Tensor) -> dict:
    return {"name": name, "dtype": PLAN_DTYPE[t.dtype], "shape": list(t.shape)}


def run_recipe(tmp: Path, weights: dict, inputs: dict, outputs: dict, body, flags: int = 0, repeats: int = 1):
    """``body(recipe)`` emits launches between begin_profile and packaging.  ``inputs`` are CPU tensors,
    ``outputs`` maps name -> (dtype, shape).  Returns the outputs as CPU tensors and the session stats."""
    weights = dict(weights) or {"unused.pad": torch.zeros(8, dtype=torch.bfloat16)}
    recipe = RecipeBuilder(describe(weights))
    out_specs = [{"name": n, "dtype": PLAN_DTYPE[d], "shape": list(s)} for n, (d, s) in outputs.items()]
    recipe.begin_profile("default", [spec(n, t) for n, t in inputs.items()], out_specs)
    body(recipe)
    aim = build_aim(tmp, weights, recipe)
    runner = Runner(aim, flags=flags)
    dev_in = {n: (t.view(torch.uint8) if t.dtype == torch.float8_e4m3fn else t).cuda() for n, t in inputs.items()}
    dev_out = {n: torch.zeros(s, dtype=torch.uint8 if d in (torch.float8_e4m3fn, torch.uint8) else d, device="cuda")
               for n, (d, s) in outputs.items()}
    for _ in range(repeats):
        runner.run(dev_in, dev_out)
    torch.cuda.synchronize()
    got = {}
    for n, (d, s) in outputs.items():
        t = dev_out[n].cpu()
        got[n] = t.view(torch.float8_e4m3fn) if d == torch.float8_e4m3fn else t
    return got, runner.stats()

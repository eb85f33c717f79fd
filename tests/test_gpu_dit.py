"""The flow-matching DiT action head end to end on the GPU against the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from aginfer_b200 import runtime as rt
from aginfer_b200.recipes import dit
from aginfer_b200.recipes.package import build_aim
from aginfer_b200.runner import Runner
from oracle import dit as oracle_dit
from oracle import ops
from tests.test_dit_cpu import TINY

pytestmark = pytest.mark.gpu


def run_chunk(tmp_path, cfg, weights, inputs, gemm_tactic="auto", repeats=2, block_kernel=None, flags=0, packed=False):
    inventory = None
    if packed:      # the packaging-time layout pass; the recipe sees the packed shapes and picks the kernels for them
        from aginfer_b200.recipes.package import describe
        weights = dit.pack_checkpoint(cfg, weights)
        inventory = describe(weights)
    recipe = dit.build_recipe(cfg, inventory, gemm_tactic=gemm_tactic, block_kernel=block_kernel)
    aim = build_aim(tmp_path, weights, recipe, steps=cfg.steps, action_horizon=cfg.horizon, state_length=cfg.state_dim)
    runner = Runner(aim, flags=flags)
    dev = {k: v.cuda() for k, v in inputs.items()}
    out = runner.empty_outputs()
    for _ in range(repeats):
        runner.run(dev, out)
    torch.cuda.synchronize()
    assert int(out["status"].item()) == 0, f"a bounded wait ran out: status {int(out['status'].item()):#x}"
    return out["actions"].cpu(), runner.stats()


@pytest.mark.parametrize("tactic,block_kernel", [("simt", False), ("auto", False), ("auto", True)])
def test_tiny_dit_matches_oracle(tmp_path, tactic, block_kernel):
    w, x = dit.synthetic_weights(TINY), dit.synthetic_inputs(TINY)
    got, stats = run_chunk(tmp_path, TINY, w, x, tactic, block_kernel=block_kernel)
    want = oracle_dit.forward(TINY, w, x["backbone_features"], x["state"], x["noise"])
    assert ops.cosine(got, want) >= 0.999
    assert ops.max_rel_err(got, want) < 2e-2
    assert stats["graph_launches"] == 2 and stats["graphs_built"] == 1


@pytest.mark.parametrize("flags", [rt.NO_GRAPH_REPLAY, rt.NO_GRAPH_REPLAY | rt.NO_COOPERATIVE_LAUNCH, rt.PROGRAMMATIC_LAUNCH])
def test_tiny_dit_block_kernel_launch_modes(tmp_path, flags):
    # plain launches with and without the cooperative attribute, and graph replay with programmatic edges
    w, x = dit.synthetic_weights(TINY), dit.synthetic_inputs(TINY)
    got, _ = run_chunk(tmp_path, TINY, w, x, block_kernel=True, flags=flags)
    base, _ = run_chunk(tmp_path / "base", TINY, w, x, block_kernel=True)
    assert torch.equal(got, base)


@pytest.mark.parametrize("block_kernel,packed", [(False, False), (True, False), (False, True)],
                         ids=["launch_per_op", "block_kernel", "packed_weights"])
def test_full_size_action_chunk_matches_oracle(tmp_path, block_kernel, packed):
    # BASELINE config 3: 16 blocks x 1536, 17 tokens, 300 backbone tokens, 4 Euler steps, seed 2
    cfg = dit.DitConfig()
    w, x = dit.synthetic_weights(cfg, seed=2), dit.synthetic_inputs(cfg, seed=2)
    got, stats = run_chunk(tmp_path, cfg, w, x, block_kernel=block_kernel, packed=packed)
    want = oracle_dit.forward(cfg, w, x["backbone_features"], x["state"], x["noise"])
    cos, err = ops.cosine(got, want), ops.max_rel_err(got, want)
    print(f"full DiT (block kernel {block_kernel}, packed {packed}): cosine={cos:.6f} max_rel_err={err:.3e} "
          f"launches/chunk={stats['launches_per_enqueue']}")
    assert cos >= 0.999 and err < 2e-2
    # a fresh session reproduces the chunk bit for bit: partial sums are added in a fixed order
    again, _ = run_chunk(tmp_path / "again", cfg, w, x, repeats=1, block_kernel=block_kernel, packed=packed)
    assert torch.equal(again, got)


def test_run_options_pick_the_step_count_and_the_noise(tmp_path):
    # reference: RunOptions.denoising_steps / initial_noise_override (include/aginfer/runtime.h:84-90)
    from dataclasses import replace
    cfg = TINY
    w, x = dit.synthetic_weights(cfg), dit.synthetic_inputs(cfg)
    recipe = dit.build_recipe(cfg, step_profiles=(1, 4))
    aim = build_aim(tmp_path, w, recipe, steps=cfg.steps, action_horizon=cfg.horizon, state_length=cfg.state_dim)
    runner = Runner(aim)
    dev = {k: v.cuda() for k, v in x.items()}
    out = runner.empty_outputs()
    other_noise = torch.randn(cfg.horizon, cfg.action_dim, generator=torch.Generator().manual_seed(99)).to(torch.bfloat16)
    for steps, noise in ((0, None), (1, None), (4, None), (4, other_noise), (0, other_noise)):
        runner.run(dev, out, denoising_steps=steps, noise_override=None if noise is None else noise.cuda())
        torch.cuda.synchronize()
        assert int(out["status"].item()) == 0
        want = oracle_dit.forward(replace(cfg, steps=steps or cfg.steps), w, x["backbone_features"], x["state"],
                                  x["noise"] if noise is None else noise)
        got = out["actions"].cpu()
        assert ops.cosine(got, want) >= 0.999 and ops.max_rel_err(got, want) < 2e-2, (steps, noise is not None)
    # each step count keeps its own graph; a count the package does not carry is refused, not approximated
    assert runner.stats()["graphs_built"] >= 3
    with pytest.raises(rt.RuntimeStatusError, match="no recipe for 3 denoising steps"):
        runner.run(dev, out, denoising_steps=3)

"""One decoder layer (BASELINE config 1) and its FP8 form, end to end on the GPU against the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from aginfer_b200.recipes import decoder_layer as layer
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner
from oracle import decoder_layer as oracle_layer
from oracle import ops

pytestmark = pytest.mark.gpu


def run_layer(tmp_path, cfg, weights, hidden, tactic="auto"):
    recipe = layer.build_recipe(cfg, describe(weights), gemm_tactic=tactic)
    aim = build_aim(tmp_path, weights, recipe, sequence_length=cfg.tokens)
    runner = Runner(aim)
    out = runner.empty_outputs()
    for _ in range(2):
        runner.run({"hidden_in": hidden.cuda()}, out)
    torch.cuda.synchronize()
    return out["hidden_out"].cpu(), runner.stats()


@pytest.mark.parametrize("fp8", [False, True], ids=["bf16", "fp8"])
def test_decoder_layer_matches_oracle(tmp_path, fp8):
    # hidden 2048, 16/2 heads x 128, SwiGLU 11008, 288 tokens, seed 0
    cfg = layer.LayerConfig(fp8=fp8)
    w, x = layer.synthetic_weights(cfg, seed=0), layer.synthetic_input(cfg, seed=0)
    got, stats = run_layer(tmp_path, cfg, w, x)
    want = oracle_layer.forward(cfg, w, x)
    err, cos = ops.max_rel_err(got, want), ops.cosine(got, want)
    print(f"decoder layer fp8={fp8}: max_rel_err={err:.3e} cosine={cos:.6f} launches={stats['launches_per_enqueue']}")
    # BF16: 2e-2.  FP8: four per-tensor dynamic quantisations in the block put the oracle's own resolution at
    # 3-4% of the output range (ops.FP8_BLOCK_TOL)
    assert err < (ops.FP8_BLOCK_TOL if fp8 else 2e-2) and cos > 0.999


def test_small_ragged_layer_with_the_audit_gemm(tmp_path):
    # 70 tokens, odd sizes: exercises tile tails; the CUDA-core GEMM tactic cross-checks the tensor-core one
    cfg = layer.LayerConfig(hidden=256, heads=4, kv_heads=2, head_dim=64, intermediate=704, tokens=70)
    w, x = layer.synthetic_weights(cfg, seed=5), layer.synthetic_input(cfg, seed=5)
    want = oracle_layer.forward(cfg, w, x)
    for tactic in ("simt", "auto"):
        got, _ = run_layer(tmp_path / tactic, cfg, w, x, tactic)
        assert ops.max_rel_err(got, want) < 2e-2, tactic

"""LingBot-VLA-shaped episode (BASELINE config 5): recipe construction and oracle plumbing on CPU."""
from __future__ import annotations

import collections
import dataclasses

import torch

from aginfer_b200 import planfmt
from aginfer_b200.recipes import lingbot, qwen_vl
from aginfer_b200.recipes.package import describe
from aginfer_b200.target import CudaArch
from oracle import lingbot as oracle_lingbot
from tests.test_qwen_vl_cpu import table as backbone_table

TINY_BACKBONE = dataclasses.replace(lingbot.BACKBONE_7B, v_layers=1, v_full_layers=(0,), layers=2, vocab=256)
TINY = lingbot.EpisodeConfig(backbone=TINY_BACKBONE, e_layers=2, steps=2)


def table(cfg):
    t = backbone_table(cfg.backbone)
    t.update({k: ("BF16", v) for k, v in lingbot.expert_shapes(cfg).items()})
    return t


def test_full_size_episode_compiles_to_a_plan():
    cfg = lingbot.EpisodeConfig()
    assert (cfg.backbone.tokens, cfg.backbone.patches, cfg.e_kv_dim, cfg.first_action_position()) == (256, 768, 512, 88)
    recipe = lingbot.build_recipe(cfg, table(cfg))
    launches = recipe.plan()["shape_dispatch"][0]["launches"]
    kinds = collections.Counter(l["kernel"] for l in launches)
    assert kinds["agi_euler_step"] == cfg.steps
    assert kinds["agi_attention_fa_amax_bf16_d128"] == 28          # backbone: feeds an FP8 quantisation
    assert kinds["agi_attention_mma_bf16_d128"] == 18 * 10         # expert: 50 query rows, keys split over warps
    # the expert's projections that share an input share a launch: Q | K | V (cluster of 8) and gate | up (of 2)
    assert kinds["agi_gemm_tc_bf16_x3_c8"] == 18 * 10 and kinds["agi_gemm_tc_bf16_x3_c2"] == 18 * 10
    compiled = planfmt.compile_execution_plan(recipe.plan(), CudaArch.SM100, weight_size=recipe.weight_bytes)
    assert compiled.input_names == ("pixels", "input_ids", "positions", "state", "noise")
    assert "actions" in compiled.output_names
    alg = lingbot.algorithmic(cfg)
    assert abs(alg["backbone_fp8_weight_bytes"] / 7.20e9 - 1) < 0.01 and abs(alg["expert_params"] / 283e6 - 1) < 0.01
    assert abs(alg["expert_weight_bytes_per_episode"] / 5.66e9 - 1) < 0.01


def test_tiny_oracle_episode_runs():
    w, x = lingbot.synthetic_weights(TINY), lingbot.synthetic_inputs(TINY)
    assert {k: (d, tuple(s)) for k, (d, s) in describe(w).items()} == table(TINY)
    actions, hidden, cache = oracle_lingbot.forward(TINY, w, x["pixels"], x["input_ids"], x["positions"], x["state"], x["noise"])
    assert actions.shape == (50, 14) and actions.dtype == torch.float32 and torch.isfinite(actions).all()
    assert cache.shape == (2, 2, 256, 512)
    # the velocity field is not degenerate: ten steps move the latent away from the noise
    assert (actions - x["noise"].float()).abs().max() > 1e-3
    # padding columns of the 14-wide vectors are inert
    assert w["expert.action_in.weight"][:, 14:].abs().max() == 0 and w["expert.action_out.weight"][14:].abs().max() == 0

"""LingBot-VLA-shaped episode (BASELINE config 5) on the GPU against the CPU oracle."""
from __future__ import annotations

import dataclasses

import pytest
import torch

from aginfer_b200.recipes import lingbot
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner
from oracle import lingbot as oracle_lingbot
from oracle import ops

pytestmark = pytest.mark.gpu


def test_reduced_depth_episode_matches_oracle(tmp_path):
    """Real widths (3584 backbone, 1024 expert, 256 + 50 tokens); 2 vision blocks, 3 decoder layers, 4 expert
    layers, 3 Euler steps.  The expert is BF16, so given the same K/V cache it is held to the action-chunk tier
    (cosine >= 0.999, max-rel <= 2e-2): the oracle's expert is fed the cache the GPU exported.  The FP8 prefill
    itself is covered block by block in test_gpu_qwen_vl.py; here its cache is only checked end to end against
    the oracle's (cosine; FP8 rounding differences accumulate over the blocks in front of it)."""
    backbone = dataclasses.replace(lingbot.BACKBONE_7B, v_layers=2, v_full_layers=(1,), layers=3, vocab=2048)
    cfg = lingbot.EpisodeConfig(backbone=backbone, e_layers=4, steps=3)
    w, x = lingbot.synthetic_weights(cfg), lingbot.synthetic_inputs(cfg)
    aim = build_aim(tmp_path, w, lingbot.build_recipe(cfg, describe(w)))
    runner = Runner(aim)
    dev = {k: v.cuda() for k, v in x.items()}
    out = runner.empty_outputs()
    for _ in range(2):
        runner.run(dev, out)
    torch.cuda.synchronize()
    got = {k: v.cpu() for k, v in out.items()}
    assert got["status"].item() == 0
    want = oracle_lingbot.action_expert(cfg, w, got["kv_cache"], x["state"], x["noise"])
    cos, err = ops.cosine(got["actions"], want), ops.max_rel_err(got["actions"], want)
    _, _, want_cache = oracle_lingbot.forward(cfg, w, x["pixels"], x["input_ids"], x["positions"], x["state"], x["noise"])
    cache_cos = ops.cosine(got["kv_cache"], want_cache)
    print(f"episode: actions cosine={cos:.6f} max_rel_err={err:.3e}; K/V cache cosine={cache_cos:.5f}; "
          f"launches={runner.stats()['launches_per_enqueue']}")
    assert cos >= 0.999 and err < 2e-2
    assert cache_cos >= 0.99
    stats = runner.stats()
    assert stats["graph_launches"] == 2 and stats["graphs_built"] == 1


def test_full_depth_episode_matches_oracle(tmp_path):
    """BASELINE config 5 as it stands: 32 vision blocks, 28 decoder layers x 3584, 18 expert layers, 10 Euler steps
    (only the vocabulary is cut, which shortens set-up and touches no arithmetic), packed FP8 operands as in the
    benchmark.

    The claim for the action chunk (cosine >= 0.999, max-rel <= 2e-2) is made for the BF16 expert given the same
    K/V cache: the oracle's expert is fed the cache the GPU exported.  Free-running, the oracle's own FP8 prefill
    produces a cache that differs from the GPU's by the arithmetic's noise floor (per-tensor dynamic scales turn a
    last-bit difference into a few percent of a block's output; the prefill is covered block by block, and with
    teacher-forced operands at 2e-2, in test_gpu_qwen_vl.py), so the free-running action chunk is reported and
    held to a looser bound."""
    from aginfer_b200.recipes import qwen_vl
    backbone = dataclasses.replace(lingbot.BACKBONE_7B, vocab=4096)
    cfg = lingbot.EpisodeConfig(backbone=backbone)
    w, x = lingbot.synthetic_weights(cfg), lingbot.synthetic_inputs(cfg)
    packed = qwen_vl.pack_checkpoint(w)
    aim = build_aim(tmp_path, packed, lingbot.build_recipe(cfg, describe(packed), packed=True))
    del packed
    runner = Runner(aim)
    dev = {k: v.cuda() for k, v in x.items()}
    out = runner.empty_outputs()
    for _ in range(2):
        runner.run(dev, out)
    torch.cuda.synchronize()
    got = {k: v.cpu() for k, v in out.items()}
    assert got["status"].item() == 0
    want = oracle_lingbot.action_expert(cfg, w, got["kv_cache"], x["state"], x["noise"])
    cos, err = ops.cosine(got["actions"], want), ops.max_rel_err(got["actions"], want)
    free_actions, _, free_cache = oracle_lingbot.forward(cfg, w, x["pixels"], x["input_ids"], x["positions"], x["state"],
                                                         x["noise"])
    free_cos, cache_cos = ops.cosine(got["actions"], free_actions), ops.cosine(got["kv_cache"], free_cache)
    print(f"full-depth episode: actions given the same cache cosine={cos:.6f} max_rel_err={err:.3e}; free-running "
          f"actions cosine={free_cos:.5f}, K/V cache cosine={cache_cos:.5f}; launches={runner.stats()['launches_per_enqueue']}")
    assert cos >= 0.999 and err < 2e-2
    assert cache_cos >= 0.95 and free_cos >= 0.995      # measured: 0.9823 and 0.9996

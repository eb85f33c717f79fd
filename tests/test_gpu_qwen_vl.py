"""Qwen2.5-VL-shaped FP8 prefill (BASELINE config 4) on the GPU against the CPU oracle."""
from __future__ import annotations

import pytest
import torch

from aginfer_b200.recipes import Tensor, U32, qwen_vl
from aginfer_b200.recipes.builder import grid_for
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner
from oracle import ops
from oracle import qwen_vl as oracle_vl
from tests.gpu_util import run_recipe

pytestmark = pytest.mark.gpu


def test_patchify_and_unwindow_are_bit_exact(tmp_path):
    cfg = qwen_vl.VlConfig()
    pixels = qwen_vl.synthetic_inputs(cfg)["pixels"]
    merged = torch.randn(cfg.merged, cfg.hidden, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)

    def body(r):
        r.launch("agi_patchify_f32_bf16", (grid_for(cfg.patches * cfg.patch_k), 1, 1), (256, 1, 1),
                 [Tensor("pixels"), Tensor("rows"), Tensor("pos"), U32(cfg.images), U32(cfg.channels),
                  U32(cfg.image_size), U32(cfg.patch), U32(cfg.temporal), U32(cfg.window), U32(cfg.merge),
                  U32(cfg.patch_k), U32(cfg.patch_k)])
        r.launch("agi_unwindow_rows_bf16", (grid_for(cfg.merged * cfg.hidden // 8), 1, 1), (256, 1, 1),
                 [Tensor("merged"), Tensor("raster"), U32(cfg.images), U32(cfg.grid // cfg.merge),
                  U32(cfg.window // cfg.merge), U32(cfg.hidden), U32(cfg.hidden), U32(cfg.hidden)])

    got, _ = run_recipe(tmp_path, {}, {"pixels": pixels, "merged": merged},
                        {"rows": (torch.bfloat16, (cfg.patches, cfg.patch_k)), "pos": (torch.int32, (3, cfg.patches)),
                         "raster": (torch.bfloat16, (cfg.merged, cfg.hidden))}, body)
    want_rows, want_pos = oracle_vl.patchify(cfg, pixels)
    assert torch.equal(got["rows"], want_rows) and torch.equal(got["pos"], want_pos)
    assert torch.equal(got["raster"], oracle_vl.unwindow(cfg, merged))


def run_prefill(tmp_path, cfg, w, x):
    aim = build_aim(tmp_path, w, qwen_vl.build_recipe(cfg, describe(w)))
    runner = Runner(aim)
    dev = {k: v.cuda() for k, v in x.items()}
    out = runner.empty_outputs()
    for _ in range(2):
        runner.run(dev, out)
    torch.cuda.synchronize()
    return {k: v.cpu() for k, v in out.items()}, runner.stats()


def test_reduced_depth_prefill_matches_oracle(tmp_path):
    # real widths and token counts; 4 vision blocks (the last with full attention) and 4 decoder layers
    cfg = qwen_vl.VlConfig(v_layers=4, v_full_layers=(3,), layers=4, vocab=4096)
    w, x = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
    got, stats = run_prefill(tmp_path, cfg, w, x)
    assert got["status"].item() == 0
    # vision tower alone (merged tokens reach the oracle's language model through the same path)
    want_hidden, want_cache = oracle_vl.forward(cfg, w, x["pixels"], x["input_ids"], x["positions"])
    cos, err = ops.cosine(got["hidden_out"], want_hidden), ops.max_rel_err(got["hidden_out"], want_hidden)
    cache_err = ops.max_rel_err(got["kv_cache"], want_cache)
    print(f"prefill 4+4: cosine={cos:.6f} max_rel_err={err:.3e} kv max_rel_err={cache_err:.3e} "
          f"launches={stats['launches_per_enqueue']}")
    assert cos >= 0.999 and err < 2e-2 and cache_err < 2e-2
    assert stats["graph_launches"] == 2 and stats["graphs_built"] == 1

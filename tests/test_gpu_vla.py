"""GR00T-N1.5-shaped model end to end on the GPU: pixels and token ids in, action chunk out, one profile."""
from __future__ import annotations

import pytest
import torch

from aginfer_b200.recipes import vla
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner
from oracle import dit as oracle_dit
from oracle import ops
from oracle import vla as oracle_vla

pytestmark = pytest.mark.gpu


def test_reduced_depth_vla_matches_oracle(tmp_path):
    """Real widths (2048 backbone, 1536 head, 288 context tokens); 2 vision blocks, 2 decoder layers, 4 DiT blocks.

    The action chunk is held to its tier (cosine >= 0.999, max-rel <= 2e-2) for the BF16 head given the same
    context: the oracle's head is fed the hidden states the GPU's prefill exported.  The FP8 prefill in front of
    it is covered block by block in test_gpu_qwen_vl.py; free-running, its output and with it the actions are
    checked by cosine."""
    cfg = vla.reduced()
    w, x = vla.synthetic_weights(cfg), vla.synthetic_inputs(cfg)
    aim = build_aim(tmp_path, w, vla.build_recipe(cfg, describe(w)))
    runner = Runner(aim)
    dev = {k: v.cuda() for k, v in x.items()}
    out = runner.empty_outputs()
    for _ in range(2):
        runner.run(dev, out)
    torch.cuda.synchronize()
    got = {k: v.cpu() for k, v in out.items()}
    assert got["status"].item() == 0
    want = oracle_dit.forward(cfg.head, w, got["hidden_out"], x["state"], x["noise"])
    cos, err = ops.cosine(got["actions"], want), ops.max_rel_err(got["actions"], want)
    free_actions, free_hidden = oracle_vla.forward(cfg, w, x["pixels"], x["input_ids"], x["positions"], x["state"], x["noise"])
    free_cos, hidden_cos = ops.cosine(got["actions"], free_actions), ops.cosine(got["hidden_out"], free_hidden)
    print(f"vla: actions given the same context cosine={cos:.6f} max_rel_err={err:.3e}; free-running actions "
          f"cosine={free_cos:.5f}, context cosine={hidden_cos:.5f}; launches={runner.stats()['launches_per_enqueue']}")
    assert cos >= 0.999 and err < 2e-2
    assert hidden_cos >= 0.99 and free_cos >= 0.99
    stats = runner.stats()
    assert stats["graph_launches"] == 2 and stats["graphs_built"] == 1

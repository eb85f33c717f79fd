"""DiT recipe: structure checks on CPU (no GPU), and the oracle's own invariants on a tiny shape."""
import torch

from aginfer_b200 import planfmt
from aginfer_b200.recipes import dit
from aginfer_b200.target import CudaArch
from oracle import dit as oracle_dit

TINY = dit.DitConfig(layers=2, hidden=128, heads=4, head_dim=32, mlp=256, action_dim=32, state_dim=64, horizon=16,
                     backbone_tokens=24, backbone_dim=128, steps=2, encoder_hidden=128, out_dim=128, time_dim=64)


def test_weight_inventory_matches_the_published_size():
    cfg = dit.DitConfig()
    shapes = dit.weight_shapes(cfg)
    per_block = sum(torch.Size(v).numel() for k, v in shapes.items() if ".blocks." in k and k.endswith(".weight"))
    assert per_block == 541_065_216            # the 541 M block parameters the baseline floors are computed from
    acc = dit.algorithmic_bytes(cfg)
    assert acc["per_chunk"] < cfg.steps * acc["total_weights"]   # hoisting saves traffic
    assert acc["once"] + acc["per_step"] == acc["total_weights"]


def test_recipe_compiles_and_is_one_graph_safe_profile():
    cfg = dit.DitConfig()
    r = dit.build_recipe(cfg)
    plan = r.plan()
    compiled = planfmt.compile_execution_plan(plan, CudaArch.SM100, weight_size=r.weight_bytes)
    assert compiled.input_names == ("backbone_features", "state", "noise") and compiled.output_names == ("actions",)
    launches = plan["shape_dispatch"][0]["launches"]
    assert plan["cuda_graph_templates"] == [{"profile": "default"}]
    per_step = [l for l in launches if l["kernel"] == "agi_euler_step"]
    assert len(per_step) == cfg.steps
    kernels = {l["kernel"] for l in launches}
    assert {"agi_gemm_tc_bf16_x16", "agi_gemm_stream_bf16_t3", "agi_attention_mma_bf16", "agi_layernorm_bf16"} <= kernels
    # every weight of the checkpoint is used by some launch
    used = {a["weights_offset"] for l in launches for a in l["arguments"] if "weights_offset" in a}
    assert used == set(r.weight_offsets.values())


def test_oracle_runs_and_is_deterministic_on_a_tiny_shape():
    w = dit.synthetic_weights(TINY, seed=2)
    x = dit.synthetic_inputs(TINY, seed=2)
    a = oracle_dit.forward(TINY, w, x["backbone_features"], x["state"], x["noise"])
    b = oracle_dit.forward(TINY, w, x["backbone_features"], x["state"], x["noise"])
    assert a.shape == (16, 32) and a.dtype == torch.float32 and torch.equal(a, b)
    assert torch.isfinite(a).all() and not torch.equal(a, x["noise"].float())
    assert dit.build_recipe(TINY).plan()["arena_bytes"] > 0

"""DiT recipe: structure checks on CPU (no GPU), and the oracle's own invariants on a tiny shape."""
import pytest
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


def _check_recipe(cfg, r, expect_kernels):
    plan = r.plan()
    compiled = planfmt.compile_execution_plan(plan, CudaArch.SM100, weight_size=r.weight_bytes)
    assert compiled.input_names == ("backbone_features", "state", "noise") and compiled.output_names == ("actions", "status")
    launches = plan["shape_dispatch"][0]["launches"]
    assert plan["cuda_graph_templates"] == [{"profile": "default"}]
    per_step = [l for l in launches if l["kernel"] == "agi_euler_step"]
    assert len(per_step) == cfg.steps
    kernels = {l["kernel"] for l in launches}
    assert expect_kernels <= kernels
    # every weight of the checkpoint is used by some launch
    used = {a["weights_offset"] for l in launches for a in l["arguments"] if "weights_offset" in a}
    assert used == set(r.weight_offsets.values())
    return launches


def test_recipe_compiles_and_is_one_graph_safe_profile():
    cfg = dit.DitConfig()
    launches = _check_recipe(cfg, dit.build_recipe(cfg),
                             {"agi_gemm_tc_bf16_x16", "agi_gemm_stream_bf16_t3", "agi_attention_mma_bf16", "agi_layernorm_bf16"})
    assert len(launches) > 400


def test_block_kernel_recipe_is_one_launch_per_denoising_step():
    cfg = dit.DitConfig()
    launches = _check_recipe(cfg, dit.build_recipe(cfg, block_kernel=True), {"agi_coop_dit_blocks_bf16_t3", "agi_store_pointers16"})
    blocks = [l for l in launches if l["kernel"].startswith("agi_coop_dit_blocks")]
    assert len(blocks) == cfg.steps and len(launches) <= 150
    for step, l in enumerate(blocks):
        assert l["grid"] == [148, 1, 1] and l["block"] == [384, 1, 1] and l["shared_bytes"] <= 227 * 1024
        scalars = [a["scalar_u32"] for a in l["arguments"] if "scalar_u32" in a]
        layers, T, D, heads, head_dim, mlp, span, ctx, cross_mask, mod_offset, slots = scalars
        assert (layers, T, D, heads, head_dim, mlp, ctx) == (16, 17, 1536, 32, 48, 6144, 300)
        assert span == 1536 and cross_mask == 0x5555 and mod_offset == step * 2 * D and slots >= 3
    # each launch gets its own grid-wide arrival counter, inside the per-run area the prologue clears
    counters = [l["arguments"][7]["arena_offset"] for l in blocks]
    assert len(set(counters)) == cfg.steps and all(64 <= c < 1024 for c in counters)
    # the tiny shape is covered too
    assert any(l["kernel"].startswith("agi_coop_dit_blocks")
               for l in dit.build_recipe(TINY, block_kernel=True).plan()["shape_dispatch"][0]["launches"])
    # a shape outside the kernel's limits is refused, not silently built differently
    wide = dit.DitConfig(layers=2, hidden=2048, heads=32, head_dim=64, mlp=4096)
    try:
        dit.build_recipe(wide, block_kernel=True)
        raise AssertionError("expected a ValueError")
    except ValueError:
        pass


def test_oracle_runs_and_is_deterministic_on_a_tiny_shape():
    w = dit.synthetic_weights(TINY, seed=2)
    x = dit.synthetic_inputs(TINY, seed=2)
    a = oracle_dit.forward(TINY, w, x["backbone_features"], x["state"], x["noise"])
    b = oracle_dit.forward(TINY, w, x["backbone_features"], x["state"], x["noise"])
    assert a.shape == (16, 32) and a.dtype == torch.float32 and torch.equal(a, b)
    assert torch.isfinite(a).all() and not torch.equal(a, x["noise"].float())
    assert dit.build_recipe(TINY).plan()["arena_bytes"] > 0


def test_packed_checkpoint_routes_the_block_matrices_to_the_tensor_core_stream_kernel():
    """The packaging-time layout pass keeps names and values (it is undone exactly) and the recipe, given the packed
    shapes, multiplies those matrices with agi_gemm_tcs_bf16*; the cross-attention K / V projections stay row-major."""
    import collections

    import torch

    from aginfer_b200.recipes.builder import tcs_tiling
    from aginfer_b200.recipes.layout import unpack_kblock_swizzled
    from aginfer_b200.recipes.package import describe
    cfg = dit.DitConfig(layers=2)
    w = dit.synthetic_weights(cfg, seed=2)
    packed = dit.pack_checkpoint(cfg, w)
    names = dit.packed_names(cfg)
    assert len(names) == 4 + 6 and all(packed[n].dim() == 3 for n in names)
    assert all(torch.equal(unpack_kblock_swizzled(packed[n], w[n].shape[0]), w[n]) for n in names)
    assert all(packed[k] is v for k, v in w.items() if k not in names)
    recipe = dit.build_recipe(cfg, describe(packed))
    kernels = collections.Counter(l["kernel"] for l in recipe.plan()["shape_dispatch"][0]["launches"])
    tcs = {k: v for k, v in kernels.items() if k.startswith("agi_gemm_tcs_bf16")}
    assert sum(tcs.values()) == cfg.steps * cfg.layers * 4 and kernels["agi_gemm_tc_bf16_x16"] >= 1
    with pytest.raises(ValueError, match="row-major"):
        dit.build_recipe(cfg, describe(packed), block_kernel=True)
    # the geometry chosen for the head's four shapes: at most two CTAs per SM, K slices of 3-4 blocks
    for tiles, K, want in ((48, 1536, (6, 1, 4)), (36, 1536, (8, 1, 3)), (12, 1536, (8, 1, 3)), (12, 6144, (8, 3, 4))):
        t = tcs_tiling(17, tiles, K)
        assert (t["cluster"], t["groups"], t["kb"]) == want and t["ctas"] <= 296 and t["shared_bytes"] <= 113 * 1024
    assert tcs_tiling(33, 12, 1536) is None and tcs_tiling(17, 12, 1000) is None

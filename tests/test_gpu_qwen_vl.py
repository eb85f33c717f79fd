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


def run_prefill(tmp_path, cfg, w, x, trace=False, packed=False, operand_trace=()):
    if packed:
        w = qwen_vl.pack_checkpoint(w)
    aim = build_aim(tmp_path, w, qwen_vl.build_recipe(cfg, describe(w), trace=trace, packed=packed,
                                                       operand_trace=operand_trace))
    runner = Runner(aim)
    dev = {k: v.cuda() for k, v in x.items()}
    out = runner.empty_outputs()
    for _ in range(2):
        runner.run(dev, out)
    torch.cuda.synchronize()
    return {k: v.cpu() for k, v in out.items()}, runner.stats()


REDUCED = dict(v_layers=4, v_full_layers=(3,), layers=4, vocab=4096)
FULL = dict(vocab=4096)          # all 32 vision blocks and 36 decoder layers; only the vocabulary is cut


@pytest.mark.parametrize("depth", [REDUCED, FULL], ids=["reduced_depth", "full_depth"])
@pytest.mark.parametrize("packed", [False, True], ids=["row_major", "packed"])
def test_prefill_matches_oracle_block_by_block(tmp_path, packed, depth):
    """Real widths and token counts; reduced depth = 4 vision blocks (the last with full attention) and 4 decoder
    layers, full depth = BASELINE config 4 as it stands.

    Every GEMM input is quantised per tensor with a scale taken from the tensor's largest element, so a
    last-bit difference in one activation moves the scale of a whole tensor and the next GEMM sees a
    different E4M3 grid.  The parity claim is therefore made block by block: each block's output on the GPU
    against the oracle's block fed with the GPU's own input, at ops.FP8_BLOCK_TOL (the oracle's own
    resolution under one-ulp disturbances, measured in tests/test_qwen_vl_cpu.py); K/V, patch embedding,
    merger and final norm, which have at most one quantisation upstream, at 2e-2; indexing bit-exact."""
    cfg = qwen_vl.VlConfig(**depth)
    w, x = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
    got, stats = run_prefill(tmp_path, cfg, w, x, trace=True, packed=packed)
    assert got["status"].item() == 0
    patches, pos = oracle_vl.patchify(cfg, x["pixels"])
    vt, ht = got["vision_trace"], got["hidden_trace"]
    errs = {"patch_embed": ops.max_rel_err(vt[0], ops.gemm(patches, w["visual.patch_embed.proj.weight"]))}
    for i in range(cfg.v_layers):
        errs[f"vision_block_{i}"] = ops.max_rel_err(vt[i + 1], oracle_vl.vision_block(cfg, w, i, vt[i], pos))
    errs["merger"] = ops.max_rel_err(got["merged_out"], oracle_vl.merger(cfg, w, vt[-1]))
    assert torch.equal(ht[0], oracle_vl.embed_prefix(cfg, w, got["merged_out"], x["input_ids"]))   # indexing: exact
    for i in range(cfg.layers):
        want_h, want_k, want_v = oracle_vl.decoder_layer(cfg, w, i, ht[i], x["positions"])
        errs[f"decoder_layer_{i}"] = ops.max_rel_err(ht[i + 1], want_h)
        errs[f"kv_{i}"] = max(ops.max_rel_err(got["kv_cache"][i, 0], want_k), ops.max_rel_err(got["kv_cache"][i, 1], want_v))
    errs["final_norm"] = ops.max_rel_err(got["hidden_out"], ops.rmsnorm(ht[-1], w["model.norm.weight"], cfg.eps))
    worst = {kind: max(v for k, v in errs.items() if k.startswith(kind)) for kind in ("vision_block", "decoder_layer", "kv_")}
    print(f"teacher-forced block errors ({len(errs)} checks): worst", {k: round(v, 5) for k, v in worst.items()},
          {k: round(v, 5) for k, v in errs.items() if not k.startswith(("vision_block", "decoder_layer", "kv_"))})
    for name, err in errs.items():
        assert err < (ops.FP8_BLOCK_TOL if name.startswith(("vision_block", "decoder_layer")) else 2e-2), (name, errs)
    want_hidden, _ = oracle_vl.forward(cfg, w, x["pixels"], x["input_ids"], x["positions"])
    cos = ops.cosine(got["hidden_out"], want_hidden)
    print(f"end to end: cosine={cos:.5f} max_rel_err={ops.max_rel_err(got['hidden_out'], want_hidden):.3e} "
          f"launches={stats['launches_per_enqueue']}")
    # free-running over all blocks the two drift apart by the arithmetic's own noise floor: the oracle against a
    # copy of itself disturbed by one ulp in a tenth of the attention outputs ends at 0.9775 after 68 blocks
    # (tests/test_qwen_vl_cpu.py measures one block of it), so the end-to-end figure is a sanity bound, not the claim
    assert cos >= (0.99 if depth is REDUCED else 0.95)
    assert stats["graph_launches"] == 2 and stats["graphs_built"] == 1


def test_fp8_blocks_hold_the_tight_tier_when_the_operands_are_teacher_forced(tmp_path):
    """The north star's 2e-2 for block outputs, with the quantised GEMM operands teacher-forced.

    Free-running FP8 blocks are compared at 5e-2 above because a last-bit difference upstream moves a whole
    tensor's scale.  Here that effect is taken out instead of tolerated: the recipe exports, for a few blocks, the
    E4M3 bytes and the scale of every GEMM input as they stand on the device; the oracle's block is fed those
    operands, so the two sides multiply identical numbers and may differ only by accumulation order and one bf16
    rounding (held to 2e-2, the tier of GEMM and block outputs).  What sits between two GEMMs (norm, rotary
    embedding, attention, SwiGLU, quantiser) is checked through the operands themselves: each exported operand,
    dequantised, against the oracle's own tensor at that point, within the E4M3 grid's resolution (half a step of
    the top binade = 16 / 448 of the range) plus the 1e-2 that kernels fed identical inputs are held to, and its
    scale against amax / 448 of the same tensor."""
    cfg = qwen_vl.VlConfig(**REDUCED)
    blocks = ("visual.blocks.0", "visual.blocks.3", "model.layers.0", "model.layers.3")
    w, x = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
    got, _ = run_prefill(tmp_path, cfg, w, x, trace=True, operand_trace=blocks)
    assert got["status"].item() == 0
    _, pos = oracle_vl.patchify(cfg, x["pixels"])
    report = {}
    for block in blocks:
        i = int(block.rsplit(".", 1)[1])
        operands = [(got[f"{block}.operand{j}"].view(torch.float8_e4m3fn), got[f"{block}.scale{j}"].reshape(())) for j in range(4)]
        if block.startswith("visual."):
            want, refs = oracle_vl.vision_block_forced(cfg, w, i, got["vision_trace"][i], pos, operands)
            out = got["vision_trace"][i + 1]
        else:
            want, refs = oracle_vl.decoder_layer_forced(cfg, w, i, got["hidden_trace"][i], x["positions"], operands)
            out = got["hidden_trace"][i + 1]
        err = ops.max_rel_err(out, want)
        grid = [ops.max_rel_err(q.float() * s, ref) for (q, s), ref in zip(operands, refs)]
        scales = [abs(float(s) / (float(ref.float().abs().max()) / 448.0) - 1.0) for (q, s), ref in zip(operands, refs)]
        report[block] = (round(err, 5), [round(g, 4) for g in grid], [round(v, 5) for v in scales])
        assert err <= 2e-2, (block, err)
        assert max(grid) <= 16.0 / 448.0 + 1e-2, (block, grid)      # half a top-binade step + the kernels' own 1e-2
        assert max(scales) <= 1e-2, (block, scales)
    print("operand-teacher-forced blocks (output error, operand error per quantisation point, scale deviation):", report)

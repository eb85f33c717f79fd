"""Qwen2.5-VL-shaped prefill (BASELINE config 4): recipe construction and oracle plumbing on CPU."""
from __future__ import annotations

import collections

import torch

from aginfer_b200 import planfmt
from aginfer_b200.recipes import qwen_vl
from aginfer_b200.recipes.package import describe
from aginfer_b200.target import CudaArch
from oracle import ops
from oracle import qwen_vl as oracle_vl

SMALL = qwen_vl.VlConfig(v_layers=2, v_full_layers=(1,), layers=2, vocab=512)


def table(cfg):
    """name -> (dtype, shape) of the checkpoint without materialising it."""
    t = {"visual.patch_embed.proj.weight": ("BF16", (cfg.v_hidden, cfg.patch_k)),
         "visual.merger.ln_q.weight": ("BF16", (cfg.v_hidden,)), "model.norm.weight": ("BF16", (cfg.hidden,)),
         "model.embed_tokens.weight": ("BF16", (cfg.vocab, cfg.hidden))}

    def fp8(name, n, k, bias=True):
        t[f"{name}.weight"], t[f"{name}.weight_scale"] = ("F8_E4M3", (n, k)), ("F32", ())
        if bias:
            t[f"{name}.bias"] = ("BF16", (n,))

    for i in range(cfg.v_layers):
        for name, (n, k, _, _) in qwen_vl.vision_linears(cfg, i).items():
            fp8(name, n, k)
        t[f"visual.blocks.{i}.norm1.weight"] = t[f"visual.blocks.{i}.norm2.weight"] = ("BF16", (cfg.v_hidden,))
    fp8("visual.merger.mlp.0", cfg.merged_dim, cfg.merged_dim)
    fp8("visual.merger.mlp.2", cfg.hidden, cfg.merged_dim)
    for i in range(cfg.layers):
        for name, (n, k) in qwen_vl.llm_linears(cfg, i).items():
            fp8(name, n, k, bias=name.split(".")[-1] in ("q_proj", "k_proj", "v_proj"))
        t[f"model.layers.{i}.input_layernorm.weight"] = ("BF16", (cfg.hidden,))
        t[f"model.layers.{i}.post_attention_layernorm.weight"] = ("BF16", (cfg.hidden,))
    return t


def test_table_matches_the_synthetic_checkpoint():
    w = qwen_vl.synthetic_weights(SMALL)
    assert {k: (d, tuple(s)) for k, (d, s) in describe(w).items()} == table(SMALL)


def test_full_size_recipe_compiles_to_a_plan():
    cfg = qwen_vl.VlConfig()
    assert (cfg.patches, cfg.merged, cfg.tokens, cfg.v_mlp_padded, cfg.patch_k) == (512, 128, 288, 3456, 1216)
    recipe = qwen_vl.build_recipe(cfg, table(cfg))
    launches = recipe.plan()["shape_dispatch"][0]["launches"]
    kinds = collections.Counter(l["kernel"] for l in launches)
    # 5 linears per vision block, 2 merger, 7 per decoder layer, plus the bf16 patch embedding
    fp8 = sum(n for k, n in kinds.items() if k.startswith("agi_gemm_") and "e4m3" in k)
    assert fp8 == 4 * 32 + 2 + 5 * 36                 # q|k|v share a launch; so do the vision tower's gate|up
    assert kinds["agi_gemm_tc_e4m3_x3"] == 32 + 36
    ungrouped = qwen_vl.build_recipe(cfg, table(cfg), group=False).plan()["shape_dispatch"][0]["launches"]
    assert sum(1 for l in ungrouped if "e4m3" in l["kernel"] and "gemm" in l["kernel"]) == 5 * 32 + 2 + 7 * 36
    assert kinds["agi_quantize_e4m3_bf16"] == 4 * 32 + 2 + 4 * 36      # q/k/v and gate/up share one quantisation
    assert kinds["agi_absmax_bf16"] == 1                               # only the merger's GELU output needs its own pass
    assert kinds["agi_patchify_f32_bf16"] == kinds["agi_unwindow_rows_bf16"] == kinds["agi_gather_rows_bf16"] == 1
    compiled = planfmt.compile_execution_plan(recipe.plan(), CudaArch.SM100, weight_size=recipe.weight_bytes)
    decoded = planfmt.decode_plan(compiled.data)
    assert len(decoded["shape_dispatch"][0]["launches"]) == len(launches)
    alg = qwen_vl.algorithmic(cfg)
    assert abs(alg["fp8_weight_bytes"] / 3.44e9 - 1) < 0.01 and abs(alg["flops"] / 2.25e12 - 1) < 0.01


def test_window_order_and_its_inverse():
    cfg = SMALL
    order = oracle_vl.window_order(cfg)
    assert sorted(map(tuple, order.tolist())) == [(y, x) for y in range(16) for x in range(16)]
    # every run of 64 tokens is one 8 x 8 window, every run of 4 one 2 x 2 merge group
    for w0 in range(0, 256, 64):
        ys, xs = order[w0:w0 + 64, 0], order[w0:w0 + 64, 1]
        assert ys.max() - ys.min() == 7 and xs.max() - xs.min() == 7
    for g0 in range(0, 256, 4):
        assert len({(y // 2, x // 2) for y, x in order[g0:g0 + 4].tolist()}) == 1
    # unwindow puts merged token (gy, gx) at raster row gy * 8 + gx
    tags = torch.tensor([[img * 64 + (y // 2) * 8 + x // 2] for img in range(cfg.images)
                         for y, x in order[::4].tolist()], dtype=torch.float32)
    assert oracle_vl.unwindow(cfg, tags).reshape(-1).tolist() == list(range(cfg.images * 64))


def test_patchify_matches_a_strided_view():
    cfg = SMALL
    pixels = qwen_vl.synthetic_inputs(cfg)["pixels"]
    rows, pos = oracle_vl.patchify(cfg, pixels)
    assert rows.shape == (512, 1216) and pos.shape == (3, 512)
    token = 256 + 77                                            # second image
    py, px = pos[0, token].item(), pos[1, token].item()
    tile = pixels[1, :, py * 14:(py + 1) * 14, px * 14:(px + 1) * 14]
    want = torch.stack([tile, tile], dim=1).reshape(-1).to(torch.bfloat16)
    assert torch.equal(rows[token, :1176], want) and rows[token, 1176:].abs().max() == 0


def test_rope_positions_follow_the_prefix_layout():
    pos = qwen_vl.rope_positions(qwen_vl.VlConfig())
    assert pos.shape == (3, 288)
    assert pos[:, 0].tolist() == [0, 0, 0] and pos[:, 63].tolist() == [0, 7, 7]
    assert pos[:, 64].tolist() == [8, 8, 8] and pos[:, 127].tolist() == [8, 15, 15]
    assert pos[:, 128].tolist() == [16, 16, 16] and pos[:, 287].tolist() == [175, 175, 175]


def test_small_oracle_runs_and_padding_is_inert():
    cfg = qwen_vl.VlConfig(v_layers=1, v_full_layers=(0,), layers=1, vocab=256)
    w, x = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
    hidden, cache = oracle_vl.forward(cfg, w, x["pixels"], x["input_ids"], x["positions"])
    assert hidden.shape == (288, 2048) and cache.shape == (1, 2, 288, 256)
    assert torch.isfinite(hidden.float()).all() and hidden.float().std() > 0.1
    # rows 3420.. of gate/up and columns 3420.. of down are zero bytes
    assert w["visual.blocks.0.mlp.gate_proj.weight"].view(torch.uint8)[3420:].max() == 0
    assert w["visual.blocks.0.mlp.down_proj.weight"].view(torch.uint8)[:, 3420:].max() == 0


def test_fp8_block_tolerance_is_the_oracles_own_resolution():
    """One decoder layer of the oracle against itself with the attention output moved by one bf16 ulp on a
    tenth of its elements: the per-tensor dynamic E4M3 scales turn that into a few percent of the output range.
    This is why FP8 blocks are compared at ops.FP8_BLOCK_TOL and kernels (identical inputs) at 1e-2."""
    cfg = qwen_vl.VlConfig(v_layers=1, v_full_layers=(0,), layers=1, vocab=256)
    w, x = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
    h = torch.randn(cfg.tokens, cfg.hidden, generator=torch.Generator().manual_seed(11)).to(torch.bfloat16)
    ref, ref_k, _ = oracle_vl.decoder_layer(cfg, w, 0, h, x["positions"])
    worst = 0.0
    for seed in (1, 2, 3):
        out, k, _ = oracle_vl.decoder_layer(cfg, w, 0, h, x["positions"], attn_hook=lambda a: ops.ulp_noise(a, 0.1, seed))
        assert torch.equal(k, ref_k)                      # upstream of the disturbance: untouched
        worst = max(worst, ops.max_rel_err(out, ref))
        assert ops.cosine(out, ref) > 0.999
    assert 1e-2 < worst < ops.FP8_BLOCK_TOL, worst


def test_packed_layout_round_trip_and_addressing():
    from aginfer_b200.recipes.layout import (pack_kblock_swizzled, padded_token_rows, padded_weight_rows,
                                             unpack_kblock_swizzled)
    w = (torch.randn(300, 384, generator=torch.Generator().manual_seed(2)) * 50).to(torch.float8_e4m3fn)
    p = pack_kblock_swizzled(w)
    assert p.shape == (3, 512, 128) and p.dtype == torch.float8_e4m3fn and padded_weight_rows(300) == 512
    assert torch.equal(unpack_kblock_swizzled(p, 300).view(torch.uint8), w.view(torch.uint8))
    raw, src = p.view(torch.uint8).reshape(-1), w.view(torch.uint8)
    for r, kbyte in ((0, 0), (77, 200), (299, 383), (130, 129)):
        kb, c, b = kbyte // 128, (kbyte % 128) // 16, kbyte % 16
        assert raw[(kb * 512 + r) * 128 + ((c ^ (r & 7)) << 4) + b] == src[r, kbyte]
    assert raw.reshape(3, 512, 128)[:, 300:].max() == 0                       # padding rows are zero
    h = torch.randn(16, 64).to(torch.bfloat16)                                 # two-byte elements: 64 per block
    assert torch.equal(unpack_kblock_swizzled(pack_kblock_swizzled(h), 16), h)
    assert padded_token_rows(288) == 768 and padded_token_rows(256) == 512
    packed = qwen_vl.pack_checkpoint(qwen_vl.synthetic_weights(SMALL))
    assert packed["model.layers.0.mlp.down_proj.weight"].shape == (86, 2048, 128)
    assert packed["model.embed_tokens.weight"].shape == (512, 2048)           # bf16 tensors are left alone

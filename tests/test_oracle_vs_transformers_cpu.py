"""The oracle's Qwen2.5-VL conventions pinned to a published implementation (Hugging Face ``transformers``).

The reference project has no model arithmetic, so nothing in it can pin ``oracle/qwen_vl.py``.  What can differ
silently from the published architecture is convention, not arithmetic: which rotary pair turns with which
position stream and at which frequency, the order of patch tokens inside windows and their way back, where the
biases are, how the merger groups patches.  These tests run the oracle's vision tower and decoder layer with
the per-tensor FP8 quantisation switched off (identity) on a tiny random configuration and compare them with
``transformers``' Qwen2.5-VL modules carrying the same weights, in fp32 on the CPU.

Known, deliberate differences, inside the tolerance: the oracle rounds to bf16 where the GPU recipe stores
bf16, and its merger uses the tanh form of GELU (the module uses erf).  Tolerances are stated where they are
used.  Skipped where ``transformers`` (or its Qwen2.5-VL model) is not importable.
"""
from __future__ import annotations

import pytest
import torch

from aginfer_b200.recipes import qwen_vl
from oracle import ops
from oracle import qwen_vl as oracle_vl

hf = pytest.importorskip("transformers.models.qwen2_5_vl.modeling_qwen2_5_vl")
hf_cfg = pytest.importorskip("transformers.models.qwen2_5_vl.configuration_qwen2_5_vl")

CFG = qwen_vl.VlConfig(images=1, v_layers=2, v_full_layers=(1,), v_hidden=128, v_heads=4, v_mlp=256, layers=1, hidden=256,
                       heads=4, kv_heads=2, head_dim=64, intermediate=512, vocab=64, text_tokens=8, sections=(8, 12, 12))


@pytest.fixture()
def unquantised(monkeypatch):
    """Identity in place of the dynamic E4M3 quantisation: the oracle then is the plain architecture."""
    monkeypatch.setattr(ops, "quantize_e4m3", lambda x: (x, torch.ones(())))


def linear(out: dict, ours: str, module, bias: bool = True) -> None:
    out[f"{ours}.weight"] = module.weight.detach().clone()
    out[f"{ours}.weight_scale"] = torch.ones(())
    if bias and module.bias is not None:
        out[f"{ours}.bias"] = module.bias.detach().clone()


def close(got: torch.Tensor, want: torch.Tensor, cosine: float = 0.9999, max_rel: float = 2e-2) -> None:
    assert ops.cosine(got, want) >= cosine, ops.cosine(got, want)
    assert ops.max_rel_err(got, want) <= max_rel, ops.max_rel_err(got, want)


# The two module-level comparisons run with sharp attention (large query / key weights), because with the usual
# small random weights every attention row is nearly uniform and no rotary convention could be told from another.
# Sharp attention also amplifies the oracle's bf16 roundings of q and k, hence the wider band; a wrong convention
# lands far outside it (one frequency ladder instead of two in the vision tower: cosine 0.90; height and width
# sections swapped in the decoder: cosine 0.9991, max relative error 0.10).
BLOCK = dict(cosine=0.9995, max_rel=4e-2)


def test_mrope_is_the_published_multimodal_rotary_embedding():
    g = torch.Generator().manual_seed(0)
    S, H, D = 24, 4, 64
    q, k = torch.randn(S, H, D, generator=g), torch.randn(S, 2, D, generator=g)
    positions = torch.stack([torch.randint(0, 40, (S,), generator=g) for _ in range(3)]).int()
    inv_freq = 1e6 ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    freqs = positions.float()[:, None, :, None] * inv_freq[None, None, None, :]           # [3, 1, S, D / 2]
    emb = torch.cat([freqs, freqs], dim=-1)
    want_q, want_k = hf.apply_multimodal_rotary_pos_emb(q.transpose(0, 1)[None], k.transpose(0, 1)[None], emb.cos(),
                                                        emb.sin(), [8, 12, 12])
    close(ops.mrope(q.bfloat16(), positions, 1e6, (8, 12, 12)).float(), want_q[0].transpose(0, 1))
    close(ops.mrope(k.bfloat16(), positions, 1e6, (8, 12, 12)).float(), want_k[0].transpose(0, 1))


def test_vision_tower_matches_the_published_module(unquantised):
    cfg = CFG
    torch.manual_seed(1)
    config = hf_cfg.Qwen2_5_VLVisionConfig(depth=cfg.v_layers, hidden_size=cfg.v_hidden, intermediate_size=cfg.v_mlp,
                                           num_heads=cfg.v_heads, patch_size=cfg.patch, spatial_merge_size=cfg.merge,
                                           temporal_patch_size=cfg.temporal, window_size=cfg.window * cfg.patch,
                                           out_hidden_size=cfg.hidden, fullatt_block_indexes=list(cfg.v_full_layers))
    config._attn_implementation = "eager"
    model = hf.Qwen2_5_VisionTransformerPretrainedModel(config).float().eval()
    for p in model.parameters():           # the default initialisation leaves norms at 1 and biases at 0: make them count
        torch.nn.init.normal_(p, std=0.05) if p.dim() > 1 else torch.nn.init.normal_(p, std=0.2)
    for name, p in model.named_parameters():
        if "norm" in name or "ln_q" in name:
            torch.nn.init.normal_(p, mean=1.0, std=0.1)
        if "attn.qkv.weight" in name:      # sharp attention: the scores, and with them the rotary convention, matter
            torch.nn.init.normal_(p, std=0.3)

    w: dict = {}
    conv = model.patch_embed.proj.weight.detach().reshape(cfg.v_hidden, -1)
    w["visual.patch_embed.proj.weight"] = torch.nn.functional.pad(conv, (0, cfg.patch_k - conv.shape[1]))
    for i, blk in enumerate(model.blocks):
        b = f"visual.blocks.{i}"
        w[f"{b}.norm1.weight"], w[f"{b}.norm2.weight"] = blk.norm1.weight.detach().clone(), blk.norm2.weight.detach().clone()
        linear(w, f"{b}.attn.qkv", blk.attn.qkv)
        linear(w, f"{b}.attn.proj", blk.attn.proj)
        for part in ("gate_proj", "up_proj", "down_proj"):
            linear(w, f"{b}.mlp.{part}", getattr(blk.mlp, part))
    w["visual.merger.ln_q.weight"] = model.merger.ln_q.weight.detach().clone()
    linear(w, "visual.merger.mlp.0", model.merger.mlp[0])
    linear(w, "visual.merger.mlp.2", model.merger.mlp[2])

    pixels = torch.rand(cfg.images, cfg.channels, cfg.image_size, cfg.image_size, generator=torch.Generator().manual_seed(2))
    # the module takes patch rows grouped by 2 x 2 merge unit, units in raster order, each row flattened (c, t, y, x)
    G, m, p = cfg.grid // cfg.merge, cfg.merge, cfg.patch
    rows = []
    for gy in range(G):
        for gx in range(G):
            for sy in range(m):
                for sx in range(m):
                    py, px = gy * m + sy, gx * m + sx
                    tile = pixels[0, :, py * p:(py + 1) * p, px * p:(px + 1) * p]
                    rows.append(tile[:, None].expand(-1, cfg.temporal, -1, -1).reshape(-1))
    with torch.no_grad():
        want = model(torch.stack(rows), grid_thw=torch.tensor([[1, cfg.grid, cfg.grid]])).pooler_output
    got = oracle_vl.unwindow(cfg, oracle_vl.vision_tower(cfg, w, pixels))
    assert got.shape == want.shape == (cfg.merged, cfg.hidden)
    close(got.float(), want, **BLOCK)


def test_decoder_layer_matches_the_published_module(unquantised):
    cfg = CFG
    torch.manual_seed(3)
    rope = {"rope_type": "default", "mrope_section": list(cfg.sections), "rope_theta": cfg.theta}
    text = hf_cfg.Qwen2_5_VLTextConfig(hidden_size=cfg.hidden, intermediate_size=cfg.intermediate, num_hidden_layers=1,
                                       num_attention_heads=cfg.heads, num_key_value_heads=cfg.kv_heads, rms_norm_eps=cfg.eps,
                                       vocab_size=cfg.vocab, max_position_embeddings=512, rope_parameters=rope,
                                       rope_scaling=rope, rope_theta=cfg.theta)
    text._attn_implementation = "eager"
    layer = hf.Qwen2_5_VLDecoderLayer(text, layer_idx=0).float().eval()
    for name, p in layer.named_parameters():
        torch.nn.init.normal_(p, mean=1.0, std=0.1) if "norm" in name else torch.nn.init.normal_(p, std=0.05)
        if "q_proj.weight" in name or "k_proj.weight" in name:      # sharp attention, as above
            torch.nn.init.normal_(p, std=0.3)
    rotary = hf.Qwen2_5_VLRotaryEmbedding(config=text)

    S = cfg.tokens
    h = torch.randn(S, cfg.hidden, generator=torch.Generator().manual_seed(4))
    positions = qwen_vl.rope_positions(cfg)                                   # [3, S] int32, images first
    ids = positions.long()[:, None, :]                                        # [3, batch, S]
    cos, sin = rotary(h[None], ids)
    mask = torch.full((S, S), float("-inf")).triu(1)[None, None]
    with torch.no_grad():
        want = layer(h[None], attention_mask=mask, position_ids=ids, position_embeddings=(cos, sin))
    want = want[0] if isinstance(want, tuple) else want

    w: dict = {}
    l = "model.layers.0"
    w[f"{l}.input_layernorm.weight"] = layer.input_layernorm.weight.detach().clone()
    w[f"{l}.post_attention_layernorm.weight"] = layer.post_attention_layernorm.weight.detach().clone()
    for part in ("q_proj", "k_proj", "v_proj", "o_proj"):
        linear(w, f"{l}.self_attn.{part}", getattr(layer.self_attn, part))
    for part in ("gate_proj", "up_proj", "down_proj"):
        linear(w, f"{l}.mlp.{part}", getattr(layer.mlp, part))
    assert f"{l}.self_attn.q_proj.bias" in w and f"{l}.self_attn.o_proj.bias" not in w     # biases: q/k/v only
    got, _, _ = oracle_vl.decoder_layer(cfg, w, 0, h.bfloat16(), positions)
    close(got.float(), want.reshape(S, cfg.hidden), **BLOCK)

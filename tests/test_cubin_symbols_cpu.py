"""Every kernel a recipe names must be an entry point of the built CUBIN (the loader resolves them by name with
cuModuleGetFunction at the first Enqueue, so a typo would only show up on a GPU)."""
from __future__ import annotations

import dataclasses
import struct

import pytest

from aginfer_b200.build import build_all
from aginfer_b200.recipes import decoder_layer, dit, lingbot, qwen_vl
from tests.test_lingbot_cpu import table as episode_table
from tests.test_qwen_vl_cpu import table as prefill_table


def function_symbols(blob: bytes) -> set[str]:
    """Names of STT_FUNC symbols in an ELF64 little-endian image (the symbol table only; no code is read)."""
    assert blob[:4] == b"\x7fELF" and blob[4] == 2 and blob[5] == 1
    shoff, = struct.unpack_from("<Q", blob, 0x28)
    shentsize, shnum = struct.unpack_from("<HH", blob, 0x3A)
    sections = [struct.unpack_from("<IIQQQQIIQQ", blob, shoff + i * shentsize) for i in range(shnum)]
    names = set()
    for sh_name, sh_type, _, _, offset, size, link, _, _, entsize in sections:
        if sh_type != 2:      # SHT_SYMTAB
            continue
        str_off = sections[link][4]
        for at in range(offset, offset + size, entsize):
            st_name, st_info = struct.unpack_from("<IB", blob, at)
            if st_info & 0xF == 2:      # STT_FUNC
                end = blob.index(b"\0", str_off + st_name)
                names.add(blob[str_off + st_name:end].decode())
    return names


@pytest.fixture(scope="module")
def entry_points() -> set[str]:
    _, cubin = build_all()
    return function_symbols(cubin.read_bytes())


def recipes():
    yield "dit", dit.build_recipe(dit.DitConfig(), stream_profile=True)
    layer = decoder_layer.LayerConfig()
    for fp8 in (False, True):
        cfg = dataclasses.replace(layer, fp8=fp8)
        shapes = {}
        for name, (n, k) in decoder_layer.linear_shapes(cfg).items():
            shapes[f"model.layers.0.{name}.weight"] = ("F8_E4M3" if fp8 else "BF16", (n, k))
            if fp8:
                shapes[f"model.layers.0.{name}.weight_scale"] = ("F32", ())
        for p in ("q_proj", "k_proj", "v_proj"):
            shapes[f"model.layers.0.self_attn.{p}.bias"] = ("BF16", (decoder_layer.linear_shapes(cfg)[f"self_attn.{p}"][0],))
        shapes["model.layers.0.input_layernorm.weight"] = ("BF16", (cfg.hidden,))
        shapes["model.layers.0.post_attention_layernorm.weight"] = ("BF16", (cfg.hidden,))
        yield f"decoder_layer fp8={fp8}", decoder_layer.build_recipe(cfg, shapes)
    vl = qwen_vl.VlConfig()
    for packed in (False, True):
        yield f"qwen_vl packed={packed}", qwen_vl.build_recipe(vl, prefill_table(vl), packed=packed, trace=True)
    ep = lingbot.EpisodeConfig()
    yield "lingbot", lingbot.build_recipe(ep, episode_table(ep), packed=True)


def test_every_recipe_kernel_is_an_entry_point_of_the_cubin(entry_points):
    assert "vector_add_f32" in entry_points and len(entry_points) > 100
    for label, recipe in recipes():
        used = {l["kernel"] for p in recipe.plan()["shape_dispatch"] for l in p["launches"]}
        assert used <= entry_points, (label, sorted(used - entry_points))

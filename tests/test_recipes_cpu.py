"""Recipe builder and packaging on CPU: the artifact set compiles with modelc and loads through the C ABI."""
import json

import pytest
import torch

import aginfer_b200 as agi
from aginfer_b200 import runtime as rt
from aginfer_b200.build import build_all
from aginfer_b200.recipes import Arena, RecipeBuilder, Tensor, U32, Weight, io
from aginfer_b200.recipes.builder import RESERVED, TC_COUNTER_BYTES, TC_SCRATCH_BYTES
from aginfer_b200.recipes.package import build_aim, describe

OVERRIDES = dict(cuda_arch_override=100, cuda_driver_version_override=12080, cuda_runtime_version_override=12080,
                 cublaslt_abi_override=12, cudnn_abi_override=9)


@pytest.fixture(scope="module", autouse=True)
def built():
    build_all()


def small_recipe():
    weights = {"b.weight": torch.zeros(64, 32, dtype=torch.bfloat16), "a.scale": torch.ones((), dtype=torch.float32),
               "c.weight": torch.zeros(16, 32, dtype=torch.float8_e4m3fn)}
    r = RecipeBuilder(describe(weights))
    r.begin_profile("default", [io("x", "BF16", [4, 32])], [io("y", "BF16", [4, 64])])
    h = r.alloc(4 * 32 * 2)
    r.rmsnorm(Tensor("x"), Weight("b.weight"), h, 4, 32)
    r.gemm(h, Weight("b.weight"), Tensor("y"), 4, 64, 32)
    return weights, r


def test_weight_offsets_follow_name_order_and_alignment():
    weights, r = small_recipe()
    assert r.weight_offsets == {"a.scale": 0, "b.weight": 256, "c.weight": 256 + 4096}
    assert r.weight_bytes == 256 + 4096 + 512
    plan = r.plan()
    launches = plan["shape_dispatch"][0]["launches"]
    assert launches[0]["kernel"] == "agi_fill_u32" and launches[0]["arguments"][2] == {"scalar_u32": RESERVED // 4}
    assert {"weights_offset": 256} in launches[1]["arguments"]
    assert plan["arena_bytes"] % 256 == 0 and plan["arena_bytes"] >= RESERVED + 256
    with pytest.raises(KeyError):
        r.launch("k", (1, 1, 1), (1, 1, 1), [Weight("missing")])


def test_arena_stack_discipline():
    r = RecipeBuilder({"w": ("BF16", (8,))})
    a = r.alloc(1000)
    mark = r.mark()
    b = r.alloc(5000)
    r.release(mark)
    c = r.alloc(100)
    base = RESERVED + TC_SCRATCH_BYTES + TC_COUNTER_BYTES   # fixed regions come first
    assert a.offset == base and b.offset == c.offset == base + 1024
    assert r.arena_bytes == base + 1024 + 5120
    first, second = r.counter(), r.counter(2)
    assert (first.offset, second.offset) == (64, 68)


def test_packaged_recipe_loads_through_the_c_abi(tmp_path):
    weights, r = small_recipe()
    aim = build_aim(tmp_path, weights, r)
    info = agi.AimReader.read(aim)
    assert info.manifest["cuda_arches"] == ["sm100"] and info.manifest["checkpoint_dtypes"] == ["BF16", "F32", "F8_E4M3"]
    assert info.manifest["tactics"]["sm100"]["entry_count"] == 3
    assert [t["name"] for t in info.tensors["items"]] == ["a.scale", "b.weight", "c.weight"]
    assert [t["blob_offset"] for t in info.tensors["items"]] == [r.weight_offsets[k] for k in sorted(weights)]
    session = rt.Session.create(rt.Runtime.create(**OVERRIDES), rt.Model.load(aim))
    assert session.stats()["launches_per_enqueue"] == 3
    assert session.required_workspace()["arena_bytes"] == r.arena_bytes
    tactics = json.loads((tmp_path / "artifacts/sm100/tactics.json").read_text())
    assert {t["op"] for t in tactics["tactics"]} == {"prologue", "rmsnorm", "gemm_bf16"}


def test_cubin_exports_every_kernel_the_builder_names():
    from aginfer_b200.build import CUBIN
    blob = CUBIN.read_bytes()
    for name in ("vector_add_f32", "agi_fill_u32", "agi_absmax_bf16", "agi_quantize_e4m3_bf16", "agi_rmsnorm_bf16",
                 "agi_layernorm_bf16", "agi_rope_bf16", "agi_mrope_bf16", "agi_attention_bf16", "agi_swiglu_bf16",
                 "agi_gemm_simt_bf16", "agi_gemm_simt_e4m3", "agi_euler_step"):
        assert name.encode() + b"\0" in blob, name

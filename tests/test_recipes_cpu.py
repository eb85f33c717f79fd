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


def _kernels(body, weights=None):
    weights = weights or {"w": torch.zeros(4096, 4096, dtype=torch.bfloat16), "w2": torch.zeros(4096, 1024, dtype=torch.bfloat16)}
    r = RecipeBuilder(describe(weights))
    r.begin_profile("default", [io("x", "BF16", [64, 8192])], [io("y", "BF16", [64, 8192])])
    body(r)
    return r.plan()["shape_dispatch"][0]["launches"][1:]      # without the prologue


def test_launch_geometry_choices_for_few_tokens():
    """The builder's choices that the action head and the action expert rely on, as launch records."""
    from aginfer_b200.recipes.builder import stream_splits, stream_tiling, tc_cluster_tiling
    # a long K becomes four rings side by side in a cluster; a K that one ring covers in <= 4 chunks stays whole
    assert stream_splits(17, 1536, 6144, 2) == 4 and stream_splits(17, 6144, 1536, 2) == 1
    assert stream_splits(50, 1024, 4096, 2) == 1 and stream_splits(17, 1536, 6144, 1) == 1      # > 32 tokens; FP8
    t = stream_tiling(17, 1536, 6144, 2, splits=4)
    assert (t["rows"], t["grid"], t["slots"]) == (16, 96, 2) and 3 * t["shared_bytes"] <= 227 * 1024
    x, y = Tensor("x"), Tensor("y")
    (down,) = _kernels(lambda r: r.gemm(x, Weight("w"), y, 17, 1536, 4096 + 2048, ldx=8192))
    assert down["kernel"] == "agi_gemm_stream_bf16_t3_k4" and down["grid"] == [96, 1, 4]
    # projections that share their input: one grouped launch, K slices of every tile in a cluster when tokens are few
    parts = lambda r, n: [(Weight("w2"), None, None, y, n, 8192), (Weight("w2") + n * 2048, None, None, r.alloc(64 * 8192 * 2), n, 8192)]
    (few,) = _kernels(lambda r: r.gemm_group(x, parts(r, 1024), 50, 1024))
    (many,) = _kernels(lambda r: r.gemm_group(x, parts(r, 1024), 300, 1024))
    assert few["kernel"] == "agi_gemm_tc_bf16_x3_c8" and few["grid"] == [16, 1, 8]
    assert many["kernel"] == "agi_gemm_tc_bf16_x3" and many["grid"][2] == 1
    assert tc_cluster_tiling(50, 8192, 1024, 2, sizes=(2, 4, 8))["cluster"] == 2
    # few query rows: the key-split kernel, by head width; static keys / values are flagged in the mask word
    kw = dict(q_rows=50, kv_rows=306, q_heads=8, kv_heads=4, q_stride=1024, k_stride=512, v_stride=512, o_stride=1024)
    (wide,) = _kernels(lambda r: r.attention(x, x, x, y, head_dim=128, kv_static=True, kv_static_rows=256, **kw))
    assert wide["kernel"] == "agi_attention_mma_bf16_d128" and wide["grid"] == [8, 4, 1]
    assert wide["shared_bytes"] == 2 * 320 * 136 * 2 and wide["arguments"][14] == {"scalar_u32": 0x100 | (256 << 16)}
    kw.update(q_rows=17, kv_rows=300, q_heads=32, kv_heads=32, q_stride=1536, k_stride=1536, v_stride=1536, o_stride=1536)
    (narrow,) = _kernels(lambda r: r.attention(x, x, x, y, head_dim=48, **kw))
    assert narrow["kernel"] == "agi_attention_mma_bf16" and narrow["arguments"][14] == {"scalar_u32": 0}
    (streaming,) = _kernels(lambda r: r.attention(x, x, x, y, head_dim=128, **{**kw, "q_rows": 288, "kv_rows": 288, "q_heads": 16,
                                                                                "kv_heads": 2, "q_stride": 2048, "k_stride": 256,
                                                                                "v_stride": 256, "o_stride": 2048}))
    assert streaming["kernel"].startswith("agi_attention_fa_bf16_d128")

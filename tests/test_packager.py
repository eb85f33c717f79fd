"""Behavioural tests of the packager, following the reference's tests/test_{plan,aim,checkpoint,compiler}.py,
plus the sm100 target row that this backend adds."""
from __future__ import annotations

import json
import struct
from pathlib import Path

import pytest

import aginfer_b200 as agi
from aginfer_b200.target import cubin_is_arch_specific, cubin_targets


def fake_cubin(arch: int, new_flavour: bool = False) -> bytes:
    """A 64-byte ELF header that looks like a CUBIN for ``arch``."""
    head = bytearray(64)
    head[:9] = b"\x7fELF\x02\x01\x01" + (b"\x41\x08" if new_flavour else b"\x33\x07")
    struct.pack_into("<HHI", head, 16, 2, 190, 124)
    struct.pack_into("<I", head, 48, (0x06000002 | (arch << 8) | 0x8) if new_flavour else (arch | arch << 16))
    struct.pack_into("<H", head, 52, 64)
    return bytes(head)


def make_checkpoint(root: Path, model_type: str = "groot") -> Path:
    root.mkdir(parents=True)
    (root / "config.json").write_text(json.dumps(
        {"model_type": model_type, "architectures": [f"{model_type.title()}ForConditionalGeneration"]}))
    header = json.dumps({"layer.weight": {"dtype": "F16", "shape": [2, 2], "data_offsets": [0, 8]}},
                        separators=(",", ":")).encode()
    (root / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + bytes(range(8)))
    return root


def make_artifacts(root: Path, arches=("sm89",), new_flavour: bool = False) -> Path:
    root.mkdir(parents=True)
    (root / "toolchain.json").write_text(json.dumps({
        "cuda_driver_min": 12000, "cuda_runtime_min": 12000, "cuda_runtime_max": 12999, "cublaslt_abi": 12,
        "cudnn_abi": 9}))
    for arch in arches:
        folder = root / arch
        folder.mkdir()
        (folder / "kernels.cubin").write_bytes(fake_cubin(int(arch[2:]), new_flavour))
        (folder / "plan.json").write_text(json.dumps({
            "cuda_arch": arch, "arena_bytes": 4096, "workspace_bytes": 2048,
            "shape_dispatch": [{
                "profile": "default",
                "inputs": [{"name": "input_ids", "dtype": "I32", "shape": [1]},
                           {"name": "pixel_values", "dtype": "F16", "shape": [1]},
                           {"name": "state", "dtype": "F16", "shape": [1]}],
                "outputs": [{"name": "actions", "dtype": "F16", "shape": [1]}],
                "launches": [{"kernel": "noop", "grid": [1, 1, 1], "block": [1, 1, 1], "arguments": []}]}],
            "cuda_graph_templates": [{"profile": "default"}]}))
        (folder / "tactics.json").write_text(json.dumps(
            {"cuda_arch": arch, "tactics": [{"op": "gemm", "algorithm": "verified-1"}]}))
    return root


def make_profile(path: Path) -> Path:
    bounds = {"min": 1, "opt": 2, "max": 4}
    fields = ("sequence_length", "image_height", "image_width", "image_count", "state_length", "action_horizon")
    path.write_text(json.dumps({"profiles": [{"name": "default", "batch": 1, **{f: bounds for f in fields}}],
                                "default_denoising": {"steps": 4}}))
    return path


def _options(root: Path, arches, **kw):
    return agi.CompileOptions(source=str(root / "checkpoint"), revision=None, adapter="groot_n1_5",
                              platform=agi.Platform.LINUX_X86_64_GNU, cuda_arches=tuple(arches),
                              profile_path=root / "profile.json", artifact_dir=root / "artifacts",
                              output=root / "model.aim", offline=True, **kw)


def test_arch_parsing_accepts_feature_suffix():
    for text in ("sm100", "sm_100", "sm100a", "SM_100a", "100", "sm100f"):
        assert agi.CudaArch.parse(text) is agi.CudaArch.SM100
    assert agi.CudaArch.parse("sm_89") is agi.CudaArch.SM89
    with pytest.raises(ValueError):
        agi.CudaArch.parse("sm90")
    assert agi.CudaArch.SM100.name_string == "sm100"
    agi.validate_target(agi.Platform.LINUX_X86_64_GNU, [agi.CudaArch.SM100])
    with pytest.raises(ValueError, match="not supported"):
        agi.validate_target(agi.Platform.LINUX_AARCH64_SBSA, [agi.CudaArch.SM100])


def test_cubin_flavours():
    assert cubin_targets(fake_cubin(89)) == {89}
    assert cubin_targets(fake_cubin(100, True)) == {100}
    assert cubin_is_arch_specific(fake_cubin(100, True))
    # a new-flavour sm_120 image must not pass for sm100 through its low flag byte
    assert 100 not in cubin_targets(fake_cubin(120, True))
    assert cubin_targets(b"\0" * 64) is None


def test_round_trip_multi_arch_and_weight_sharing(tmp_path):
    plan = b"p" * 10
    info = agi.AimWriter.write(
        tmp_path / "m.aim", platform=agi.Platform.LINUX_X86_64_GNU, manifest={"runtime_abi": 1}, graph={"opset": 1},
        tensors={"count": 0},
        variants=[agi.VariantPayload(agi.CudaArch.SM100, fake_cubin(100, True), b"shared weights", plan),
                  agi.VariantPayload(agi.CudaArch.SM89, fake_cubin(89), b"shared weights", plan)])
    assert [v.arch for v in info.variants] == [agi.CudaArch.SM89, agi.CudaArch.SM100]
    assert info.variants[0].weights.offset == info.variants[1].weights.offset
    assert info.variants[0].plan.offset == info.variants[1].plan.offset
    assert info.select_variant(agi.CudaArch.SM100).arch is agi.CudaArch.SM100
    with pytest.raises(agi.CompatibilityError):
        info.select_variant(agi.CudaArch.SM120)


def test_single_byte_corruption_is_caught(tmp_path):
    path = tmp_path / "m.aim"
    info = agi.AimWriter.write(path, platform=agi.Platform.LINUX_X86_64_GNU, manifest={}, graph={}, tensors={},
                               variants=[agi.VariantPayload(agi.CudaArch.SM100, fake_cubin(100, True), b"w", b"p")])
    raw = bytearray(path.read_bytes())
    raw[info.variants[0].kernels.offset] ^= 1
    path.write_bytes(raw)
    with pytest.raises(agi.FormatError, match="file checksum"):
        agi.AimReader.read(path)
    raw[info.variants[0].kernels.offset] ^= 1
    raw = raw[:-1]
    path.write_bytes(raw)
    with pytest.raises(agi.FormatError, match="file size mismatch"):
        agi.AimReader.read(path)


def test_wrong_arch_and_ptx_rejected(tmp_path):
    def write(kernels, arch=agi.CudaArch.SM100):
        agi.AimWriter.write(tmp_path / "x.aim", platform=agi.Platform.LINUX_X86_64_GNU, manifest={}, graph={},
                            tensors={}, variants=[agi.VariantPayload(arch, kernels, b"w", b"p")])
    with pytest.raises(agi.ValidationError, match="exact sm100"):
        write(fake_cubin(120, True))
    with pytest.raises(agi.ValidationError, match="PTX"):
        write(fake_cubin(100, True) + b"\n.target sm_100a\n")


def test_checkpoint_packs_without_casting(tmp_path):
    checkpoint = agi.load_checkpoint(str(make_checkpoint(tmp_path / "checkpoint")), offline=True)
    assert checkpoint.dtypes == {"F16"}
    blob, table = agi.pack_weights(checkpoint.tensors)
    assert blob == bytes(range(8))
    assert table[0]["dtype"] == "F16" and table[0]["stride"] == [2, 1]


def test_checkpoint_rejections(tmp_path):
    root = make_checkpoint(tmp_path / "a")
    (root / "pytorch_model.bin").write_bytes(b"pickle")
    with pytest.raises(agi.ValidationError, match="pickle"):
        agi.load_checkpoint(str(root))
    root = tmp_path / "b"
    root.mkdir()
    (root / "config.json").write_text('{"model_type":"groot"}')
    header = json.dumps({"bad": {"dtype": "I8", "shape": [1], "data_offsets": [0, 1]}}).encode()
    (root / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + b"x")
    with pytest.raises(agi.ValidationError, match="unsupported dtype"):
        agi.load_checkpoint(str(root))
    root = tmp_path / "c"
    root.mkdir()
    (root / "config.json").write_text('{"model_type":"groot"}')
    agi.write_safetensors(root / "model.safetensors", {"w": ("F8_E4M3", [4], b"\1\2\3\4")})
    with pytest.raises(agi.ValidationError, match="quantization_config"):
        agi.load_checkpoint(str(root))
    (root / "config.json").write_text(json.dumps({"model_type": "groot", "quantization_config": {
        "quant_method": "modelopt", "quantization_format": "fp8", "scales": "explicit"}}))
    assert agi.load_checkpoint(str(root)).dtypes == {"F8_E4M3"}


def test_weight_layout_matches_pack(tmp_path):
    root = tmp_path / "ck"
    root.mkdir()
    (root / "config.json").write_text('{"model_type":"groot"}')
    tensors = {"b.weight": ("BF16", [3, 5], bytes(30)), "a.scale": ("F32", [], b"\0\0\x80\x3f"),
               "c": ("F16", [200], bytes(range(200)) * 2)}
    agi.write_safetensors(root / "model.safetensors", tensors)
    blob, table = agi.pack_weights(agi.load_checkpoint(str(root)).tensors)
    offsets, total = agi.weight_layout({k: len(v[2]) for k, v in tensors.items()})
    assert total == len(blob)
    assert {t["name"]: t["blob_offset"] for t in table} == offsets == {"a.scale": 0, "b.weight": 256, "c": 512}
    assert blob[512:912] == tensors["c"][2]


def test_compile_for_sm100(tmp_path):
    make_checkpoint(tmp_path / "checkpoint")
    make_profile(tmp_path / "profile.json")
    make_artifacts(tmp_path / "artifacts", ("sm100",), new_flavour=True)
    info = agi.compile_model(_options(tmp_path, (agi.CudaArch.SM100,)))
    assert info.manifest["cuda_arches"] == ["sm100"]
    assert info.manifest["checkpoint_dtypes"] == ["F16"]
    assert info.manifest["deployment_features"] == {"ptx": False, "jit": False, "autotune": False,
                                                    "runtime_weight_repacking": False, "cpu_fallback": False}
    variant = info.variants[0]
    raw = (tmp_path / "model.aim").read_bytes()
    summary = agi.inspect_plan(raw[variant.plan.offset: variant.plan.offset + variant.plan.size])
    assert summary["arch"] == 100 and summary["launch_count"] == 1


def test_missing_artifact_fails_closed(tmp_path):
    make_checkpoint(tmp_path / "checkpoint")
    make_profile(tmp_path / "profile.json")
    artifacts = make_artifacts(tmp_path / "artifacts", ("sm100",), new_flavour=True)
    (artifacts / "sm100" / "tactics.json").unlink()
    with pytest.raises(agi.ValidationError, match="tactic database"):
        agi.compile_model(_options(tmp_path, (agi.CudaArch.SM100,)))


def test_cli_round_trip(tmp_path, capsys):
    from aginfer_b200.modelc import main
    make_checkpoint(tmp_path / "checkpoint")
    make_profile(tmp_path / "profile.json")
    make_artifacts(tmp_path / "artifacts", ("sm100",), new_flavour=True)
    code = main(["compile", "--source", str(tmp_path / "checkpoint"), "--adapter", "groot_n1_5", "--platform",
                 "linux-x86_64-gnu", "--cuda-arch", "sm100a", "--profile", str(tmp_path / "profile.json"),
                 "--artifact-dir", str(tmp_path / "artifacts"), "--offline", "--output", str(tmp_path / "m.aim")])
    assert code == 0 and "wrote" in capsys.readouterr().out
    assert main(["inspect", str(tmp_path / "m.aim")]) == 0
    assert json.loads(capsys.readouterr().out)["cuda_arches"] == ["sm100"]
    assert main(["inspect", str(tmp_path / "missing.aim")]) == 2

"""The packager against outputs recorded from the reference (tests/golden/format_golden.json)."""
from __future__ import annotations

import hashlib
import json
import os
from pathlib import Path

import pytest

import aginfer_b200 as agi
from aginfer_b200.errors import AgInferError

GOLDEN = json.loads(Path(__file__).with_name("golden").joinpath("format_golden.json").read_text())
ERRORS = {"ValidationError": agi.ValidationError, "FormatError": agi.FormatError, "ValueError": ValueError}


def test_known_digests():
    # Values the survey of the reference recorded independently of the golden file.
    first = bytes.fromhex(GOLDEN["plans"][0]["hex"])
    assert len(first) == 767
    assert hashlib.sha256(first).hexdigest() == "5581782a901e7b6de25a3e88ed034911a9108c77f0b8c1373d3bd4e696028904"
    assert first.endswith(b"\0vector4\0input\0output\0copy_f32\0")
    fixture = bytes.fromhex(GOLDEN["runtime_fixture_hex"])
    assert len(fixture) == 4224
    assert hashlib.sha256(fixture).hexdigest() == "8f906684734e3f2241b9fb8e6358074d1090fee77105e3ee3cc395c4489074cc"


@pytest.mark.parametrize("case", GOLDEN["plans"], ids=lambda c: c["label"])
def test_plan_bytes_equal_reference(case):
    compiled = agi.compile_execution_plan(case["plan"], agi.CudaArch(case["arch"]), weight_size=case["weight_size"])
    assert compiled.data.hex() == case["hex"]
    # and the decoder inverts the encoder
    again = agi.compile_execution_plan(agi.decode_plan(compiled.data), agi.CudaArch(case["arch"]),
                                       weight_size=case["weight_size"])
    assert again.data == compiled.data


@pytest.mark.parametrize("case", GOLDEN["plan_errors"], ids=lambda c: c["label"])
def test_plan_rejections_equal_reference(case):
    with pytest.raises(ERRORS[case["error"]]) as caught:
        agi.compile_execution_plan(case["plan"], agi.CudaArch(case["arch"]), weight_size=case["weight_size"])
    assert str(caught.value) == case["message"]


def _write(case, path):
    return agi.AimWriter.write(
        path, platform=agi.Platform(case["platform"]), manifest=case["manifest"], graph=case["graph"],
        tensors=case["tensors"],
        variants=[agi.VariantPayload(agi.CudaArch(v["arch"]), bytes.fromhex(v["kernels"]), bytes.fromhex(v["weights"]),
                                     bytes.fromhex(v["plan"])) for v in case["variants"]])


@pytest.mark.parametrize("case", GOLDEN["aims"], ids=lambda c: c["label"])
def test_container_bytes_equal_reference(case, tmp_path):
    info = _write(case, tmp_path / "x.aim")
    assert (tmp_path / "x.aim").read_bytes().hex() == case["hex"]
    assert [int(v.arch) for v in info.variants] == sorted(v["arch"] for v in case["variants"])


@pytest.mark.parametrize("case", GOLDEN["aim_errors"], ids=lambda c: c["label"])
def test_container_rejections_equal_reference(case, tmp_path):
    with pytest.raises(ERRORS[case["error"]]) as caught:
        _write(case, tmp_path / "x.aim")
    assert str(caught.value) == case["message"]


def test_reader_accepts_reference_fixture(tmp_path):
    path = tmp_path / "test.aim"
    path.write_bytes(bytes.fromhex(GOLDEN["runtime_fixture_hex"]))
    info = agi.AimReader.read(path)
    assert [v.arch for v in info.variants] == [agi.CudaArch.SM89, agi.CudaArch.SM120]
    assert info.variants[0].weights.offset == info.variants[1].weights.offset == 1280
    assert info.variants[0].plan.offset == 1536 and info.variants[1].plan.offset == 2816
    assert info.file_sha256.startswith("29119ba4") and info.file_sha256.endswith("01a15a")


def _helpers(root: Path):
    """The same tiny checkpoint / artifacts / profile the reference's tests build (tests/helpers.py)."""
    from tests.test_packager import make_artifacts, make_checkpoint, make_profile
    make_checkpoint(root / "checkpoint")
    make_profile(root / "profile.json")
    make_artifacts(root / "artifacts", ("sm89", "sm120"))


def test_compile_model_equals_reference(tmp_path, monkeypatch):
    _helpers(tmp_path)
    monkeypatch.chdir(tmp_path)
    want = GOLDEN["compile_model"]
    checkpoint = agi.load_checkpoint("checkpoint", offline=True)
    assert checkpoint.revision == want["revision"]
    blob, table = agi.pack_weights(checkpoint.tensors)
    assert blob.hex() == want["blob_hex"] and table == want["table"]
    agi.compile_model(agi.CompileOptions(
        source="checkpoint", revision=None, adapter="groot_n1_5", platform=agi.Platform.LINUX_X86_64_GNU,
        cuda_arches=(agi.CudaArch.SM89, agi.CudaArch.SM120), profile_path=Path("profile.json"),
        artifact_dir=Path("artifacts"), output=Path("model.aim"), offline=True))
    assert Path("model.aim").read_bytes().hex() == want["aim_hex"]

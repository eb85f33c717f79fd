"""The native loader through its C ABI, against answers recorded from the reference's C++ runtime
(tests/golden/loader_golden.json) and, when it has been built, against the reference runtime itself."""
from __future__ import annotations

import ctypes
import hashlib
import json
import re
import subprocess
from pathlib import Path

import pytest

from aginfer_b200 import runtime as rt
from aginfer_b200.build import build_runtime
from tests.aim_mutations import cases

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = json.loads((ROOT / "tests/golden/loader_golden.json").read_text())
BASE = bytes.fromhex(json.loads((ROOT / "tests/golden/format_golden.json").read_text())["runtime_fixture_hex"])
REF_PROBE = ROOT / "oracle/_ref/ref_probe"
OVERRIDES = dict(cuda_driver_version_override=12080, cuda_runtime_version_override=12080, cublaslt_abi_override=12,
                 cudnn_abi_override=9)


@pytest.fixture(scope="module", autouse=True)
def library():
    build_runtime()
    return rt.load_library()


def probe(path: Path, arch: int, profile: str) -> list[str]:
    """The same report oracle/ref_probe.cc prints, produced through this library's C ABI."""
    lines = []

    def stage(name, fn):
        try:
            value = fn()
            lines.append(f"{name}=OK|")
            return value
        except rt.RuntimeStatusError as exc:
            lines.append(f"{name}={exc.name}|{str(exc).split(': ', 1)[1]}")
            return None

    model = stage("load", lambda: rt.Model.load(path))
    if model is None:
        return lines
    runtime = stage("runtime", lambda: rt.Runtime.create(cuda_arch_override=arch, **OVERRIDES))
    session = stage("session", lambda: rt.Session.create(runtime, model, profile))
    if session is None:
        return lines
    target = session.target_info()
    lines.append(f"target={target['platform']}|{target['cuda_arch']}|{target['runtime_abi']}")
    for kind, infos in (("input", session.input_info()), ("output", session.output_info())):
        for t in infos:
            dims = "".join(f"{v}," for v in t.shape)
            steps = "".join(f"{v}," for v in t.stride)
            lines.append(f"{kind}={t.name}|{rt.DTYPES[t.dtype]}|{t.location}|{t.byte_size}|{dims}|{steps}")
    ws = session.required_workspace()
    lines.append(f"workspace={ws['arena_bytes']}|{ws['workspace_bytes']}")
    stage("workspace_missing", lambda: session.required_workspace("no-such-profile"))
    return lines


MUTATIONS = {label: (arch, profile, data) for label, arch, profile, data in cases(BASE)}


@pytest.mark.parametrize("case", GOLDEN["mutations"], ids=lambda c: c["label"])
def test_mutated_package_matches_reference(case, tmp_path):
    arch, profile, data = MUTATIONS[case["label"]]
    assert hashlib.sha256(data).hexdigest() == case["sha256"], "mutation drifted from the recorded one"
    path = tmp_path / "case.aim"
    path.write_bytes(data)
    assert probe(path, arch, profile) == case["probe"]


@pytest.mark.parametrize("case", GOLDEN["plans"], ids=lambda c: c["label"])
def test_rich_plans_match_reference(case, tmp_path):
    path = tmp_path / "case.aim"
    path.write_bytes(bytes.fromhex(case["aim_hex"]))
    assert probe(path, case["arch"], case["profile"]) == case["probe"]


@pytest.mark.skipif(not REF_PROBE.exists(), reason="reference runtime not built (make -C oracle)")
def test_live_reference_agrees(tmp_path):
    for label, (arch, profile, data) in MUTATIONS.items():
        path = tmp_path / "case.aim"
        path.write_bytes(data)
        cmd = [str(REF_PROBE), str(path), str(arch)] + ([profile] if profile else [])
        want = subprocess.run(cmd, capture_output=True, text=True, check=True).stdout.splitlines()
        assert probe(path, arch, profile) == want, label


def test_missing_file_and_abi():
    with pytest.raises(rt.RuntimeStatusError) as caught:
        rt.Model.load("/nonexistent/model.aim")
    assert caught.value.name == "NOT_FOUND"
    with pytest.raises(rt.RuntimeStatusError) as caught:
        rt.Runtime.create(required_runtime_abi=2, cuda_arch_override=100, **OVERRIDES)
    assert caught.value.name == "INCOMPATIBLE_ABI"


def test_header_declares_exactly_the_exported_symbols(library):
    header = (ROOT / "include/aginfer_b200.h").read_text()
    declared = set(re.findall(r"^AGI_API [^;(]*?\b(agi_\w+)\(", header, flags=re.M))
    assert declared == set(rt.EXPORTS), declared ^ set(rt.EXPORTS)
    for name in declared:
        assert getattr(library, name) is not None
    nm = subprocess.run(["nm", "-D", "--defined-only", str(rt._LIB_PATH)], capture_output=True, text=True).stdout
    exported = set(re.findall(r"\b(agi_\w+)$", nm, flags=re.M))
    assert exported == declared


def test_sha256_backends_agree():
    for size in (0, 1, 55, 56, 63, 64, 65, 119, 120, 4096, 100003):
        data = bytes((i * 131 + size) & 0xFF for i in range(size))
        want = hashlib.sha256(data).digest()
        assert rt.sha256(data) == want and rt.sha256(data, portable=True) == want


def test_sm100_package_loads_and_reports(tmp_path):
    import aginfer_b200 as agi
    from tests.test_packager import fake_cubin
    plan = agi.compile_execution_plan({
        "cuda_arch": "sm100", "arena_bytes": 1024, "workspace_bytes": 0,
        "shape_dispatch": [{"profile": "p", "inputs": [{"name": "x", "dtype": "BF16", "shape": [17, 1536]}],
                            "outputs": [{"name": "y", "dtype": "F8_E4M3", "shape": [4, 8], "stride": [16, 1]}],
                            "launches": [{"kernel": "k", "grid": [148, 1, 1], "block": [256, 1, 1],
                                          "shared_bytes": 65536, "arguments": [{"tensor": "x"}, {"tensor": "y"}]}]}],
        "cuda_graph_templates": [{"profile": "p"}]}, agi.CudaArch.SM100, weight_size=8)
    manifest = {"toolchain": {"cuda_driver_min": 12080, "cuda_runtime_min": 12080, "cuda_runtime_max": 12999,
                              "cublaslt_abi": 12, "cudnn_abi": 9}}
    path = tmp_path / "m.aim"
    agi.AimWriter.write(path, platform=agi.Platform.LINUX_X86_64_GNU, manifest=manifest, graph={}, tensors={},
                        variants=[agi.VariantPayload(agi.CudaArch.SM100, fake_cubin(100, True), b"w" * 8, plan.data)])
    model = rt.Model.load(path)
    assert model.arches == [100]
    session = rt.Session.create(rt.Runtime.create(cuda_arch_override=100, **OVERRIDES), model)
    assert session.target_info()["cuda_arch"] == "sm100"
    (x,), (y,) = session.input_info(), session.output_info()
    assert (x.name, x.dtype, x.shape, x.stride, x.byte_size) == ("x", "BF16", (17, 1536), (1536, 1), 17 * 1536 * 2)
    assert (y.dtype, y.stride, y.byte_size) == ("F8_E4M3", (16, 1), 56)
    assert session.stats()["launches_per_enqueue"] == 1
    # argument validation happens before any CUDA call, so it is observable without a GPU
    buf = ctypes.create_string_buffer(17 * 1536 * 2)
    good = rt.TensorView("x", "BF16", (17, 1536), (1536, 1), ctypes.addressof(buf), len(buf))
    out = rt.TensorView("y", "F8_E4M3", (4, 8), (16, 1), ctypes.addressof(buf), 56)
    for bad, text in ((rt.TensorView("x", "BF16", (17, 1535), (1536, 1), good.data, good.byte_size), "shape or stride"),
                      (rt.TensorView("x", "F16", (17, 1536), (1536, 1), good.data, good.byte_size), "dtype or memory"),
                      (rt.TensorView("x", "BF16", (17, 1536), (1536, 1), good.data, 10), "byte size"),
                      (rt.TensorView("x", "BF16", (17, 1536), (1536, 1), 0, good.byte_size), "buffer"),
                      (rt.TensorView("z", "BF16", (17, 1536), (1536, 1), good.data, good.byte_size), "unexpected tensor")):
        with pytest.raises(rt.RuntimeStatusError, match=text) as caught:
            session.enqueue([bad], [out])
        assert caught.value.name == "INVALID_ARGUMENT"
    with pytest.raises(rt.RuntimeStatusError, match="count does not match"):
        session.enqueue([good, good], [out])
    with pytest.raises(rt.RuntimeStatusError, match="no exact sm120"):
        rt.Session.create(rt.Runtime.create(cuda_arch_override=120, **OVERRIDES), model)


def _steps_package(tmp_path):
    """A package whose plan carries a profile, two step-count siblings of it and one malformed sibling."""
    import aginfer_b200 as agi
    from tests.test_packager import fake_cubin
    io_in = [{"name": "state", "dtype": "BF16", "shape": [1, 64]}, {"name": "noise", "dtype": "BF16", "shape": [16, 32]}]
    io_out = [{"name": "actions", "dtype": "F32", "shape": [16, 32]}]
    launch = {"kernel": "k", "grid": [1, 1, 1], "block": [32, 1, 1], "arguments": [{"tensor": "noise"}, {"tensor": "actions"}]}

    def profile(name, launches, outputs=io_out):
        return {"profile": name, "inputs": io_in, "outputs": outputs, "launches": [launch] * launches}

    plan = agi.compile_execution_plan({
        "cuda_arch": "sm100", "arena_bytes": 1024, "workspace_bytes": 0,
        "shape_dispatch": [profile("default", 4), profile("default/steps=2", 2), profile("default/steps=8", 8),
                           profile("default/steps=3", 3, [{"name": "actions", "dtype": "F32", "shape": [8, 32]}]),
                           profile("other", 1),
                           {"profile": "plain", "inputs": io_in[:1], "outputs": io_out,
                            "launches": [{**launch, "arguments": [{"tensor": "state"}, {"tensor": "actions"}]}]}],
        "cuda_graph_templates": []}, agi.CudaArch.SM100, weight_size=8)
    manifest = {"toolchain": {"cuda_driver_min": 12080, "cuda_runtime_min": 12080, "cuda_runtime_max": 12999,
                              "cublaslt_abi": 12, "cudnn_abi": 9}}
    path = tmp_path / "steps.aim"
    agi.AimWriter.write(path, platform=agi.Platform.LINUX_X86_64_GNU, manifest=manifest, graph={}, tensors={},
                        variants=[agi.VariantPayload(agi.CudaArch.SM100, fake_cubin(100, True), b"w" * 8, plan.data)])
    return rt.Model.load(path)


def test_run_options_select_a_step_count_profile_and_override_the_noise(tmp_path):
    # reference: RunOptions (include/aginfer/runtime.h:84-90) are accepted and ignored (cpp/runtime.cc:499-500);
    # here denoising_steps and initial_noise_override select work.  Everything below is decided before the first
    # CUDA call, so it shows on a machine without a GPU: a call that passes validation ends in CUDA_ERROR here.
    model = _steps_package(tmp_path)
    session = rt.Session.create(rt.Runtime.create(cuda_arch_override=100, **OVERRIDES), model, "default")
    buf = ctypes.create_string_buffer(16 * 32 * 4)
    state = rt.TensorView("state", "BF16", (1, 64), (64, 1), ctypes.addressof(buf), 128)
    noise = rt.TensorView("noise", "BF16", (16, 32), (32, 1), ctypes.addressof(buf), 1024)
    actions = rt.TensorView("actions", "F32", (16, 32), (32, 1), ctypes.addressof(buf), 2048)

    def outcome(inputs, options):
        with pytest.raises(rt.RuntimeStatusError) as caught:
            session.enqueue(inputs, [actions], options=options)
        return caught.value.name, str(caught.value)

    assert outcome([state, noise], None)[0] == "CUDA_ERROR"                      # validated, then no driver
    assert session.stats()["launches_per_enqueue"] == 4
    assert outcome([state, noise], rt.run_options(2))[0] == "CUDA_ERROR"
    assert session.stats()["launches_per_enqueue"] == 2                          # the sibling profile was selected
    assert outcome([state, noise], rt.run_options(8, seed=7, deterministic=True))[0] == "CUDA_ERROR"
    assert session.stats()["launches_per_enqueue"] == 8
    name, text = outcome([state, noise], rt.run_options(5))
    assert name == "INVALID_ARGUMENT" and "no recipe for 5 denoising steps" in text and "default/steps=5" in text
    name, text = outcome([state, noise], rt.run_options(3))
    assert name == "CORRUPT_PACKAGE" and "does not have the tensors" in text
    assert outcome([state, noise], rt.run_options(0))[0] == "CUDA_ERROR"
    assert session.stats()["launches_per_enqueue"] == 4

    # the override stands in for "noise": with or without a "noise" among the inputs, under any name of its own
    override = rt.TensorView("whatever", "BF16", (16, 32), (32, 1), ctypes.addressof(buf), 1024)
    assert outcome([state], rt.run_options(0, override))[0] == "CUDA_ERROR"
    assert outcome([state, noise], rt.run_options(2, override))[0] == "CUDA_ERROR"
    # ... and is validated like any other view
    short = rt.TensorView("noise", "BF16", (8, 32), (32, 1), ctypes.addressof(buf), 1024)
    name, text = outcome([state], rt.run_options(0, short))
    assert name == "INVALID_ARGUMENT" and "shape or stride" in text
    name, text = outcome([state], None)
    assert name == "INVALID_ARGUMENT" and "count does not match" in text
    # a profile without step-count siblings, or without an input named "noise", says so
    other = rt.Session.create(rt.Runtime.create(cuda_arch_override=100, **OVERRIDES), model, "other")
    with pytest.raises(rt.RuntimeStatusError, match="no recipe for 2 denoising steps"):
        other.enqueue([state, noise], [actions], options=rt.run_options(2))
    plain = rt.Session.create(rt.Runtime.create(cuda_arch_override=100, **OVERRIDES), model, "plain")
    with pytest.raises(rt.RuntimeStatusError, match="no input named noise"):
        plain.enqueue([state], [actions], options=rt.run_options(0, override))

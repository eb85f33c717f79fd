"""Record what the reference's C++ runtime answers for each file of tests/aim_mutations.py.

    make -C oracle REF=/path/to/AgInfer && python tests/golden/make_loader_golden.py

Runs ``oracle/_ref/ref_probe`` (the reference runtime, linked from its own sources) on
every case and writes ``loader_golden.json``: label, SHA-256 of the mutated file, and the
probe's output lines.  A second section does the same for richer plans (every argument
kind, strides, several profiles) compiled by this repository's packager.
"""
from __future__ import annotations

import hashlib
import json
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from tests.aim_mutations import cases  # noqa: E402


def probe(data: bytes, arch: int, profile: str) -> list[str]:
    with tempfile.TemporaryDirectory() as tmp:
        path = Path(tmp) / "case.aim"
        path.write_bytes(data)
        cmd = [str(ROOT / "oracle" / "_ref" / "ref_probe"), str(path), str(arch)] + ([profile] if profile else [])
        done = subprocess.run(cmd, capture_output=True, text=True, check=True)
    return done.stdout.splitlines()


def main() -> int:
    golden = json.loads((ROOT / "tests" / "golden" / "format_golden.json").read_text())
    base = bytes.fromhex(golden["runtime_fixture_hex"])
    out = {"mutations": [], "plans": []}
    for label, arch, profile, data in cases(base):
        out["mutations"].append({"label": label, "arch": arch, "profile": profile,
                                 "sha256": hashlib.sha256(data).hexdigest(), "probe": probe(data, arch, profile)})
    for case in golden["aims"][:1]:
        pass
    import aginfer_b200 as agi
    from tests.test_packager import fake_cubin
    for case in golden["plans"]:
        arch = case["arch"]
        plan = agi.compile_execution_plan(case["plan"], agi.CudaArch(arch), weight_size=case["weight_size"]).data
        manifest = {"toolchain": {"cuda_driver_min": 12000, "cuda_runtime_min": 12000, "cuda_runtime_max": 12999,
                                  "cublaslt_abi": 12, "cudnn_abi": 9}}
        with tempfile.TemporaryDirectory() as tmp:
            path = Path(tmp) / "p.aim"
            agi.AimWriter.write(path, platform=agi.Platform.LINUX_X86_64_GNU, manifest=manifest, graph={}, tensors={},
                                variants=[agi.VariantPayload(agi.CudaArch(arch), fake_cubin(arch),
                                                             b"w" * case["weight_size"], plan)])
            data = path.read_bytes()
        for profile in [d["profile"] for d in case["plan"]["shape_dispatch"]]:
            out["plans"].append({"label": f"{case['label']} / {profile}", "arch": arch, "profile": profile,
                                 "aim_hex": data.hex(), "probe": probe(data, arch, profile)})
    target = Path(__file__).with_name("loader_golden.json")
    target.write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(f"wrote {target}: {len(out['mutations'])} mutations, {len(out['plans'])} plan cases")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

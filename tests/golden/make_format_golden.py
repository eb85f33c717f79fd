"""Generate ``format_golden.json`` by running the reference packager on fixed inputs.

Run where the reference checkout is available:

    python tests/golden/make_format_golden.py /path/to/AgInfer

It imports the reference's ``aginfer`` package and its test helpers, feeds them the cases
below (the reference's own test inputs plus variations) and records inputs and the exact
bytes / messages produced.  The committed JSON is what the CPU tests compare this
repository's packager against; nothing at test time needs the reference.
"""
from __future__ import annotations

import copy
import json
import os
import sys
import tempfile
from pathlib import Path


def main() -> int:
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_format_golden.py /path/to/AgInfer")
    ref = Path(sys.argv[1])
    sys.path[:0] = [str(ref / "src"), str(ref)]
    from aginfer.aim import AimWriter, VariantPayload
    from aginfer.checkpoint import load_checkpoint, pack_weights
    from aginfer.compiler import CompileOptions, compile_model
    from aginfer.errors import AgInferError
    from aginfer.plan import compile_execution_plan
    from aginfer.schema import CudaArch, Platform
    from tests.helpers import create_artifacts, create_checkpoint, create_profile, fake_cubin
    from tests.test_plan import _plan

    out: dict = {"plans": [], "plan_errors": [], "aims": [], "aim_errors": []}

    def plan_case(label, plan, arch, weight_size):
        try:
            data = compile_execution_plan(plan, CudaArch(arch), weight_size=weight_size).data
            out["plans"].append({"label": label, "plan": plan, "arch": arch, "weight_size": weight_size,
                                 "hex": data.hex()})
        except AgInferError as exc:
            out["plan_errors"].append({"label": label, "plan": plan, "arch": arch, "weight_size": weight_size,
                                       "error": type(exc).__name__, "message": str(exc)})

    base = _plan()
    plan_case("reference test plan", base, 89, 64)
    rich = copy.deepcopy(base)
    rich["cuda_arch"] = "sm120"
    rich["arena_bytes"] = 1 << 20
    rich["shape_dispatch"].append({
        "profile": "second",
        "inputs": [{"name": "a", "dtype": "BF16", "shape": [3, 5], "stride": [8, 1]},
                   {"name": "ids", "dtype": "I32", "shape": [7], "location": "host"},
                   {"name": "q", "dtype": "F8_E4M3", "shape": [2, 3, 4], "byte_size": 64}],
        "outputs": [{"name": "y", "dtype": "F16", "shape": [1, 1, 1, 1, 1, 1, 1, 2]}],
        "launches": [
            {"kernel": "k1", "grid": [148, 2, 1], "block": [128, 4, 2], "shared_bytes": 49152,
             "arguments": [{"tensor": "a"}, {"scalar_f32": 0.125}, {"scalar_f32": -3}, {"scalar_u32": 4294967295},
                           {"arena_offset": 1048575}, {"weights_offset": 4095}, {"tensor": "y"}]},
            {"kernel": "copy_f32", "grid": [1, 1, 1], "block": [1, 1, 1]},
            {"kernel": "kérnel", "grid": [4294967295, 1, 1], "block": [1, 1, 1024], "arguments": [{"tensor": "q"}]},
        ]})
    rich["cuda_graph_templates"] = [{"profile": "second"}]
    plan_case("two profiles, every argument kind, strides, host tensor", rich, 120, 4096)

    def broken(label, edit, arch=89, weight_size=64, source=base):
        plan = copy.deepcopy(source)
        edit(plan)
        plan_case(label, plan, arch, weight_size)

    d0 = lambda p: p["shape_dispatch"][0]
    l0 = lambda p: d0(p)["launches"][0]
    broken("unknown tensor", lambda p: l0(p)["arguments"].__setitem__(0, {"tensor": "missing"}))
    broken("host tensor argument", lambda p: d0(p)["inputs"][0].__setitem__("location", "host"))
    broken("oversized block", lambda p: l0(p).__setitem__("block", [1024, 2, 1]))
    broken("wrong arch string", lambda p: p.__setitem__("cuda_arch", "sm120"))
    broken("arena offset out of range", lambda p: l0(p)["arguments"].__setitem__(3, {"arena_offset": 256}))
    broken("weights offset out of range", lambda p: l0(p)["arguments"].__setitem__(4, {"weights_offset": 64}))
    broken("two kinds in one argument", lambda p: l0(p)["arguments"].__setitem__(2, {"scalar_u32": 1, "scalar_f32": 1.0}))
    broken("non-finite scalar", lambda p: l0(p)["arguments"].__setitem__(2, {"scalar_f32": float("inf")}))
    broken("scalar beyond fp32", lambda p: l0(p)["arguments"].__setitem__(2, {"scalar_f32": 1e39}))
    broken("bool scalar", lambda p: l0(p)["arguments"].__setitem__(2, {"scalar_u32": True}))
    broken("unknown kind", lambda p: l0(p)["arguments"].__setitem__(2, {"scalar_i32": 1}))
    broken("zero grid", lambda p: l0(p).__setitem__("grid", [0, 1, 1]))
    broken("grid rank", lambda p: l0(p).__setitem__("grid", [1, 1]))
    broken("empty kernel name", lambda p: l0(p).__setitem__("kernel", ""))
    broken("duplicate tensor", lambda p: d0(p)["outputs"][0].__setitem__("name", "input"))
    broken("duplicate profile", lambda p: p["shape_dispatch"].append(copy.deepcopy(d0(p))))
    broken("no outputs", lambda p: d0(p).__setitem__("outputs", []))
    broken("no launches", lambda p: d0(p).__setitem__("launches", []))
    broken("bad dtype", lambda p: d0(p)["inputs"][0].__setitem__("dtype", "I8"))
    broken("rank 9", lambda p: d0(p)["inputs"][0].__setitem__("shape", [1] * 9))
    broken("zero extent", lambda p: d0(p)["inputs"][0].__setitem__("shape", [0]))
    broken("stride rank", lambda p: d0(p)["inputs"][0].__setitem__("stride", [1, 1]))
    broken("byte_size too small", lambda p: d0(p)["inputs"][0].__setitem__("byte_size", 15))
    broken("graph template unknown", lambda p: p.__setitem__("cuda_graph_templates", [{"profile": "nope"}]))
    broken("graph template duplicate", lambda p: p.__setitem__("cuda_graph_templates", [{"profile": "vector4"}] * 2))
    broken("graph templates missing", lambda p: p.pop("cuda_graph_templates"))
    broken("arena missing", lambda p: p.pop("arena_bytes"))
    broken("negative workspace", lambda p: p.__setitem__("workspace_bytes", -1))
    broken("shared too large", lambda p: l0(p).__setitem__("shared_bytes", 2**32))
    broken("no graph template is fine", lambda p: p.__setitem__("cuda_graph_templates", []))

    manifest = {"runtime_abi": 1, "toolchain": {"cuda_driver_min": 12000, "cuda_runtime_min": 12000,
                                                "cuda_runtime_max": 12999, "cublaslt_abi": 12, "cudnn_abi": 9}}

    def aim_case(label, platform, manifest, graph, tensors, variants):
        record = {"label": label, "platform": platform, "manifest": manifest, "graph": graph, "tensors": tensors,
                  "variants": [{"arch": a, "kernels": k.hex(), "weights": w.hex(), "plan": p.hex()}
                               for a, k, w, p in variants]}
        with tempfile.TemporaryDirectory() as tmp:
            path = Path(tmp) / "x.aim"
            try:
                AimWriter.write(path, platform=Platform(platform), manifest=manifest, graph=graph, tensors=tensors,
                                variants=[VariantPayload(CudaArch(a), k, w, p) for a, k, w, p in variants])
                record["hex"] = path.read_bytes().hex()
                out["aims"].append(record)
            except (AgInferError, ValueError) as exc:
                record["error"] = type(exc).__name__
                record["message"] = str(exc)
                out["aim_errors"].append(record)

    tiny_plan = b'{"arena_bytes":1,"workspace_bytes":2}'
    aim_case("two arches sharing weights and plan", 1, manifest, {"opset": 1}, {"count": 0},
             [(89, fake_cubin("sm89"), b"shared weights", tiny_plan),
              (120, fake_cubin("sm120"), b"shared weights", tiny_plan)])
    aim_case("variants given out of order, non-ascii manifest", 1, {**manifest, "note": "café ☃"},
             {"opset": 1, "z": [1, 2], "a": None}, {"count": 0, "items": []},
             [(120, fake_cubin("sm120"), b"w" * 300, b"p" * 257), (89, fake_cubin("sm89"), b"w" * 256, b"p" * 257)])
    aim_case("aarch64 sm110", 2, manifest, {}, {}, [(110, fake_cubin("sm110"), b"w", b"p")])
    aim_case("ptx rejected", 1, {}, {}, {}, [(89, b".version 8.0\n.target sm_89", b"w", b"p")])
    aim_case("platform/arch pair rejected", 2, {}, {}, {}, [(89, fake_cubin("sm89"), b"w", b"p")])
    aim_case("wrong-arch cubin rejected", 1, {}, {}, {}, [(89, fake_cubin("sm120"), b"w", b"p")])
    aim_case("empty weights rejected", 1, {}, {}, {}, [(89, fake_cubin("sm89"), b"", b"p")])
    aim_case("duplicate arch rejected", 1, {}, {}, {}, [(89, fake_cubin("sm89"), b"w", b"p")] * 2)
    aim_case("not an ELF rejected", 1, {}, {}, {}, [(89, b"\0" * 64, b"w", b"p")])

    # The loader fixture of the reference's C++ test, and an end-to-end compile.
    with tempfile.TemporaryDirectory() as tmp:
        os.system(f"cd {ref} && PYTHONPATH={ref}/src {sys.executable} tests/make_runtime_fixture.py {tmp}/test.aim")
        out["runtime_fixture_hex"] = (Path(tmp) / "test.aim").read_bytes().hex()
    with tempfile.TemporaryDirectory() as tmp:
        here = os.getcwd()
        os.chdir(tmp)
        try:
            create_checkpoint(Path("checkpoint"))
            create_profile(Path("profile.json"))
            create_artifacts(Path("artifacts"), ("sm89", "sm120"))
            checkpoint = load_checkpoint("checkpoint", offline=True)
            blob, table = pack_weights(checkpoint.tensors)
            compile_model(CompileOptions(source="checkpoint", revision=None, adapter="groot_n1_5",
                                         platform=Platform.LINUX_X86_64_GNU,
                                         cuda_arches=(CudaArch.SM89, CudaArch.SM120),
                                         profile_path=Path("profile.json"), artifact_dir=Path("artifacts"),
                                         output=Path("model.aim"), offline=True))
            out["compile_model"] = {"revision": checkpoint.revision, "blob_hex": blob.hex(), "table": table,
                                    "aim_hex": Path("model.aim").read_bytes().hex()}
        finally:
            os.chdir(here)

    target = Path(__file__).with_name("format_golden.json")
    target.write_text(json.dumps(out, indent=1, ensure_ascii=True, sort_keys=True) + "\n")
    print(f"wrote {target}: {len(out['plans'])} plans, {len(out['plan_errors'])} plan errors, "
          f"{len(out['aims'])} aims, {len(out['aim_errors'])} aim errors")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())

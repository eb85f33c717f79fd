"""``plan.json`` -> binary ``AIMPLN1`` execution plan, and its decoder.

The wire format is the one the reference's loader parses (``cpp/plan.h:26-95``) and its
compiler emits (``src/aginfer/plan.py:62-214``): a 128-byte header, then the profile
(64 B), tensor (160 B), launch (64 B) and argument (32 B) tables back to back, then a
NUL-separated string table whose offset 0 is the empty string.  ``compile_execution_plan``
produces byte-identical output to the reference for every plan the reference accepts and
refuses what it refuses (same messages for the cases its tests pin, ``tests/test_plan.py``).

Design differences from the reference implementation: records are described once as
``Record`` layouts that both the encoder and ``decode_plan`` use, so the recipe generators
and the tests can read a compiled plan back instead of re-deriving offsets.
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass
from typing import Any, Sequence

from .errors import FormatError, ValidationError
from .target import CudaArch

PLAN_MAGIC = b"AIMPLN1\0"
MAX_TENSOR_RANK = 8

DTYPE_IDS = {"F32": 1, "F16": 2, "BF16": 3, "F8_E4M3": 4, "I32": 5}
DTYPE_SIZES = {"F32": 4, "F16": 2, "BF16": 2, "F8_E4M3": 1, "I32": 4}
LOCATION_IDS = {"host": 1, "device": 2}
IO_IDS = {"input": 1, "output": 2}
ARG_IDS = {"tensor": 1, "scalar_u32": 2, "scalar_f32": 3, "arena_offset": 4, "weights_offset": 5}

_U32_MAX = 2**32 - 1
_U64_MAX = 2**64 - 1
_I64_MAX = 2**63 - 1


class Record:
    """A fixed-size little-endian record: field names plus a ``struct`` layout."""

    def __init__(self, layout: str, names: Sequence[str]):
        self.codec = struct.Struct("<" + layout)
        self.names = tuple(names)
        self.size = self.codec.size

    def pack(self, *values: Any) -> bytes:
        return self.codec.pack(*values)

    def unpack(self, data: bytes, offset: int) -> tuple:
        return self.codec.unpack_from(data, offset)


HEADER = Record(
    "8sHHIIIIIIIQQQQQQQQ24s",
    ("magic", "schema_major", "schema_minor", "header_size", "arch", "profile_count",
     "tensor_count", "launch_count", "argument_count", "string_bytes", "arena_bytes",
     "workspace_bytes", "profiles_offset", "tensors_offset", "launches_offset",
     "arguments_offset", "strings_offset", "file_size", "reserved"),
)
PROFILE = Record("6I40s", ("name", "first_tensor", "tensor_count", "first_launch", "launch_count", "flags", "reserved"))
TENSOR = Record("6IQ8q8q", ("name", "dtype", "location", "io_kind", "rank", "flags", "byte_size"))
LAUNCH = Record("12I16s", ("kernel", "profile", "first_argument", "argument_count"))
ARGUMENT = Record("IIQQQ", ("kind", "index", "offset", "value", "reserved"))
assert (HEADER.size, PROFILE.size, TENSOR.size, LAUNCH.size, ARGUMENT.size) == (128, 64, 160, 64, 32)


@dataclass(frozen=True)
class CompiledPlan:
    data: bytes
    profiles: tuple[str, ...]
    input_names: tuple[str, ...]
    output_names: tuple[str, ...]
    launch_count: int


class _Strings:
    def __init__(self) -> None:
        self.blob = bytearray(b"\0")
        self.index: dict[str, int] = {}

    def intern(self, text: Any, label: str) -> int:
        if not isinstance(text, str) or not text or "\0" in text:
            raise ValidationError(f"{label} must be a non-empty string without NUL bytes")
        raw = text.encode("utf-8")
        if len(raw) > 4096:
            raise ValidationError(f"{label} is too long")
        at = self.index.get(text)
        if at is None:
            at = self.index[text] = len(self.blob)
            self.blob += raw + b"\0"
        return at


def _uint(value: Any, label: str, limit: int = _U64_MAX) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ValidationError(f"{label} must be an unsigned integer")
    if not 0 <= value <= limit:
        raise ValidationError(f"{label} must be an unsigned integer no greater than {limit}")
    return value


def _posint(value: Any, label: str, limit: int = _I64_MAX) -> int:
    number = _uint(value, label, limit)
    if number == 0:
        raise ValidationError(f"{label} must be positive")
    return number


def _dim3(value: Any, label: str) -> tuple[int, int, int]:
    if not isinstance(value, list) or len(value) != 3:
        raise ValidationError(f"{label} must contain exactly three dimensions")
    return tuple(_posint(v, label, _U32_MAX) for v in value)  # type: ignore[return-value]


def contiguous_stride(shape: Sequence[int]) -> tuple[int, ...]:
    out, run = [], 1
    for extent in reversed(shape):
        out.append(run)
        run *= extent
    return tuple(reversed(out))


def required_bytes(shape: Sequence[int], stride: Sequence[int], itemsize: int) -> int:
    return (sum((n - 1) * s for n, s in zip(shape, stride)) + 1) * itemsize


def _tensor_record(spec: Any, io_kind: str, strings: _Strings, label: str) -> tuple:
    if not isinstance(spec, dict):
        raise ValidationError(f"{label} must be an object")
    name = strings.intern(spec.get("name"), f"{label}.name")
    dtype = spec.get("dtype")
    if dtype not in DTYPE_IDS:
        raise ValidationError(f"{label}.dtype must be one of {', '.join(DTYPE_IDS)}")
    location = spec.get("location", "device")
    if location not in LOCATION_IDS:
        raise ValidationError(f"{label}.location must be host or device")
    raw_shape = spec.get("shape")
    if not isinstance(raw_shape, list) or not 1 <= len(raw_shape) <= MAX_TENSOR_RANK:
        raise ValidationError(f"{label}.shape must contain 1 to {MAX_TENSOR_RANK} dimensions")
    shape = tuple(_posint(v, f"{label}.shape") for v in raw_shape)
    raw_stride = spec.get("stride")
    if raw_stride is None:
        stride = contiguous_stride(shape)
    else:
        if not isinstance(raw_stride, list) or len(raw_stride) != len(shape):
            raise ValidationError(f"{label}.stride must have the same rank as shape")
        stride = tuple(_posint(v, f"{label}.stride") for v in raw_stride)
    needed = required_bytes(shape, stride, DTYPE_SIZES[dtype])
    byte_size = _uint(spec.get("byte_size", needed), f"{label}.byte_size")
    if byte_size < needed:
        raise ValidationError(f"{label}.byte_size is smaller than the declared shape and stride")
    pad = (0,) * (MAX_TENSOR_RANK - len(shape))
    return (name, DTYPE_IDS[dtype], LOCATION_IDS[location], IO_IDS[io_kind], len(shape), 0,
            byte_size, *shape, *pad, *stride, *pad)


def _argument_record(arg: Any, tensors: dict[str, int], on_device: set[str],
                     arena_bytes: int, weight_size: int, label: str) -> tuple:
    if not isinstance(arg, dict) or len(arg) != 1:
        raise ValidationError(f"{label} must contain exactly one argument kind")
    (kind, raw), = arg.items()
    if kind not in ARG_IDS:
        raise ValidationError(f"{label} has unsupported kind {kind!r}")
    code = ARG_IDS[kind]
    if kind == "tensor":
        if raw not in tensors:
            raise ValidationError(f"{label} references unknown tensor {raw!r}")
        if raw not in on_device:
            raise ValidationError(f"{label} references a host tensor; Kernel arguments must be device tensors")
        return (code, tensors[raw], 0, 0, 0)
    if kind == "scalar_u32":
        return (code, 0, 0, _uint(raw, label, _U32_MAX), 0)
    if kind == "scalar_f32":
        if isinstance(raw, bool) or not isinstance(raw, (int, float)) or not math.isfinite(raw):
            raise ValidationError(f"{label} must be a finite float")
        try:
            bits = struct.unpack("<I", struct.pack("<f", float(raw)))[0]
        except OverflowError as exc:
            raise ValidationError(f"{label} is outside the FP32 range") from exc
        return (code, 0, 0, bits, 0)
    offset = _uint(raw, label)
    limit = arena_bytes if kind == "arena_offset" else weight_size
    if offset >= limit:
        raise ValidationError(f"{label} offset {offset} is outside its {limit}-byte allocation")
    return (code, 0, offset, 0, 0)


def _graph_profiles(value: Any, dispatches: list[Any]) -> set[str]:
    if not isinstance(value, list):
        raise ValidationError("cuda_graph_templates must be a list")
    known = {d.get("profile") for d in dispatches if isinstance(d, dict) and isinstance(d.get("profile"), str)}
    chosen: set[str] = set()
    for i, item in enumerate(value):
        if not isinstance(item, dict) or item.get("profile") not in known:
            raise ValidationError(f"cuda_graph_templates[{i}] references an unknown profile")
        if item["profile"] in chosen:
            raise ValidationError(f"duplicate CUDA Graph template for profile {item['profile']}")
        chosen.add(item["profile"])
    return chosen


def compile_execution_plan(plan: dict[str, Any], arch: CudaArch, *, weight_size: int) -> CompiledPlan:
    """Validate ``plan`` and serialise it for ``arch`` (replaces ``plan.py:62-214``)."""
    if not isinstance(plan, dict):
        raise ValidationError("execution plan must be an object")
    if plan.get("cuda_arch") != arch.name_string:
        raise ValidationError(f"execution plan target must be exactly {arch.name_string}")
    arena_bytes = _uint(plan.get("arena_bytes"), "arena_bytes")
    workspace_bytes = _uint(plan.get("workspace_bytes"), "workspace_bytes")
    dispatches = plan.get("shape_dispatch")
    if not isinstance(dispatches, list) or not dispatches:
        raise ValidationError("execution plan needs a non-empty shape_dispatch list")
    graph_profiles = _graph_profiles(plan.get("cuda_graph_templates"), dispatches)

    strings = _Strings()
    profiles, tensors, launches, arguments = bytearray(), bytearray(), bytearray(), bytearray()
    n_tensors = n_launches = n_arguments = 0
    profile_names: list[str] = []
    first_io: tuple[tuple[str, ...], tuple[str, ...]] = ((), ())

    for p_index, dispatch in enumerate(dispatches):
        if not isinstance(dispatch, dict):
            raise ValidationError(f"shape_dispatch[{p_index}] must be an object")
        profile = dispatch.get("profile")
        p_name = strings.intern(profile, f"shape_dispatch[{p_index}].profile")
        if profile in profile_names:
            raise ValidationError(f"duplicate execution profile: {profile}")
        profile_names.append(profile)

        first_tensor = n_tensors
        by_name: dict[str, int] = {}
        on_device: set[str] = set()
        io_names: dict[str, list[str]] = {"input": [], "output": []}
        for key, io_kind in (("inputs", "input"), ("outputs", "output")):
            specs = dispatch.get(key)
            if not isinstance(specs, list) or not specs:
                raise ValidationError(f"profile {profile}: {key} must be a non-empty list")
            for i, spec in enumerate(specs):
                record = _tensor_record(spec, io_kind, strings, f"profile {profile} {key}[{i}]")
                name = spec["name"]
                if name in by_name:
                    raise ValidationError(f"profile {profile}: duplicate tensor name {name}")
                by_name[name] = n_tensors
                if record[2] == LOCATION_IDS["device"]:
                    on_device.add(name)
                io_names[io_kind].append(name)
                tensors += TENSOR.pack(*record)
                n_tensors += 1
        if p_index == 0:
            first_io = (tuple(io_names["input"]), tuple(io_names["output"]))

        first_launch = n_launches
        specs = dispatch.get("launches")
        if not isinstance(specs, list) or not specs:
            raise ValidationError(f"profile {profile}: launches must be a non-empty list")
        for l_index, launch in enumerate(specs):
            where = f"profile {profile} launch {l_index}"
            if not isinstance(launch, dict):
                raise ValidationError(f"{where} must be an object")
            kernel = strings.intern(launch.get("kernel"), f"{where}.kernel")
            grid = _dim3(launch.get("grid"), f"{where}.grid")
            block = _dim3(launch.get("block"), f"{where}.block")
            if math.prod(block) > 1024:
                raise ValidationError(f"{where}: block has more than 1024 threads")
            shared = _uint(launch.get("shared_bytes", 0), "shared_bytes", _U32_MAX)
            args = launch.get("arguments", [])
            if not isinstance(args, list):
                raise ValidationError(f"{where}.arguments must be a list")
            first_argument = n_arguments
            for a_index, arg in enumerate(args):
                arguments += ARGUMENT.pack(*_argument_record(
                    arg, by_name, on_device, arena_bytes, weight_size, f"{where} argument {a_index}"))
                n_arguments += 1
            launches += LAUNCH.pack(kernel, p_index, first_argument, len(args), *grid, *block, shared, 0, b"\0" * 16)
            n_launches += 1
        profiles += PROFILE.pack(p_name, first_tensor, n_tensors - first_tensor, first_launch,
                                 n_launches - first_launch, 1 if profile in graph_profiles else 0, b"\0" * 40)

    at_profiles = HEADER.size
    at_tensors = at_profiles + len(profiles)
    at_launches = at_tensors + len(tensors)
    at_arguments = at_launches + len(launches)
    at_strings = at_arguments + len(arguments)
    total = at_strings + len(strings.blob)
    header = HEADER.pack(PLAN_MAGIC, 1, 0, HEADER.size, int(arch), len(profile_names), n_tensors, n_launches,
                         n_arguments, len(strings.blob), arena_bytes, workspace_bytes, at_profiles, at_tensors,
                         at_launches, at_arguments, at_strings, total, b"\0" * 24)
    data = b"".join((header, profiles, tensors, launches, arguments, strings.blob))
    assert len(data) == total
    return CompiledPlan(data, tuple(profile_names), first_io[0], first_io[1], n_launches)


def inspect_plan(data: bytes) -> dict[str, int]:
    """Check the fixed header and return its summary fields (``plan.py:217-238``)."""
    if len(data) < HEADER.size:
        raise FormatError("execution plan is smaller than its fixed header")
    head = dict(zip(HEADER.names, HEADER.unpack(data, 0)))
    if head["magic"] != PLAN_MAGIC:
        raise FormatError("bad AIM execution plan magic")
    if head["schema_major"] != 1 or head["header_size"] != HEADER.size:
        raise FormatError("unsupported AIM execution plan schema")
    if head["file_size"] != len(data):
        raise FormatError("execution plan size mismatch")
    if any(head["reserved"]):
        raise FormatError("non-zero execution plan reserved bytes")
    keep = ("arch", "profile_count", "tensor_count", "launch_count", "argument_count", "arena_bytes", "workspace_bytes")
    return {key: head[key] for key in keep}


_ID_TO = {
    "dtype": {v: k for k, v in DTYPE_IDS.items()},
    "location": {v: k for k, v in LOCATION_IDS.items()},
    "io": {v: k for k, v in IO_IDS.items()},
    "arg": {v: k for k, v in ARG_IDS.items()},
}


def decode_plan(data: bytes) -> dict[str, Any]:
    """Turn a binary plan back into the ``plan.json`` object it was compiled from.

    Defaults are made explicit (strides, byte sizes, ``shared_bytes``), so
    ``compile_execution_plan(decode_plan(x)) == x`` for every compiled plan ``x``.
    No counterpart in the reference; used by tests and by the recipe tooling.
    """
    head = dict(zip(HEADER.names, HEADER.unpack(data, 0)))
    inspect_plan(data)
    table = data[head["strings_offset"]: head["strings_offset"] + head["string_bytes"]]

    def text(at: int) -> str:
        return table[at: table.index(b"\0", at)].decode("utf-8")

    tensor_names: list[str] = []
    dispatches = []
    graph_templates = []
    for p in range(head["profile_count"]):
        name, t0, tn, l0, ln, flags, _ = PROFILE.unpack(data, head["profiles_offset"] + p * PROFILE.size)
        io: dict[str, list[dict[str, Any]]] = {"input": [], "output": []}
        for t in range(t0, t0 + tn):
            rec = TENSOR.unpack(data, head["tensors_offset"] + t * TENSOR.size)
            rank = rec[4]
            tensor_names.append(text(rec[0]))
            io[_ID_TO["io"][rec[3]]].append({
                "name": text(rec[0]), "dtype": _ID_TO["dtype"][rec[1]], "location": _ID_TO["location"][rec[2]],
                "shape": list(rec[7:7 + rank]), "stride": list(rec[15:15 + rank]), "byte_size": rec[6]})
        launches = []
        for l in range(l0, l0 + ln):
            rec = LAUNCH.unpack(data, head["launches_offset"] + l * LAUNCH.size)
            args = []
            for a in range(rec[2], rec[2] + rec[3]):
                kind, index, offset, value, _ = ARGUMENT.unpack(data, head["arguments_offset"] + a * ARGUMENT.size)
                key = _ID_TO["arg"][kind]
                if key == "tensor":
                    args.append({key: tensor_names[index]})
                elif key == "scalar_u32":
                    args.append({key: value})
                elif key == "scalar_f32":
                    args.append({key: struct.unpack("<f", struct.pack("<I", value))[0]})
                else:
                    args.append({key: offset})
            launches.append({"kernel": text(rec[0]), "grid": list(rec[4:7]), "block": list(rec[7:10]),
                             "shared_bytes": rec[10], "arguments": args})
        profile = text(name)
        dispatches.append({"profile": profile, "inputs": io["input"], "outputs": io["output"], "launches": launches})
        if flags & 1:
            graph_templates.append({"profile": profile})
    return {"cuda_arch": f"sm{head['arch']}", "arena_bytes": head["arena_bytes"],
            "workspace_bytes": head["workspace_bytes"], "shape_dispatch": dispatches,
            "cuda_graph_templates": graph_templates}

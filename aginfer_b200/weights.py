"""Checkpoint ingest and the packed weight blob.

The blob layout is what fixes every ``weights_offset`` a plan may name: tensors sorted by
name, each start rounded up to 256 bytes, raw checkpoint bytes, no casting and no
repacking (reference ``src/aginfer/checkpoint.py:152-179``).  ``weight_layout`` computes
that layout from names and sizes alone, which is what the recipe generators need;
``pack_weights`` materialises it.  ``load_checkpoint`` keeps the reference's ingest rules
(``checkpoint.py:74-149, 233-243``): no pickle files beside the safetensors, only
F32/F16/BF16/F8_E4M3 tensors, FP8 only with a ModelOpt ``quantization_config`` that says
E4M3 with explicit scales.  ``write_safetensors`` is the inverse used to author synthetic
checkpoints.
"""
from __future__ import annotations

import hashlib
import json
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterable, Mapping

from .errors import ValidationError
from .target import CHECKPOINT_DTYPE_BYTES

PICKLE_SUFFIXES = frozenset({".bin", ".pt", ".pth", ".ckpt", ".pkl", ".pickle"})
METADATA_FILES = ("added_tokens.json", "config.json", "generation_config.json", "preprocessor_config.json",
                  "processor_config.json", "special_tokens_map.json", "tokenizer.json", "tokenizer_config.json")


@dataclass(frozen=True)
class TensorRecord:
    name: str
    dtype: str
    shape: tuple[int, ...]
    source: Path
    source_offset: int
    byte_length: int


@dataclass(frozen=True)
class Checkpoint:
    root: Path
    revision: str
    config: dict[str, Any]
    tensors: tuple[TensorRecord, ...]
    safetensor_files: tuple[Path, ...]

    @property
    def dtypes(self) -> frozenset[str]:
        return frozenset(t.dtype for t in self.tensors)


def _numel(shape: Iterable[int]) -> int:
    n = 1
    for extent in shape:
        n *= extent
    return n


def _row_major(shape: tuple[int, ...]) -> list[int]:
    out, run = [], 1
    for extent in reversed(shape):
        out.append(run)
        run *= extent
    return out[::-1]


def write_safetensors(path: Path, tensors: Mapping[str, tuple[str, list[int], bytes]],
                      metadata: Mapping[str, str] | None = None) -> None:
    """Write ``{name: (dtype, shape, raw bytes)}`` in the safetensors layout."""
    header: dict[str, Any] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    at = 0
    for name, (dtype, shape, raw) in tensors.items():
        if len(raw) != _numel(shape) * CHECKPOINT_DTYPE_BYTES[dtype]:
            raise ValidationError(f"tensor {name}: {len(raw)} bytes do not match {dtype}{shape}")
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [at, at + len(raw)]}
        at += len(raw)
    encoded = json.dumps(header, separators=(",", ":")).encode()
    encoded += b" " * (-(8 + len(encoded)) % 8)
    with Path(path).open("wb") as out:
        out.write(struct.pack("<Q", len(encoded)))
        out.write(encoded)
        for _, _, raw in tensors.values():
            out.write(raw)


def inspect_safetensors(path: Path) -> tuple[TensorRecord, ...]:
    """Parse and bounds-check one safetensors header without touching tensor data."""
    size = path.stat().st_size
    if size < 8:
        raise ValidationError(f"truncated safetensors file: {path}")
    with path.open("rb") as stream:
        (header_size,) = struct.unpack("<Q", stream.read(8))
        if not 1 < header_size <= min(100 * 1024 * 1024, size - 8):
            raise ValidationError(f"invalid safetensors header size in {path}")
        try:
            header = json.loads(stream.read(header_size))
        except (UnicodeDecodeError, json.JSONDecodeError) as exc:
            raise ValidationError(f"invalid safetensors JSON header in {path}: {exc}") from exc
    if not isinstance(header, dict):
        raise ValidationError(f"safetensors header must be an object: {path}")
    base = 8 + header_size
    payload = size - base
    records, spans = [], []
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        if not isinstance(entry, dict):
            raise ValidationError(f"invalid tensor entry in {path}")
        try:
            dtype = str(entry["dtype"])
            shape = tuple(int(v) for v in entry["shape"])
            begin, end = (int(v) for v in entry["data_offsets"])
        except (KeyError, TypeError, ValueError) as exc:
            raise ValidationError(f"invalid metadata for tensor {name} in {path}") from exc
        if dtype not in CHECKPOINT_DTYPE_BYTES:
            raise ValidationError(f"tensor {name} uses unsupported dtype {dtype}")
        if any(extent < 0 for extent in shape):
            raise ValidationError(f"tensor {name} has a negative dimension")
        if begin < 0 or end <= begin or end > payload:
            raise ValidationError(f"tensor {name} has invalid data offsets")
        expected = _numel(shape) * CHECKPOINT_DTYPE_BYTES[dtype]
        if end - begin != expected:
            raise ValidationError(f"tensor {name} byte length mismatch: metadata={end - begin}, expected={expected}")
        spans.append((begin, end, name))
        records.append(TensorRecord(name, dtype, shape, path, base + begin, end - begin))
    spans.sort()
    for (_, prev_end, prev_name), (begin, _, name) in zip(spans, spans[1:]):
        if begin < prev_end:
            raise ValidationError(f"overlapping tensor data in {path}: {prev_name} and {name}")
    return tuple(records)


def _check_fp8(config: dict[str, Any], records: list[TensorRecord]) -> None:
    if all(r.dtype != "F8_E4M3" for r in records):
        return
    q = config.get("quantization_config")
    if not isinstance(q, dict):
        raise ValidationError("FP8 tensors require a ModelOpt Unified HF quantization_config")
    method = str(q.get("quant_method", "")).lower()
    fmt = str(q.get("quantization_format", q.get("format", ""))).lower()
    scales = str(q.get("scales", q.get("scale_mode", ""))).lower()
    if "modelopt" not in method or fmt not in {"fp8", "e4m3", "fp8_e4m3"} or scales != "explicit":
        raise ValidationError("only ModelOpt Unified HF E4M3 FP8 with explicit scales is accepted")


def _tree_revision(root: Path) -> str:
    h = hashlib.sha256()
    for path in sorted(p for p in root.rglob("*") if p.is_file()):
        rel = path.relative_to(root).as_posix().encode()
        h.update(len(rel).to_bytes(4, "little") + rel + path.stat().st_size.to_bytes(8, "little"))
        with path.open("rb") as stream:
            while chunk := stream.read(1 << 20):
                h.update(chunk)
    return f"local-sha256:{h.hexdigest()}"


def load_checkpoint(source: str, revision: str | None = None, offline: bool = False) -> Checkpoint:
    """Open a local Hugging Face style snapshot directory (remote download is not offered)."""
    root = Path(source).expanduser()
    if not root.is_dir():
        raise ValidationError("offline mode only accepts an existing local Hugging Face snapshot")
    root = root.resolve()
    pickles = sorted(p.relative_to(root) for p in root.rglob("*") if p.suffix.lower() in PICKLE_SUFFIXES)
    if pickles:
        raise ValidationError("unsafe pickle checkpoint files are forbidden: " + ", ".join(map(str, pickles[:5])))
    config_path = root / "config.json"
    if not config_path.is_file():
        raise ValidationError(f"missing Hugging Face config.json in {root}")
    try:
        config = json.loads(config_path.read_text(encoding="utf-8"))
    except (OSError, UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise ValidationError(f"cannot parse {config_path}: {exc}") from exc
    if not isinstance(config, dict):
        raise ValidationError("config.json must contain an object")
    files = tuple(sorted(root.rglob("*.safetensors")))
    if not files:
        raise ValidationError(f"no safetensors files found in {root}")
    records: dict[str, TensorRecord] = {}
    for path in files:
        for record in inspect_safetensors(path):
            if record.name in records:
                raise ValidationError(f"duplicate tensor name across checkpoint shards: {record.name}")
            records[record.name] = record
    if not records:
        raise ValidationError("checkpoint contains no tensors")
    ordered = sorted(records.values(), key=lambda r: r.name)
    _check_fp8(config, ordered)
    return Checkpoint(root, revision or _tree_revision(root), config, tuple(ordered), files)


def weight_layout(sizes: Mapping[str, int], alignment: int = 256) -> tuple[dict[str, int], int]:
    """Blob offset of every tensor given ``{name: byte_length}``, and the blob's total size."""
    offsets, cursor = {}, 0
    for name in sorted(sizes):
        cursor = -(-cursor // alignment) * alignment
        offsets[name] = cursor
        cursor += sizes[name]
    return offsets, cursor


def pack_weights(tensors: Iterable[TensorRecord], alignment: int = 256) -> tuple[bytes, list[dict[str, Any]]]:
    """Concatenate checkpoint bytes in name order and describe them (``checkpoint.py:152-179``)."""
    ordered = sorted(tensors, key=lambda r: r.name)
    offsets, total = weight_layout({r.name: r.byte_length for r in ordered}, alignment)
    blob = bytearray(total)
    table = []
    handles: dict[Path, Any] = {}
    try:
        for r in ordered:
            stream = handles.get(r.source)
            if stream is None:
                stream = handles[r.source] = r.source.open("rb")
            stream.seek(r.source_offset)
            at = offsets[r.name]
            got = stream.readinto(memoryview(blob)[at: at + r.byte_length])
            if got != r.byte_length:
                raise ValidationError(f"truncated tensor data while reading {r.name}")
            table.append({
                "name": r.name, "dtype": r.dtype, "shape": list(r.shape), "stride": _row_major(r.shape),
                "layout": "checkpoint_contiguous", "blob_offset": at, "byte_length": r.byte_length,
                "sha256": hashlib.sha256(memoryview(blob)[at: at + r.byte_length]).hexdigest(),
                "quantization": {"format": "e4m3", "scale": "explicit"} if r.dtype == "F8_E4M3" else None,
            })
    finally:
        for stream in handles.values():
            stream.close()
    return bytes(blob), table


def collect_metadata(root: Path) -> dict[str, Any]:
    """Tokenizer / processor side files copied into the manifest (``checkpoint.py:182-191``)."""
    found: dict[str, Any] = {}
    for name in METADATA_FILES:
        path = root / name
        if path.is_file():
            found[name] = json.loads(path.read_text(encoding="utf-8"))
    for path in sorted(root.glob("*.yaml")) + sorted(root.glob("*.yml")):
        found[path.name] = path.read_text(encoding="utf-8")
    return found

"""AIM v1 container: deterministic writer and verifying reader.

File layout (all little-endian, every payload 256-byte aligned) is the reference's
(``docs/aim-v1.md``; ``src/aginfer/aim.py:115-228`` writer, ``:246-348`` reader): a
256-byte header, canonical-JSON manifest / graph / tensor table, per-architecture
kernel bundle + weight blob + binary plan (identical blobs stored once), and a directory
of 192-byte variant entries.  The header's file digest (byte 136) is SHA-256 of the
whole file with those 32 bytes read as zero.

The writer here plans every offset first and then streams the sections to disk while
feeding the file digest, so a multi-gigabyte weight blob is never copied into a second
in-memory image of the file; the bytes written equal the reference writer's.
"""
from __future__ import annotations

import hashlib
import json
import mmap
import os
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Iterable

from .errors import CompatibilityError, FormatError, ValidationError
from .target import (ALIGNMENT, RUNTIME_ABI, SCHEMA_MAJOR, SCHEMA_MINOR, CudaArch, Platform,
                     contains_ptx, cubin_targets, validate_target)

MAGIC = b"AIMAOT1\0"
ENDIAN_TAG = 0x01020304
HEADER_STRUCT = struct.Struct("<8sHHIIIII9Q32s32s32s32s24s")
VARIANT_STRUCT = struct.Struct("<II6Q32s32s32s40s")
HEADER_SIZE, VARIANT_SIZE = HEADER_STRUCT.size, VARIANT_STRUCT.size
FILE_HASH_OFFSET, FILE_HASH_SIZE = 136, 32
assert (HEADER_SIZE, VARIANT_SIZE) == (256, 192)


def canonical_json(value: Any) -> bytes:
    return json.dumps(value, sort_keys=True, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def _digest(data) -> bytes:
    return hashlib.sha256(data).digest()


def _round_up(n: int) -> int:
    return -(-n // ALIGNMENT) * ALIGNMENT


def check_kernel_bundle(blob, arch: CudaArch, label: str, error: type[Exception] = ValidationError) -> None:
    """PTX-free, ELF64-LE, ``e_machine`` 190, built for exactly ``arch`` (``aim.py:48-61``)."""
    if contains_ptx(blob):
        raise ValidationError(f"{label} appears to contain PTX; AIM accepts CUBIN/SASS only")
    targets = cubin_targets(blob)
    if targets is None:
        raise error(f"{label} is not a 64-bit little-endian NVIDIA CUDA ELF CUBIN")
    if int(arch) not in targets:
        raise error(f"{label} ELF flags do not target exact {arch.name_string}")


@dataclass(frozen=True)
class VariantPayload:
    arch: CudaArch
    kernels: bytes
    weights: bytes  # any bytes-like object, e.g. an mmap of a packed blob
    plan: bytes


@dataclass(frozen=True)
class Section:
    offset: int
    size: int
    sha256: bytes


@dataclass(frozen=True)
class VariantInfo:
    arch: CudaArch
    kernels: Section
    weights: Section
    plan: Section


@dataclass(frozen=True)
class AimInfo:
    path: Path
    schema_major: int
    schema_minor: int
    runtime_abi: int
    platform: Platform
    manifest: dict[str, Any]
    graph: dict[str, Any]
    tensors: dict[str, Any]
    variants: tuple[VariantInfo, ...]
    file_size: int
    file_sha256: str

    def select_variant(self, arch: CudaArch) -> VariantInfo:
        for variant in self.variants:
            if variant.arch == arch:
                return variant
        have = ", ".join(v.arch.name_string for v in self.variants)
        raise CompatibilityError(
            f"AIM has no exact {arch.name_string} variant (available: {have or 'none'}); fallback is forbidden")


class AimWriter:
    """Deterministic writer; identical payloads of one kind share a single stored copy."""

    @staticmethod
    def write(path: str | os.PathLike[str], *, platform: Platform, manifest: dict[str, Any],
              graph: dict[str, Any], tensors: dict[str, Any], variants: Iterable[VariantPayload],
              runtime_abi: int = RUNTIME_ABI, verify: bool = True) -> AimInfo:
        ordered = sorted(variants, key=lambda v: int(v.arch))
        validate_target(platform, [v.arch for v in ordered])
        if runtime_abi <= 0:
            raise ValidationError("runtime ABI must be positive")
        for v in ordered:
            tag = v.arch.name_string
            if not len(v.kernels):
                raise ValidationError(f"{tag}: empty kernel bundle")
            if not len(v.weights):
                raise ValidationError(f"{tag}: empty weight blob")
            if not len(v.plan):
                raise ValidationError(f"{tag}: empty execution plan")
            check_kernel_bundle(v.kernels, v.arch, f"{tag} kernel bundle")

        # Pass 1: place every distinct (kind, digest) payload once, in first-use order.
        cursor = HEADER_SIZE
        placed: dict[tuple[str, bytes], Section] = {}
        stream_order: list[tuple[Section, Any]] = []

        def place(kind: str, blob) -> Section:
            nonlocal cursor
            key = (kind, _digest(blob))
            hit = placed.get(key)
            if hit is not None and hit.size == len(blob):
                return hit
            cursor = _round_up(cursor)
            section = Section(cursor, len(blob), key[1])
            cursor += len(blob)
            placed[key] = section
            stream_order.append((section, blob))
            return section

        s_manifest = place("manifest", canonical_json(manifest))
        s_graph = place("graph", canonical_json(graph))
        s_tensors = place("tensors", canonical_json(tensors))
        entries = bytearray()
        for v in ordered:
            k, w, p = place("kernels", v.kernels), place("weights", v.weights), place("plan", v.plan)
            entries += VARIANT_STRUCT.pack(int(v.arch), 0, k.offset, k.size, w.offset, w.size, p.offset, p.size,
                                           k.sha256, w.sha256, p.sha256, b"\0" * 40)
        directory_offset = _round_up(cursor)
        file_size = directory_offset + len(entries)
        header = bytearray(HEADER_STRUCT.pack(
            MAGIC, SCHEMA_MAJOR, SCHEMA_MINOR, HEADER_SIZE, runtime_abi, int(platform), ENDIAN_TAG, len(ordered),
            file_size, s_manifest.offset, s_manifest.size, s_graph.offset, s_graph.size, s_tensors.offset,
            s_tensors.size, directory_offset, len(entries), _digest(entries), b"\0" * 32, s_manifest.sha256,
            s_graph.sha256, b"\0" * 24))

        # Pass 2: stream to a temporary file, digesting as we go; patch the digest; rename.
        target = Path(path)
        target.parent.mkdir(parents=True, exist_ok=True)
        scratch = target.with_name(f".{target.name}.tmp-{os.getpid()}")
        whole = hashlib.sha256()
        try:
            with scratch.open("wb") as out:
                def emit(chunk) -> None:
                    whole.update(chunk)
                    out.write(chunk)
                emit(header)
                at = HEADER_SIZE
                for section, blob in stream_order:
                    emit(b"\0" * (section.offset - at))
                    emit(blob)
                    at = section.offset + section.size
                emit(b"\0" * (directory_offset - at))
                emit(entries)
                out.seek(FILE_HASH_OFFSET)
                out.write(whole.digest())
                out.flush()
                os.fsync(out.fileno())
            os.replace(scratch, target)
        finally:
            if scratch.exists():
                scratch.unlink()
        return AimReader.read(target, verify_payloads=verify)


class AimReader:
    @staticmethod
    def read(path: str | os.PathLike[str], *, verify_payloads: bool = True) -> AimInfo:
        source = Path(path)
        try:
            with source.open("rb") as stream:
                if os.fstat(stream.fileno()).st_size < HEADER_SIZE:
                    raise FormatError("file is smaller than the AIM header")
                with mmap.mmap(stream.fileno(), 0, access=mmap.ACCESS_READ) as data:
                    view = memoryview(data)
                    try:
                        return _parse(source, view, verify_payloads)
                    finally:
                        view.release()
        except OSError as exc:
            raise FormatError(f"cannot read AIM {source}: {exc}") from exc


def _region(total: int, offset: int, size: int, label: str) -> None:
    if offset < HEADER_SIZE or size <= 0 or offset > total or size > total - offset:
        raise FormatError(f"invalid {label} region: offset={offset}, size={size}")


def _json_at(data: memoryview, offset: int, size: int, digest: bytes | None, label: str, want_dict: bool) -> Any:
    _region(len(data), offset, size, label)
    raw = bytes(data[offset: offset + size])
    if digest is not None and _digest(raw) != digest:
        raise FormatError(f"{label} checksum mismatch")
    try:
        value = json.loads(raw)
    except (UnicodeDecodeError, json.JSONDecodeError) as exc:
        raise FormatError(f"invalid {label} JSON: {exc}") from exc
    if want_dict and not isinstance(value, dict):
        raise FormatError(f"{label} must be a JSON object")
    return value


def _parse(path: Path, data: memoryview, verify_payloads: bool) -> AimInfo:
    (magic, major, minor, header_size, runtime_abi, platform_id, endian, n_variants, file_size,
     m_off, m_size, g_off, g_size, t_off, t_size, d_off, d_size,
     d_sha, f_sha, m_sha, g_sha, reserved) = HEADER_STRUCT.unpack_from(data, 0)
    if magic != MAGIC:
        raise FormatError("bad AIM magic")
    if major != SCHEMA_MAJOR:
        raise FormatError(f"unsupported AIM schema {major}.{minor}")
    if header_size != HEADER_SIZE or endian != ENDIAN_TAG:
        raise FormatError("unsupported AIM header or byte order")
    if file_size != len(data):
        raise FormatError(f"file size mismatch: header={file_size}, actual={len(data)}")
    if any(reserved):
        raise FormatError("non-zero reserved header bytes")
    try:
        platform = Platform(platform_id)
    except ValueError as exc:
        raise FormatError(f"unknown platform id {platform_id}") from exc
    _region(len(data), d_off, d_size, "variant directory")
    if d_size != n_variants * VARIANT_SIZE:
        raise FormatError("variant directory size does not match variant count")
    if _digest(data[d_off: d_off + d_size]) != d_sha:
        raise FormatError("variant directory checksum mismatch")
    whole = hashlib.sha256(data[:FILE_HASH_OFFSET])
    whole.update(b"\0" * FILE_HASH_SIZE)
    whole.update(data[FILE_HASH_OFFSET + FILE_HASH_SIZE:])
    if whole.digest() != f_sha:
        raise FormatError("file checksum mismatch")

    manifest = _json_at(data, m_off, m_size, m_sha, "manifest", True)
    graph = _json_at(data, g_off, g_size, g_sha, "graph", True)
    tensors = _json_at(data, t_off, t_size, None, "tensor table", False)

    found: list[VariantInfo] = []
    for i in range(n_variants):
        rec = VARIANT_STRUCT.unpack_from(data, d_off + i * VARIANT_SIZE)
        if rec[1] != 0 or any(rec[11]):
            raise FormatError(f"variant {i} has unsupported flags or reserved data")
        try:
            arch = CudaArch(rec[0])
        except ValueError as exc:
            raise FormatError(f"variant {i} has unsupported arch sm{rec[0]}") from exc
        if any(v.arch == arch for v in found):
            raise FormatError(f"duplicate {arch.name_string} variant")
        parts = []
        for j, label in enumerate(("kernels", "weights", "plan")):
            offset, size, digest = rec[2 + 2 * j], rec[3 + 2 * j], rec[8 + j]
            if offset % ALIGNMENT:
                raise FormatError(f"{arch.name_string} {label} is not {ALIGNMENT}-byte aligned")
            _region(len(data), offset, size, f"{arch.name_string} {label}")
            body = data[offset: offset + size]
            if verify_payloads and _digest(body) != digest:
                raise FormatError(f"{arch.name_string} {label} checksum mismatch")
            if label == "kernels":
                check_kernel_bundle(bytes(body[: 1024 * 1024]) if size > 1024 * 1024 else bytes(body), arch,
                                    f"{arch.name_string} kernel bundle", FormatError)
            parts.append(Section(offset, size, digest))
        found.append(VariantInfo(arch, *parts))
    try:
        validate_target(platform, [v.arch for v in found])
    except ValueError as exc:
        raise FormatError(str(exc)) from exc
    return AimInfo(path, major, minor, runtime_abi, platform, manifest, graph, tensors, tuple(found),
                   file_size, f_sha.hex())

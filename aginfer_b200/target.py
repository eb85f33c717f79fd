"""Target description: platforms, CUDA architectures, toolchain gate, CUBIN identification.

Mirrors the role of the reference's ``src/aginfer/schema.py`` with one added target row:
``SM100`` (B200, compiled as ``sm_100a``) on linux-x86_64.  The artifact sub-directory and
the ``cuda_arch`` strings stay ``"sm100"`` because the reference derives names as
``f"sm{int}"`` (``schema.py:37-39``); ``CudaArch.parse`` additionally accepts the
``sm100a`` / ``sm_100a`` spellings a user would pass to ``--cuda-arch``.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, fields
from enum import Enum, IntEnum
from typing import Any, Iterable

SCHEMA_MAJOR = 1
SCHEMA_MINOR = 0
RUNTIME_ABI = 1
ALIGNMENT = 256

_TRIPLES = {1: "linux-x86_64-gnu", 2: "linux-aarch64-sbsa"}


class Platform(IntEnum):
    LINUX_X86_64_GNU = 1
    LINUX_AARCH64_SBSA = 2

    @property
    def triple(self) -> str:
        return _TRIPLES[int(self)]

    @classmethod
    def parse(cls, text: str) -> "Platform":
        for number, triple in _TRIPLES.items():
            if triple == text:
                return cls(number)
        raise ValueError(f"unsupported platform: {text}")


class CudaArch(IntEnum):
    SM89 = 89
    SM100 = 100
    SM110 = 110
    SM120 = 120

    @property
    def name_string(self) -> str:
        return f"sm{int(self)}"

    @classmethod
    def parse(cls, text: str) -> "CudaArch":
        digits = text.lower().replace("_", "")
        if digits.startswith("sm"):
            digits = digits[2:]
        # "100a" / "100f" name the architecture-specific feature set of the same
        # numeric target; the package format only records the number.
        if digits[-1:] in ("a", "f") and digits[:-1].isdigit():
            digits = digits[:-1]
        try:
            return cls(int(digits))
        except (ValueError, TypeError) as exc:
            raise ValueError(f"unsupported CUDA architecture: {text}") from exc


VALID_ARCHES = {
    Platform.LINUX_X86_64_GNU: frozenset({CudaArch.SM89, CudaArch.SM100, CudaArch.SM120}),
    Platform.LINUX_AARCH64_SBSA: frozenset({CudaArch.SM110}),
}


class DType(str, Enum):
    FP32 = "F32"
    FP16 = "F16"
    BF16 = "BF16"
    FP8_E4M3 = "F8_E4M3"


CHECKPOINT_DTYPE_BYTES = {"F32": 4, "F16": 2, "BF16": 2, "F8_E4M3": 1}
SUPPORTED_CHECKPOINT_DTYPES = frozenset(CHECKPOINT_DTYPE_BYTES)


@dataclass(frozen=True)
class ToolchainRange:
    cuda_driver_min: int
    cuda_runtime_min: int
    cuda_runtime_max: int
    cublaslt_abi: int
    cudnn_abi: int

    def to_dict(self) -> dict[str, int]:
        return {f.name: getattr(self, f.name) for f in fields(self)}

    @classmethod
    def from_dict(cls, value: dict[str, Any]) -> "ToolchainRange":
        return cls(**{f.name: int(value[f.name]) for f in fields(cls)})


def validate_target(platform: Platform, arches: Iterable[CudaArch]) -> None:
    """Reject empty, duplicated or platform-foreign architecture lists (``schema.py:93-101``)."""
    arches = list(arches)
    if not arches:
        raise ValueError("at least one --cuda-arch is required")
    if len(set(arches)) != len(arches):
        raise ValueError("duplicate CUDA architecture")
    foreign = set(arches) - VALID_ARCHES[platform]
    if foreign:
        names = ", ".join(sorted(a.name_string for a in foreign))
        raise ValueError(f"{names} is not supported for {platform.triple}")


_ELF64_LE = b"\x7fELF\x02\x01\x01"
_EM_CUDA = 190
_PTX_MARKERS = (b".version ", b".target sm_", b".entry ", b".visible .entry")


def cubin_targets(blob: bytes) -> set[int] | None:
    """Numeric architectures an NVIDIA CUDA ELF image may be built for, or ``None``.

    Two ELF flavours exist.  Images with ``EI_OSABI`` 0x33 (what nvcc emits up to sm_90,
    and what the reference's test fixtures imitate) keep the architecture in ``e_flags``
    bits 0-7 and 16-23 — the rule of ``aim.py:55-61``.  Images with ``EI_OSABI`` 0x41 and
    ABI version >= 8 (nvcc 12.9 for sm_100 / sm_100a / sm_120) keep it in bits 8-15;
    e.g. ``-arch=sm_100a`` gives ``e_flags = 0x0600640a`` (0x64 = 100).
    """
    if len(blob) < 64 or bytes(blob[:7]) != _ELF64_LE:
        return None
    if struct.unpack_from("<H", blob, 18)[0] != _EM_CUDA:
        return None
    flags = struct.unpack_from("<I", blob, 48)[0]
    if blob[7] == 0x41 and blob[8] >= 8:
        return {(flags >> 8) & 0xFF}
    return {flags & 0xFF, (flags >> 16) & 0xFF}


def cubin_is_arch_specific(blob: bytes) -> bool:
    """True when a new-flavour image was built for the ``a`` feature set (e_flags bit 3)."""
    flags = struct.unpack_from("<I", blob, 48)[0]
    return blob[7] == 0x41 and bool(flags & 0x8)


def contains_ptx(blob: bytes) -> bool:
    """PTX text markers in the first MiB of a kernel bundle (``aim.py:48-52``)."""
    head = bytes(blob[: 1024 * 1024])
    return any(marker in head for marker in _PTX_MARKERS)

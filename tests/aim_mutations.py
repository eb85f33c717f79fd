"""Corrupted variants of a small, valid AIM file, for loader conformance tests.

``cases(base)`` yields ``(label, arch_override, profile, bytes)``.  Mutations that are meant
to reach checks *behind* the integrity hashes re-seal the file afterwards (``reseal``),
i.e. recompute every SHA-256 the way a writer would, so the loader sees a well-hashed but
structurally wrong package.
"""
from __future__ import annotations

import hashlib
import struct

HEADER = struct.Struct("<8sHHIIIII9Q32s32s32s32s24s")
VARIANT = struct.Struct("<II6Q32s32s32s40s")
PLAN_HEADER = struct.Struct("<8sHHIIIIIIIQQQQQQQQ24s")


def _sha(b) -> bytes:
    return hashlib.sha256(bytes(b)).digest()


def reseal(raw: bytearray) -> bytearray:
    """Recompute payload, directory, manifest, graph and file digests in place."""
    h = list(HEADER.unpack_from(raw, 0))
    n, d_off = h[7], h[15]
    for i in range(n):
        at = d_off + i * VARIANT.size
        if at + VARIANT.size > len(raw):
            break
        v = list(VARIANT.unpack_from(raw, at))
        for j in range(3):
            off, size = v[2 + 2 * j], v[3 + 2 * j]
            if off + size <= len(raw):
                v[8 + j] = _sha(raw[off: off + size])
        VARIANT.pack_into(raw, at, *v)
    # out-of-range regions hash whatever slice Python yields; such files fail earlier anyway
    h[17] = _sha(raw[d_off: d_off + h[16]])
    h[19] = _sha(raw[h[9]: h[9] + h[10]])
    h[20] = _sha(raw[h[11]: h[11] + h[12]])
    h[18] = b"\0" * 32
    HEADER.pack_into(raw, 0, *h)
    raw[136:168] = _sha(raw)
    return raw


def _edit_header(raw: bytearray, index: int, value) -> None:
    h = list(HEADER.unpack_from(raw, 0))
    h[index] = value
    HEADER.pack_into(raw, 0, *h)


def _edit_variant(raw: bytearray, which: int, index: int, value) -> None:
    d_off = HEADER.unpack_from(raw, 0)[15]
    at = d_off + which * VARIANT.size
    v = list(VARIANT.unpack_from(raw, at))
    v[index] = value
    VARIANT.pack_into(raw, at, *v)


def _variant(raw, which: int):
    d_off = HEADER.unpack_from(raw, 0)[15]
    return VARIANT.unpack_from(raw, d_off + which * VARIANT.size)


def cases(base: bytes):
    def fresh() -> bytearray:
        return bytearray(base)

    yield "valid, sm89", 89, "", bytes(base)
    yield "valid, sm120, named profile", 120, "default", bytes(base)
    yield "valid, unknown profile", 89, "missing", bytes(base)
    yield "valid, no variant for sm110", 110, "", bytes(base)

    # --- integrity failures (no re-seal) ---
    k_off = _variant(base, 0)[2]
    raw = fresh(); raw[k_off] ^= 1
    yield "kernel byte flipped", 89, "", bytes(raw)
    raw = fresh(); raw[HEADER.unpack_from(base, 0)[9]] ^= 1
    yield "manifest byte flipped", 89, "", bytes(raw)
    raw = fresh(); raw[-1] ^= 1
    yield "directory byte flipped", 89, "", bytes(raw)
    raw = fresh(); raw[300 + 700] ^= 1  # padding between sections: only the file digest covers it
    yield "padding byte flipped", 89, "", bytes(raw)
    yield "truncated by one byte", 89, "", bytes(base[:-1])
    yield "shorter than a header", 89, "", bytes(base[:100])
    raw = fresh(); raw[0] = ord("B")
    yield "bad magic", 89, "", bytes(raw)

    # --- header fields (re-sealed) ---
    for label, index, value in (("schema major 2", 1, 2), ("header size 128", 3, 128), ("runtime abi 2", 4, 2),
                                ("platform aarch64", 5, 2), ("platform 9", 5, 9), ("endian tag swapped", 6, 0x04030201),
                                ("variant count 3", 7, 3), ("file size off by one", 8, len(base) + 1),
                                ("manifest offset inside header", 9, 128), ("graph size zero", 12, 0),
                                ("tensor table beyond file", 13, len(base)), ("directory size 191", 16, 191),
                                ("reserved header byte set", 21, b"\1" + b"\0" * 23)):
        raw = fresh(); _edit_header(raw, index, value)
        yield label, 89, "", bytes(reseal(raw))

    # --- variant entries (re-sealed) ---
    for label, which, index, value in (("variant arch 90", 0, 0, 90), ("variant arch 110 on x86", 1, 0, 110),
                                       ("duplicate arch", 1, 0, 89), ("variant flags set", 0, 1, 1),
                                       ("variant reserved set", 1, 11, b"\0" * 39 + b"\1"),
                                       ("kernel offset unaligned", 0, 2, k_off + 1),
                                       ("weight size zero", 0, 5, 0), ("plan beyond file", 1, 6, len(base))):
        raw = fresh(); _edit_variant(raw, which, index, value)
        yield label, 89, "", bytes(reseal(raw))

    # --- kernel bundle contents (re-sealed) ---
    raw = fresh(); raw[k_off + 48: k_off + 52] = struct.pack("<I", 120 | 120 << 16)
    yield "cubin flags say sm120 in the sm89 slot", 89, "", bytes(reseal(raw))
    raw = fresh(); raw[k_off + 18: k_off + 20] = struct.pack("<H", 62)
    yield "cubin e_machine x86-64", 89, "", bytes(reseal(raw))
    raw = fresh(); raw[k_off + 4] = 1
    yield "cubin ELF32", 89, "", bytes(reseal(raw))
    raw = fresh(); raw[k_off + 24: k_off + 33] = b".version "
    yield "ptx marker in kernel bundle", 89, "", bytes(reseal(raw))

    # --- manifest contents (re-sealed) ---
    m_off, m_size = HEADER.unpack_from(base, 0)[9:11]
    for label, old, new in (("manifest without cuda_driver_min", b'"cuda_driver_min"', b'"cuda_driver_mix"'),
                            ("driver too old for manifest", b'"cuda_driver_min":12000', b'"cuda_driver_min":99000'),
                            ("runtime above manifest max", b'"cuda_runtime_max":12999', b'"cuda_runtime_max":12001'),
                            ("cublaslt abi differs", b'"cublaslt_abi":12', b'"cublaslt_abi":11'),
                            ("cudnn abi not a number", b'"cudnn_abi":9', b'"cudnn_abi":x')):
        raw = fresh()
        body = bytes(raw[m_off: m_off + m_size])
        assert old in body and len(old) == len(new)
        raw[m_off: m_off + m_size] = body.replace(old, new)
        yield label, 89, "", bytes(reseal(raw))

    # --- binary plan of the sm89 variant (re-sealed) ---
    p_off, p_size = _variant(base, 0)[6:8]
    ph = PLAN_HEADER.unpack_from(base, p_off)
    profiles, tensors, launches, arguments, strings = ph[12:17]

    def plan_edit(label, at, fmt, value):
        raw = fresh()
        struct.pack_into(fmt, raw, p_off + at, value)
        return label, 89, "", bytes(reseal(raw))

    yield plan_edit("plan magic", 0, "<B", ord("X"))
    yield plan_edit("plan schema major", 8, "<H", 2)
    yield plan_edit("plan header size", 12, "<I", 64)
    yield plan_edit("plan arch 120 in sm89 variant", 16, "<I", 120)
    yield plan_edit("plan profile count zero", 20, "<I", 0)
    yield plan_edit("plan tensor count too large", 24, "<I", 1000)
    yield plan_edit("plan launch count zero", 28, "<I", 0)
    yield plan_edit("plan file size", 96, "<Q", p_size - 1)
    yield plan_edit("plan reserved", 104, "<B", 1)
    yield plan_edit("plan tables out of order", 64, "<Q", tensors + 32)
    yield plan_edit("plan strings sentinel", strings, "<B", ord("x"))
    yield plan_edit("profile first tensor", profiles + 4, "<I", 1)
    yield plan_edit("profile tensor count short", profiles + 8, "<I", 3)
    yield plan_edit("profile flags 2", profiles + 20, "<I", 2)
    yield plan_edit("profile reserved", profiles + 24, "<B", 1)
    yield plan_edit("profile name offset bad", profiles, "<I", 100000)
    yield plan_edit("tensor dtype 9", tensors + 4, "<I", 9)
    yield plan_edit("tensor location 3", tensors + 8, "<I", 3)
    yield plan_edit("tensor io kind 0", tensors + 12, "<I", 0)
    yield plan_edit("tensor rank 0", tensors + 16, "<I", 0)
    yield plan_edit("tensor rank 9", tensors + 16, "<I", 9)
    yield plan_edit("tensor flags", tensors + 20, "<I", 1)
    yield plan_edit("tensor byte size too small", tensors + 24, "<Q", 3)
    yield plan_edit("tensor extent zero", tensors + 32, "<q", 0)
    yield plan_edit("tensor stride negative", tensors + 96, "<q", -1)
    yield plan_edit("tensor extent beyond rank", tensors + 40, "<q", 1)
    yield plan_edit("tensor size overflow", tensors + 32, "<q", 2**62)
    yield plan_edit("all tensors inputs", tensors + 3 * 160 + 12, "<I", 1)
    yield plan_edit("duplicate tensor name", tensors + 160, "<I", struct.unpack_from("<I", base, p_off + tensors)[0])
    yield plan_edit("launch grid zero", launches + 16, "<I", 0)
    yield plan_edit("launch block 2048", launches + 28, "<I", 2048)
    yield plan_edit("launch flags", launches + 44, "<I", 1)
    yield plan_edit("launch reserved", launches + 48, "<B", 1)
    yield plan_edit("launch wrong profile", launches + 4, "<I", 5)
    yield plan_edit("launch argument count", launches + 12, "<I", 1)
    yield plan_edit("launch kernel name bad", launches, "<I", 99999)

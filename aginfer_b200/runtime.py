"""ctypes binding of the native loader (``include/aginfer_b200.h``).

The classes follow the reference's C++ API (``include/aginfer/runtime.h:120-176``):
``Runtime.create`` -> ``Model.load`` -> ``Session.create`` -> ``Session.enqueue``.  A failing
call raises ``RuntimeStatusError`` carrying the reference's status code name.  There is
no CPU path: without the compiled library ``load_library`` raises, and ``enqueue`` needs a
CUDA device.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from pathlib import Path
from typing import Iterable, Sequence

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libaginfer_b200.so"
_lib = None

STATUS_NAMES = ("OK", "INVALID_ARGUMENT", "NOT_FOUND", "IO_ERROR", "CORRUPT_PACKAGE", "INCOMPATIBLE_PLATFORM",
                "INCOMPATIBLE_ARCHITECTURE", "INCOMPATIBLE_ABI", "CUDA_ERROR", "OUT_OF_MEMORY")
DTYPES = {"F32": 0, "F16": 1, "BF16": 2, "F8_E4M3": 3, "I32": 4}
DTYPE_NAMES = {v: k for k, v in DTYPES.items()}
HOST, DEVICE = 0, 1
NO_GRAPH_REPLAY, PROGRAMMATIC_LAUNCH, BLOCKING_UPLOAD, NO_COOPERATIVE_LAUNCH = 1, 2, 4, 8
MAX_RANK = 8


class RuntimeStatusError(RuntimeError):
    def __init__(self, code: int, message: str):
        self.code = code
        self.name = STATUS_NAMES[code] if 0 <= code < len(STATUS_NAMES) else "UNKNOWN"
        super().__init__(f"{self.name}: {message}")


class _RuntimeOptions(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("required_runtime_abi", "cuda_arch_override", "cuda_driver_version_override",
                                           "cuda_runtime_version_override", "cublaslt_abi_override",
                                           "cudnn_abi_override")]


class _TensorView(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("location", C.c_uint32), ("rank", C.c_uint32),
                ("reserved", C.c_uint32), ("shape", C.POINTER(C.c_int64)), ("stride", C.POINTER(C.c_int64)),
                ("data", C.c_void_p), ("byte_size", C.c_uint64)]


class _TensorInfo(C.Structure):
    _fields_ = [("name", C.c_char_p), ("dtype", C.c_uint32), ("location", C.c_uint32), ("rank", C.c_uint32),
                ("reserved", C.c_uint32), ("shape", C.c_int64 * MAX_RANK), ("stride", C.c_int64 * MAX_RANK),
                ("byte_size", C.c_uint64)]


class _RunOptions(C.Structure):
    _fields_ = [("denoising_steps", C.c_uint32), ("deterministic", C.c_uint32), ("seed", C.c_uint64),
                ("math_mode", C.c_uint32), ("reserved", C.c_uint32), ("initial_noise_override", C.POINTER(_TensorView))]


class _Stats(C.Structure):
    _fields_ = [("enqueues", C.c_uint64), ("kernel_launches", C.c_uint64), ("graph_launches", C.c_uint64),
                ("graphs_built", C.c_uint64), ("launches_per_enqueue", C.c_uint64), ("upload_seconds", C.c_double)]


EXPORTS = {
    "agi_status_name": (C.c_char_p, [C.c_int]),
    "agi_last_error": (C.c_char_p, []),
    "agi_version": (C.c_char_p, []),
    "agi_runtime_create": (C.c_int, [C.POINTER(_RuntimeOptions), C.POINTER(C.c_void_p)]),
    "agi_runtime_destroy": (None, [C.c_void_p]),
    "agi_runtime_get_options": (C.c_int, [C.c_void_p, C.POINTER(_RuntimeOptions)]),
    "agi_model_load": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "agi_model_destroy": (None, [C.c_void_p]),
    "agi_model_variant_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "agi_model_variant_arch": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(C.c_uint32)]),
    "agi_session_create": (C.c_int, [C.c_void_p, C.c_void_p, C.c_char_p, C.c_uint32, C.POINTER(C.c_void_p)]),
    "agi_session_destroy": (None, [C.c_void_p]),
    "agi_session_get_target_info": (C.c_int, [C.c_void_p, C.POINTER(C.c_char_p), C.POINTER(C.c_char_p),
                                               C.POINTER(C.c_uint32)]),
    "agi_session_get_input_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "agi_session_get_output_count": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "agi_session_get_input_info": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(_TensorInfo)]),
    "agi_session_get_output_info": (C.c_int, [C.c_void_p, C.c_uint32, C.POINTER(_TensorInfo)]),
    "agi_session_get_required_workspace": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint64),
                                                      C.POINTER(C.c_uint64)]),
    "agi_session_enqueue": (C.c_int, [C.c_void_p, C.POINTER(_TensorView), C.c_size_t, C.POINTER(_TensorView),
                                       C.c_size_t, C.c_void_p, C.c_void_p]),
    "agi_session_get_stats": (C.c_int, [C.c_void_p, C.POINTER(_Stats)]),
    "agi_gemm_bf16_static_scratch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32,
                                                C.c_uint32, C.c_uint32, C.c_void_p]),
    "agi_gemm_bf16_static_scratch_status": (C.c_int, [C.c_void_p, C.c_void_p]),
    "agi_sha256": (C.c_int, [C.c_void_p, C.c_size_t, C.c_int, C.POINTER(C.c_uint8)]),
}


def load_library(path: Path | None = None):
    """Open the loader library and declare every entry point of the C header."""
    global _lib
    if _lib is None or path is not None:
        target = Path(path or _LIB_PATH)
        if not target.exists():
            raise RuntimeError(f"{target} is missing: build it with `python -m aginfer_b200.build`")
        lib = C.CDLL(str(target))
        for name, (restype, argtypes) in EXPORTS.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        if path is not None:
            return lib
        _lib = lib
    return _lib


def _check(code: int) -> None:
    if code != 0:
        raise RuntimeStatusError(code, load_library().agi_last_error().decode("utf-8", "replace"))


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple[int, ...]
    stride: tuple[int, ...]
    byte_size: int
    location: int


@dataclass
class TensorView:
    """A caller-owned buffer: ``data`` is a raw address (device pointer for device tensors)."""
    name: str
    dtype: str
    shape: Sequence[int]
    stride: Sequence[int]
    data: int
    byte_size: int
    location: int = DEVICE

    @classmethod
    def from_torch(cls, name: str, tensor, dtype: str | None = None) -> "TensorView":
        import torch
        names = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32",
                 torch.float8_e4m3fn: "F8_E4M3", torch.uint8: "F8_E4M3"}
        return cls(name, dtype or names[tensor.dtype], tuple(tensor.shape), tuple(tensor.stride()), tensor.data_ptr(),
                   tensor.untyped_storage().nbytes() - tensor.storage_offset() * tensor.element_size(),
                   DEVICE if tensor.is_cuda else HOST)


def _pack_views(views: Iterable[TensorView]):
    views = list(views)
    array = (_TensorView * max(len(views), 1))()
    keep = []
    for slot, v in zip(array, views):
        shape = (C.c_int64 * max(len(v.shape), 1))(*v.shape)
        stride = (C.c_int64 * max(len(v.stride), 1))(*v.stride)
        name = v.name.encode("utf-8")
        keep += [shape, stride, name]
        slot.name, slot.dtype, slot.location, slot.rank = name, DTYPES[v.dtype], v.location, len(v.shape)
        slot.shape, slot.stride = shape, stride
        slot.data, slot.byte_size = v.data, v.byte_size
    return array, len(views), keep


class Runtime:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def create(cls, *, required_runtime_abi: int = 1, cuda_arch_override: int = 0,
               cuda_driver_version_override: int = 0, cuda_runtime_version_override: int = 0,
               cublaslt_abi_override: int = 0, cudnn_abi_override: int = 0) -> "Runtime":
        options = _RuntimeOptions(required_runtime_abi, cuda_arch_override, cuda_driver_version_override,
                                  cuda_runtime_version_override, cublaslt_abi_override, cudnn_abi_override)
        handle = C.c_void_p()
        _check(load_library().agi_runtime_create(C.byref(options), C.byref(handle)))
        return cls(handle)

    @property
    def options(self) -> dict[str, int]:
        out = _RuntimeOptions()
        _check(load_library().agi_runtime_get_options(self._h, C.byref(out)))
        return {name: getattr(out, name) for name, _ in _RuntimeOptions._fields_}

    def close(self) -> None:
        if self._h and _lib is not None:   # at interpreter shutdown the module may already be torn down
            _lib.agi_runtime_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Model:
    def __init__(self, handle):
        self._h = handle

    @classmethod
    def load(cls, aim_path: str | Path) -> "Model":
        handle = C.c_void_p()
        _check(load_library().agi_model_load(str(aim_path).encode(), C.byref(handle)))
        return cls(handle)

    @property
    def arches(self) -> list[int]:
        lib, n, arch = load_library(), C.c_uint32(), C.c_uint32()
        _check(lib.agi_model_variant_count(self._h, C.byref(n)))
        found = []
        for i in range(n.value):
            _check(lib.agi_model_variant_arch(self._h, i, C.byref(arch)))
            found.append(arch.value)
        return found

    def close(self) -> None:
        if self._h and _lib is not None:   # at interpreter shutdown the module may already be torn down
            _lib.agi_model_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Session:
    def __init__(self, handle, runtime: Runtime, model: Model):
        self._h, self._runtime, self._model = handle, runtime, model  # keep the borrowed objects alive

    @classmethod
    def create(cls, runtime: Runtime, model: Model, profile: str = "", flags: int = 0) -> "Session":
        handle = C.c_void_p()
        _check(load_library().agi_session_create(runtime._h, model._h, profile.encode(), flags, C.byref(handle)))
        return cls(handle, runtime, model)

    def target_info(self) -> dict[str, object]:
        platform, arch, abi = C.c_char_p(), C.c_char_p(), C.c_uint32()
        _check(load_library().agi_session_get_target_info(self._h, C.byref(platform), C.byref(arch), C.byref(abi)))
        return {"platform": platform.value.decode(), "cuda_arch": arch.value.decode(), "runtime_abi": abi.value}

    def _infos(self, count_fn, info_fn) -> list[TensorInfo]:
        n = C.c_uint32()
        _check(count_fn(self._h, C.byref(n)))
        found = []
        for i in range(n.value):
            raw = _TensorInfo()
            _check(info_fn(self._h, i, C.byref(raw)))
            found.append(TensorInfo(raw.name.decode(), DTYPE_NAMES[raw.dtype], tuple(raw.shape[: raw.rank]),
                                    tuple(raw.stride[: raw.rank]), raw.byte_size, raw.location))
        return found

    def input_info(self) -> list[TensorInfo]:
        lib = load_library()
        return self._infos(lib.agi_session_get_input_count, lib.agi_session_get_input_info)

    def output_info(self) -> list[TensorInfo]:
        lib = load_library()
        return self._infos(lib.agi_session_get_output_count, lib.agi_session_get_output_info)

    def required_workspace(self, profile: str = "") -> dict[str, int]:
        arena, workspace = C.c_uint64(), C.c_uint64()
        _check(load_library().agi_session_get_required_workspace(self._h, profile.encode(), C.byref(arena),
                                                                 C.byref(workspace)))
        return {"arena_bytes": arena.value, "workspace_bytes": workspace.value}

    def bind(self, inputs: Iterable[TensorView], outputs: Iterable[TensorView]):
        """Pre-pack views for repeated ``enqueue_packed`` calls (keeps ctypes work out of a timed loop)."""
        return _pack_views(inputs), _pack_views(outputs)

    def enqueue_packed(self, packed, stream: int = 0, options=None) -> None:
        """``options``: a ``run_options(...)`` value, or None for the session's profile as packaged."""
        (ins, n_in, _), (outs, n_out, _) = packed
        raw = C.byref(options[0]) if options is not None else None
        _check(load_library().agi_session_enqueue(self._h, ins, n_in, outs, n_out, raw, C.c_void_p(stream)))

    def enqueue(self, inputs: Iterable[TensorView], outputs: Iterable[TensorView], stream: int = 0,
                options=None) -> None:
        self.enqueue_packed(self.bind(inputs, outputs), stream, options)

    def stats(self) -> dict[str, float]:
        out = _Stats()
        _check(load_library().agi_session_get_stats(self._h, C.byref(out)))
        return {name: getattr(out, name) for name, _ in _Stats._fields_}

    def close(self) -> None:
        if self._h and _lib is not None:   # at interpreter shutdown the module may already be torn down
            _lib.agi_session_destroy(self._h)
        self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sha256(data: bytes, portable: bool = False) -> bytes:
    out = (C.c_uint8 * 32)()
    buf = C.create_string_buffer(bytes(data), len(data))
    _check(load_library().agi_sha256(buf, len(data), int(portable), out))
    return bytes(out)


def gemm_bf16_static_scratch(x_ptr: int, w_ptr: int, y_ptr: int, bias_ptr: int | None, M: int, N: int, K: int,
                             splits: int = 1, stream: int = 0) -> None:
    """``agi_gemm_bf16_static_scratch``: split-K bf16 GEMM whose scratch is a fixed array in the library,
    for callers that must not allocate device memory.  Arguments are raw device addresses."""
    _check(load_library().agi_gemm_bf16_static_scratch(C.c_void_p(x_ptr), C.c_void_p(w_ptr), C.c_void_p(y_ptr),
                                                       C.c_void_p(bias_ptr) if bias_ptr else None, M, N, K, splits,
                                                       C.c_void_p(stream)))


def gemm_bf16_static_scratch_status(out_ptr: int, stream: int = 0) -> None:
    """``agi_gemm_bf16_static_scratch_status``: copy the wait-status word of the last static-scratch GEMM
    into the caller's 4-byte device (or pinned host) word at ``out_ptr``, ordered on ``stream``."""
    _check(load_library().agi_gemm_bf16_static_scratch_status(C.c_void_p(out_ptr), C.c_void_p(stream)))



def run_options(denoising_steps: int = 0, initial_noise_override: TensorView | None = None, seed: int = 0,
                deterministic: bool = False, math_mode: int = 0):
    """The reference's RunOptions (include/aginfer/runtime.h:84-90) for ``Session.enqueue``: ``denoising_steps``
    selects the sibling profile ``<profile>/steps=<n>`` (0 = the session's profile as packaged) and
    ``initial_noise_override`` stands in for the input named ``noise``; the other fields are carried and have
    no effect.  Returns an opaque value that keeps the ctypes storage alive."""
    raw = _RunOptions(denoising_steps, int(deterministic), seed, math_mode, 0, None)
    keep = None
    if initial_noise_override is not None:
        array, _, keep = _pack_views([initial_noise_override])
        raw.initial_noise_override = C.cast(array, C.POINTER(_TensorView))
        keep = (array, keep)
    return raw, keep

"""B200 (sm_100a) execution backend for AgInfer's AIM launch recipe.

Host side: a format-compatible packager (``modelc``) and the bindings of the native
loader (``runtime``).  Device side: the ``sm100`` kernel bundle under ``csrc/kernels`` and
the recipe generators under ``recipes`` that emit its ``plan.json`` / ``tactics.json`` /
``toolchain.json`` artifact set.
"""
from .container import AimInfo, AimReader, AimWriter, Section, VariantInfo, VariantPayload
from .errors import AgInferError, CompatibilityError, FormatError, ValidationError
from .modelc import CompileOptions, compile_model, load_profile
from .planfmt import CompiledPlan, compile_execution_plan, decode_plan, inspect_plan
from .target import CudaArch, Platform, ToolchainRange, validate_target
from .weights import (Checkpoint, TensorRecord, inspect_safetensors, load_checkpoint, pack_weights, weight_layout,
                      write_safetensors)

__all__ = [
    "AgInferError", "AimInfo", "AimReader", "AimWriter", "Checkpoint", "CompatibilityError", "CompileOptions",
    "CompiledPlan", "CudaArch", "FormatError", "Platform", "Section", "TensorRecord", "ToolchainRange",
    "ValidationError", "VariantInfo", "VariantPayload", "compile_execution_plan", "compile_model", "decode_plan",
    "inspect_plan", "inspect_safetensors", "load_checkpoint", "load_profile", "pack_weights", "validate_target",
    "weight_layout", "write_safetensors",
]

"""Run a packaged recipe on the current CUDA device with torch tensors as caller buffers.

This is the call a user makes: ``Runner(aim).run(inputs, outputs)`` wraps
``Runtime.create -> Model.load -> Session.create -> Session.enqueue`` of ``runtime.py`` and
submits on torch's current stream.  torch only owns device memory and streams here; every
kernel comes from the AIM's CUBIN through the native loader.
"""
from __future__ import annotations

from pathlib import Path
from typing import Mapping

from . import runtime as rt

TORCH_DTYPES = {"F32": "float32", "F16": "float16", "BF16": "bfloat16", "F8_E4M3": "uint8", "I32": "int32"}


class Runner:
    def __init__(self, aim_path: str | Path, profile: str = "", flags: int = 0, probe_libraries: bool = False):
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("aginfer_b200.Runner needs a CUDA device; there is no CPU execution path")
        torch.cuda.current_stream().synchronize()  # make sure torch's context is the current one
        overrides = {} if probe_libraries else dict(cuda_runtime_version_override=12080, cublaslt_abi_override=12,
                                                    cudnn_abi_override=9)
        self.runtime = rt.Runtime.create(**overrides)
        self.model = rt.Model.load(aim_path)
        self.session = rt.Session.create(self.runtime, self.model, profile, flags)
        self.inputs = self.session.input_info()
        self.outputs = self.session.output_info()
        self._packed = None
        self._packed_key = None
        self._side = None

    def empty_outputs(self, device="cuda") -> dict:
        import torch
        return {t.name: torch.empty(t.shape, dtype=getattr(torch, TORCH_DTYPES[t.dtype]), device=device)
                for t in self.outputs}

    def run(self, inputs: Mapping[str, "object"], outputs: Mapping[str, "object"] | None = None, stream=None,
            denoising_steps: int = 0, noise_override=None) -> dict:
        """``denoising_steps`` / ``noise_override`` (a tensor) travel as the reference's RunOptions: another
        number of Euler steps runs the package's sibling profile for it, and the override replaces the ``noise``
        input (which may then be left out of ``inputs``)."""
        import torch
        outputs = dict(outputs) if outputs is not None else self.empty_outputs()
        options = None
        if denoising_steps or noise_override is not None:
            view = None
            if noise_override is not None:
                dtype = {t.name: t.dtype for t in self.inputs}.get("noise")
                view = rt.TensorView.from_torch("noise_override", noise_override, dtype)
                self._override_keep = noise_override
            options = rt.run_options(denoising_steps, view)
        key = tuple(t.data_ptr() for t in inputs.values()) + tuple(t.data_ptr() for t in outputs.values())
        if key != self._packed_key:
            dt = {t.name: t.dtype for t in self.inputs + self.outputs}
            self._packed = self.session.bind(
                [rt.TensorView.from_torch(n, t, dt.get(n)) for n, t in inputs.items()],
                [rt.TensorView.from_torch(n, t, dt.get(n)) for n, t in outputs.items()])
            self._packed_key = key
            self._keep = (dict(inputs), outputs)
        s = stream if stream is not None else torch.cuda.current_stream()
        if s.cuda_stream == 0:
            # The legacy default stream cannot be captured, so graph replay needs a real stream:
            # run on a side stream, ordered after and before the work on the default stream.
            if self._side is None:
                self._side = torch.cuda.Stream()
            self._side.wait_stream(s)
            self.session.enqueue_packed(self._packed, self._side.cuda_stream, options)
            s.wait_stream(self._side)
        else:
            self.session.enqueue_packed(self._packed, s.cuda_stream, options)
        return outputs

    def stats(self) -> dict:
        return self.session.stats()

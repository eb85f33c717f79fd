"""BASELINE config 2: the FP8 E4M3 scaled GEMM / GEMV sweep, every (M, N, K) of the grid, seed 1.

Weights ~N(0, 0.02) quantised per tensor by amax / 448; activations N(0, 1) bf16, quantised on the GPU
(bit-exact tier, checked here too); fp32 accumulation, bf16 output.  The builder picks the kernel:
bulk-stream GEMV/skinny GEMM for M <= 64, tcgen05 above."""
from __future__ import annotations

import pytest
import torch

from aginfer_b200.recipes import Tensor, Weight
from oracle import ops
from tests.gpu_util import run_recipe

pytestmark = pytest.mark.gpu
SHAPES = [(2048, 2048), (11008, 2048), (2048, 11008), (2560, 2048), (1536, 1536), (6144, 1536)]
TOKENS = [1, 16, 64, 288, 1024]


@pytest.mark.parametrize("N,K", SHAPES, ids=lambda v: str(v))
@pytest.mark.parametrize("M", TOKENS)
def test_fp8_scaled_gemm_sweep(tmp_path, M, N, K):
    g = torch.Generator().manual_seed(1)
    wq, ws = ops.quantize_e4m3((torch.randn(N, K, generator=g) * 0.02).to(torch.bfloat16))
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    xq, xs = ops.quantize_e4m3(x)

    def body(r):
        q, s = r.alloc(M * K), r.alloc(4)
        r.quantize_e4m3(Tensor("x"), q, s, M * K)
        r.gemm(q, Weight("w"), Tensor("y"), M, N, K, dtype="e4m3", scale_a=s, scale_w=Weight("w_scale"))
        r.launch("agi_copy_u32", (1, 1, 1), (32, 1, 1), [s, Tensor("scale"), __import__("aginfer_b200.recipes", fromlist=["U32"]).U32(1)])
        r.export_status(Tensor("status"))

    got, _ = run_recipe(tmp_path, {"w": wq, "w_scale": ws.reshape(())}, {"x": x},
                        {"y": (torch.bfloat16, (M, N)), "scale": (torch.int32, (1,)), "status": (torch.int32, (1,))},
                        body, repeats=2)
    assert got["status"].item() == 0
    assert got["scale"].item() == xs.view(torch.int32).item()          # activation scale: bit-exact
    assert ops.max_rel_err(got["y"], ops.gemm(xq, wq, scale_a=xs, scale_w=ws)) < 1e-2

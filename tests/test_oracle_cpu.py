"""Sanity of the CPU oracle itself (it defines the arithmetic the GPU kernels are held to)."""
import torch

from oracle import ops


def test_quantize_is_rne_saturating_and_bit_stable():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(64, 96, generator=g).to(torch.bfloat16)
    q, s = ops.quantize_e4m3(x)
    assert q.dtype == torch.float8_e4m3fn and s.dtype == torch.float32
    assert float(s) == float(x.float().abs().max() / 448.0)
    back = q.float() * s
    assert ops.max_rel_err(back, x) < 0.07          # e4m3 has 3 mantissa bits
    assert q.float().abs().max() == 448.0            # amax maps onto the largest finite value
    # hand-checked codes: 0 -> 0x00, amax -> 0x7e, -amax -> 0xfe, half-way cases round to even
    probe = torch.tensor([0.0, 448.0, -448.0, 17.0, 19.0, 0.001953125 * 1.5], dtype=torch.float32)
    codes = probe.to(torch.float8_e4m3fn).view(torch.uint8).tolist()
    assert codes == [0x00, 0x7E, 0xFE, 0x58, 0x5A, 0x02]
    z, sz = ops.quantize_e4m3(torch.zeros(8, dtype=torch.bfloat16))
    assert float(sz) == 1.0 and z.float().abs().max() == 0


def test_gemm_epilogue_order():
    x = torch.tensor([[1.0, 2.0]], dtype=torch.bfloat16)
    w = torch.tensor([[3.0, 4.0], [-1.0, 0.5]], dtype=torch.bfloat16)
    y = ops.gemm(x, w, bias=torch.tensor([1.0, 1.0], dtype=torch.bfloat16), act="silu",
                 residual=torch.tensor([[10.0, 10.0]], dtype=torch.bfloat16), out_f32=True)
    want = torch.tensor([[12.0, 1.0]])
    want = want * torch.sigmoid(want) + 10.0
    assert torch.allclose(y, want)


def test_rope_rotation_preserves_norm_and_matches_mrope_on_equal_streams():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(9, 3, 128, generator=g).to(torch.bfloat16)
    r = ops.rope(x, 1e6)
    assert torch.allclose(r.float().norm(dim=-1), x.float().norm(dim=-1), rtol=2e-2)
    pos = torch.arange(9).repeat(3, 1)
    assert torch.equal(ops.mrope(x, pos, 1e6, (16, 24, 24)), r)
    assert torch.equal(r[0], x[0])  # position 0 is the identity


def test_attention_masks():
    g = torch.Generator().manual_seed(0)
    q = torch.randn(6, 4, 16, generator=g).to(torch.bfloat16)
    k = torch.randn(6, 2, 16, generator=g).to(torch.bfloat16)
    v = torch.randn(6, 2, 16, generator=g).to(torch.bfloat16)
    causal = ops.attention(q, k, v, mask="causal")
    assert torch.allclose(causal[0].float(), v[0].float().repeat_interleave(2, 0), atol=1e-2)  # row 0 sees key 0 only
    block = ops.attention(q, k, v, mask="block", mask_arg=3)
    alone = ops.attention(q[:3], k[:3], v[:3])
    assert torch.equal(block[:3], alone)

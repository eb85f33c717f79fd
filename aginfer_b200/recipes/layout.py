"""Packed operand layout of the bulk-copy tensor-core GEMM: "K-block-major, swizzled".

A matrix [R, K] of 1- or 2-byte elements is cut into 128-byte K blocks.  Block kb of row r is stored at byte
offset ``(kb * R_padded + r) * 128``, and inside it the 16-byte chunk c sits at position ``c ^ (r & 7)``: exactly
the image of a 128-byte-swizzled K-major shared-memory tile.  A tile of consecutive rows of one K block is
therefore ONE contiguous run of global memory, which a single bulk copy (no tensor map needed) drops into
shared memory ready for ``tcgen05.mma``.  Weights are packed once when the model is packaged (this module, on
the CPU); activations are written in this layout by the quantisation kernel.
"""
from __future__ import annotations

WEIGHT_ROW_PAD = 256        # packed weights are padded to whole 256-row tiles (zero rows)


def padded_weight_rows(n: int) -> int:
    return (n + WEIGHT_ROW_PAD - 1) // WEIGHT_ROW_PAD * WEIGHT_ROW_PAD


def padded_token_rows(m: int) -> int:
    """Rows reserved for a packed activation matrix: any token tile of up to 256 rows stays inside."""
    return (m + 255) // 256 * 256 + 256


def pack_kblock_swizzled(t, rows_padded: int | None = None):
    """[R, K] tensor (1- or 2-byte dtype, K bytes a multiple of 128) -> same dtype, shape
    [K bytes / 128, R_padded, 128 / element size]."""
    import torch
    rows, _ = t.shape
    elem = t.element_size()
    raw = t.contiguous().view(torch.uint8).reshape(rows, -1)
    k_bytes = raw.shape[1]
    if k_bytes % 128:
        raise ValueError("K must be a whole number of 128-byte blocks")
    rp = rows_padded if rows_padded is not None else padded_weight_rows(rows)
    padded = torch.zeros(rp, k_bytes, dtype=torch.uint8)
    padded[:rows] = raw
    blocks = padded.reshape(rp, k_bytes // 128, 8, 16).permute(1, 0, 2, 3)          # [kb, r, chunk, 16]
    source_chunk = torch.arange(8)[None, :] ^ (torch.arange(rp) % 8)[:, None]       # position p holds chunk p ^ (r & 7)
    index = source_chunk[None, :, :, None].expand(blocks.shape[0], rp, 8, 16)
    out = torch.gather(blocks, 2, index).contiguous()
    return out.reshape(k_bytes // 128, rp, 128).view(t.dtype).reshape(k_bytes // 128, rp, 128 // elem)


def unpack_kblock_swizzled(p, rows: int):
    """Inverse of ``pack_kblock_swizzled`` (drops the padding rows)."""
    import torch
    kb, rp, _ = p.shape
    raw = p.contiguous().view(torch.uint8).reshape(kb, rp, 8, 16)
    source_pos = torch.arange(8)[None, :] ^ (torch.arange(rp) % 8)[:, None]          # chunk c sits at position c ^ (r & 7)
    index = source_pos[None, :, :, None].expand(kb, rp, 8, 16)
    blocks = torch.gather(raw, 2, index)
    flat = blocks.permute(1, 0, 2, 3).reshape(rp, kb * 128)[:rows].contiguous()
    return flat.view(p.dtype)

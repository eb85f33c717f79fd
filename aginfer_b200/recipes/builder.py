"""Recipe builder: model description -> ``plan.json`` / ``tactics.json`` for the sm100 bundle.

A recipe is the static launch list the loader replays: every kernel, grid, block and
argument is fixed here, offline.  The builder keeps three address spaces apart, exactly as
the plan format does (reference ``src/aginfer/plan.py:284-317``):

* profile tensors (caller buffers), referenced by name;
* the session arena, handed out by a bump allocator with 256-byte alignment; the first
  ``RESERVED`` bytes hold the status word and the per-run counters the prologue clears;
* the packed weight blob, whose offsets follow from the checkpoint's tensor names and sizes
  alone (``weights.weight_layout``), so a plan can be written before the blob exists.

One method per kernel family wraps the launch geometry ("tactic") for that kernel; each
use is recorded for ``tactics.json``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Mapping, Sequence

from ..target import CHECKPOINT_DTYPE_BYTES
from ..weights import weight_layout

ALIGN = 256
RESERVED = 1024          # bytes at arena offset 0: status word + counters, zeroed every run
STATUS_WORD = 0          # u32: first error recorded by a kernel (0 = none)
SM_COUNT = 148

FLAG_BIAS, FLAG_RESIDUAL, FLAG_OUT_F32, FLAG_SCALED = 1, 2, 1 << 8, 1 << 9
FLAG_LAYERNORM, FLAG_LN_MODULATE, FLAG_SLAB = 1 << 10, 1 << 11, 1 << 12
ACT = {None: 0, "gelu_tanh": 1 << 4, "silu": 2 << 4, "relu": 3 << 4}
PLAN_DTYPE_BYTES = {"F32": 4, "F16": 2, "BF16": 2, "F8_E4M3": 1, "I32": 4}

from .layout import padded_token_rows, padded_weight_rows


@dataclass(frozen=True)
class Tensor:
    """A profile input or output, by name."""
    name: str


@dataclass(frozen=True)
class Arena:
    """A byte offset into the session arena."""
    offset: int

    def __add__(self, nbytes: int) -> "Arena":
        return Arena(self.offset + nbytes)


@dataclass(frozen=True)
class Weight:
    """A checkpoint tensor (plus a byte offset inside it)."""
    name: str
    byte_offset: int = 0

    def __add__(self, nbytes: int) -> "Weight":
        return Weight(self.name, self.byte_offset + nbytes)


@dataclass(frozen=True)
class U32:
    value: int


@dataclass(frozen=True)
class F32:
    value: float


Pointer = Tensor | Arena | Weight


def ceil_div(a: int, b: int) -> int:
    return -(-a // b)


TC_SCRATCH_BYTES = 32 << 20    # fp32 partial tiles of split-K tensor-core GEMMs, [slice][M][N]
TC_COUNTER_BYTES = 16 << 10    # per-tile arrival counters of the same
TC_SMEM_BUDGET = 225 * 1024     # ring bytes per CTA: 227 KB opt-in limit minus barriers and alignment slack
ATTN_SMEM_BUDGET = 200 * 1024    # dynamic shared memory of the keys-in-shared-memory attention kernel
# One bulk copy per operand into unpadded rows was measured slower than one copy per row into padded rows:
# unpadded rows make every fragment read an 8-way bank conflict and shared-memory reads bound the MMA phase.
USE_SLAB_COPIES = False
# 16 weight rows per CTA use the whole 16-row MMA tile and halve the activation re-reads per weight byte; 8 rows
# give twice as many CTAs.  16 is chosen when it still yields at least this many CTAs.
STREAM_MIN_CTAS_FOR_16_ROWS = SM_COUNT
STREAM_SM_BYTES = 220 * 1024     # shared memory the bulk-stream GEMM CTAs of one SM may use together
STREAM_CTA_BYTES = 110 * 1024    # and the most a single CTA takes (two CTAs per SM keep one draining while one fills)


def tc_tiling(M: int, N: int, K: int, elem: int, splits: int | None = None) -> dict[str, int]:
    """Launch geometry of ``agi_gemm_tc_*``: token tile TN (multiple of 16, <= 256), K slices, ring depth."""
    m_tiles = ceil_div(M, 256)
    TN = ceil_div(ceil_div(M, m_tiles), 16) * 16
    n_tiles = ceil_div(N, 128)
    tiles = n_tiles * m_tiles
    k_blocks = K * elem // 128
    if splits is None:
        # fill the 148 SMs when the output has too few tiles; keep at least two K blocks per slice
        splits = 1 if tiles >= 120 else max(1, min(16, ceil_div(SM_COUNT, tiles), k_blocks // 2))
    per = ceil_div(k_blocks, max(1, min(splits, k_blocks)))
    splits = ceil_div(k_blocks, per)
    stage_bytes = 16384 + TN * 128
    stages = max(3, min(12, TC_SMEM_BUDGET // stage_bytes, max(per, 3)))
    return {"TN": TN, "m_tiles": m_tiles, "n_tiles": n_tiles, "tiles": tiles, "splits": splits, "stages": stages,
            "shared_bytes": stages * stage_bytes + 1024}


def tc_prefill_plan(M: int, N: int, K: int, elem: int) -> dict[str, int]:
    """Tile shape for a tensor-core GEMM over many tokens: weight rows per CTA (128, or 256 = the wide kernel
    with two accumulators), token tile TN, K slices.

    The kernels fill shared memory from L2 with 16-byte asynchronous copies, measured at about 32 bytes per
    clock and SM, which is slower than the tensor core consumes it; so the estimate per CTA is
    K blocks x max(fill, MMA) + set-up + epilogue, times the number of waves over 148 SMs, plus the
    slab pass of the finishing CTA when K is sliced.  The cheapest candidate wins."""
    k_blocks = K * elem // 128
    best: dict[str, int] | None = None
    for rows in (128, 256):
        if rows == 256 and N < 256:
            continue
        n_tiles = ceil_div(N, rows)
        seen = set()
        for cap in range(256, 48, -16):
            m_tiles = ceil_div(M, cap)
            TN = ceil_div(ceil_div(M, m_tiles), 16) * 16
            if TN in seen:
                continue
            seen.add(TN)
            for splits in (1, 2, 3, 4, 6, 8):
                per = ceil_div(k_blocks, splits)
                if ceil_div(k_blocks, per) != splits or (splits > 1 and per < 4):
                    continue
                if splits > 1 and splits * M * n_tiles * rows * 4 > TC_SCRATCH_BYTES:
                    continue
                if n_tiles * m_tiles * 4 > TC_COUNTER_BYTES:
                    continue
                stage_bytes = rows * 128 + TN * 128
                fill = stage_bytes / 28
                mma = (rows // 128) * TN * 2
                ctas = n_tiles * m_tiles * splits
                cost = ceil_div(ctas, SM_COUNT) * (per * max(fill, mma) + 5000 + TN * 25)
                if splits > 1:      # slab stores of every slice, then one CTA per tile reads them all back
                    cost += 4000 + rows * TN * (splits + 1) // 8
                if best is None or cost < best["cost"]:
                    stages = max(3, min(12, TC_SMEM_BUDGET // stage_bytes, max(per, 3)))
                    best = {"rows": rows, "TN": TN, "m_tiles": m_tiles, "n_tiles": n_tiles, "splits": splits,
                            "stages": stages, "shared_bytes": stages * stage_bytes + 1024, "cost": int(cost)}
    assert best is not None
    return best


def tc_group_tiling(M: int, n_tiles: int, K: int, elem: int) -> dict[str, int]:
    """Token tile and ring depth of the grouped tensor-core GEMM (128-row tiles, no K slices): the token tile
    with the cheapest estimate under the same model as ``tc_prefill_plan``."""
    k_blocks = K * elem // 128
    best: dict[str, int] | None = None
    for cap in range(256, 15, -16):
        m_tiles = ceil_div(M, cap)
        TN = ceil_div(ceil_div(M, m_tiles), 16) * 16
        stage_bytes = 16384 + TN * 128
        cost = ceil_div(n_tiles * m_tiles, SM_COUNT) * (k_blocks * max(stage_bytes / 28, TN * 2) + 5000 + TN * 25)
        if best is None or cost < best["cost"]:
            stages = max(3, min(12, TC_SMEM_BUDGET // stage_bytes, max(k_blocks, 3)))
            best = {"TN": TN, "m_tiles": m_tiles, "stages": stages, "shared_bytes": stages * stage_bytes + 1024,
                    "cost": int(cost)}
    assert best is not None
    return best


# K >= ratio * N counts as K-heavy; 0 (default) disables the rule: in isolation the cluster kernel wins there
# (17 tokens, 1536 x 6144: 9.4 us against 11.3 us), inside the action-head graph it does not (2.96 ms per chunk
# against 2.93 ms), because the weight-streaming kernel starts its copies before the previous kernel has finished
CLUSTER_K_RATIO = 0
PERSIST_TOKEN_SPLITS = 4             # token-tile counts the persistent GEMM's planner tries beyond the minimum
FA_HEAD_DIMS = (48, 64, 80, 128)   # compiled widths of agi_attention_fa_bf16_d*


TC_CLUSTER_SIZES = {"bf16": (2, 3, 4, 6, 8), "e4m3": (2, 4, 8)}   # compiled cluster variants


def tc_cluster_tiling(M: int, N: int, K: int, elem: int, dtype: str = "bf16",
                      sizes: Sequence[int] | None = None) -> dict[str, int] | None:
    """Geometry of ``agi_gemm_tc_*_c{C}``: the largest compiled cluster size that keeps all CTAs in one wave
    (n_tiles * C <= 148) and leaves every slice at least two K blocks."""
    if M > 64 or (K * elem) % 128:
        return None
    TN = ceil_div(M, 16) * 16
    n_tiles = ceil_div(N, 128)
    k_blocks = K * elem // 128
    usable = [c for c in (sizes or TC_CLUSTER_SIZES[dtype]) if n_tiles * c <= SM_COUNT and k_blocks >= 2 * c]
    if not usable:
        return None
    cluster = max(usable)
    per = ceil_div(k_blocks, cluster)
    if ceil_div(k_blocks, per) != cluster:      # every rank of the cluster must own a non-empty slice
        return None
    stage_bytes = 16384 + TN * 128
    gather_bytes = cluster * ceil_div(TN, cluster) * 512
    stages = max(3, min(12, (TC_SMEM_BUDGET - gather_bytes) // stage_bytes, per))
    return {"TN": TN, "n_tiles": n_tiles, "cluster": cluster, "stages": stages,
            "shared_bytes": stages * stage_bytes + 1024 + gather_bytes}


TCS_CLUSTER_SIZES = (2, 3, 4, 6, 8)       # compiled cluster variants of agi_gemm_tcs_bf16
TCS_MAX_BLOCKS = 8                        # K blocks of 64 elements per slice: the slab a CTA requests at once (128 KB)
TCS_TARGET_CTAS = 2 * SM_COUNT            # two CTAs per SM keep the SM's copy engine busy while one of them computes


def tcs_tiling(M: int, tiles: int, K: int, cluster: int | None = None, groups: int | None = None,
               kb: int | None = None) -> dict[str, int] | None:
    """Geometry of ``agi_gemm_tcs_bf16[_c{C}]`` (packed bf16 weights, at most 32 tokens): K is cut into
    ``cluster * groups`` slices of ``kb`` blocks of 64 elements; the slices of a cluster meet in distributed shared
    memory, the ``groups`` clusters of a tile (or, with cluster 1, all slices) in global fp32 slabs.

    Chosen: the most slices that keep the grid within two CTAs per SM with at least two K blocks each; one
    cluster per tile when eight slices of at most TCS_MAX_BLOCKS cover K, several clusters otherwise."""
    if M > 32 or K % 64:
        return None
    k_blocks = K // 64
    if cluster is None or groups is None or kb is None:
        options = [s for s in range(1, 33) if k_blocks % s == 0 and 2 <= k_blocks // s <= TCS_MAX_BLOCKS
                   and tiles * s <= TCS_TARGET_CTAS]
        if not options:
            options = [s for s in range(1, 33) if k_blocks % s == 0 and k_blocks // s <= TCS_MAX_BLOCKS][:1]
        if not options:
            return None
        slices = max(options)
        if slices > 8 and k_blocks % 8 == 0 and k_blocks // 8 <= TCS_MAX_BLOCKS:
            slices = 8
        if slices in (1, *TCS_CLUSTER_SIZES):
            cluster, groups = slices, 1
        else:
            cluster = max((c for c in TCS_CLUSTER_SIZES if slices % c == 0 and slices // c <= 4), default=None)
            if cluster is None:
                return None
            groups = slices // cluster
        kb = k_blocks // slices
    slices = cluster * groups
    assert slices * kb >= k_blocks and kb <= TCS_MAX_BLOCKS and (cluster == 1 or cluster in TCS_CLUSTER_SIZES)
    assert slices <= 16 if cluster == 1 else groups <= 4
    gather = cluster * ceil_div(32, cluster) * 512 if cluster > 1 else 0
    return {"cluster": cluster, "groups": groups, "kb": kb, "slices": slices, "ctas": tiles * slices,
            "shared_bytes": kb * 20480 + 1024 + gather}


STREAM_SPLITS = (4, 2)          # compiled cluster sizes of agi_gemm_stream_bf16_t{1..4}_k{S}


def stream_tiling(M: int, N: int, K: int, elem: int, extra_rows: int = 0, contiguous: bool = True,
                  splits: int = 1) -> dict[str, int]:
    """Launch geometry of ``agi_gemm_stream_*``: rows per CTA, K windows per ring slot, slots.

    Aim: at least one CTA per SM when N allows it, every CTA resident at once (one wave), and the shared
    memory of an SM split evenly between the CTAs that share it, so that as many bytes as possible are
    in flight.  16 rows per CTA halve the activation traffic per weight byte and are used when N is large
    enough to still give every SM a CTA.  ``splits`` > 1: K is cut into that many slices, one CTA of a
    thread-block cluster each (the geometry is that of one slice; ``grid`` stays the number of row groups)."""
    rows = 16 if ceil_div(N, 16) * splits >= STREAM_MIN_CTAS_FOR_16_ROWS else 8
    grid = ceil_div(N, rows)
    per_sm = ceil_div(grid * splits, SM_COUNT)
    tiles = next(v for v in (1, 2, 3, 4, 6, 8) if 8 * v >= M)
    warps = 4                                           # consumer warps (plus one producer warp)
    tail = 16 + warps * 16 * (M | 1) * 4                # alignment slack + the warps' partial tiles
    tail += (splits - 1) * rows * M * 4                 # + the other slices' partial sums, gathered by slice 0
    budget = min(STREAM_CTA_BYTES, STREAM_SM_BYTES // per_sm) - tail
    windows = K // splits * elem // 64
    row_bytes = lambda w: w * 64 + 16
    held = rows + M + extra_rows   # rows of a ring slot: weights, activations
    common = {"rows": rows, "grid": grid, "tiles": tiles, "threads": (warps + 1) * 32}
    if USE_SLAB_COPIES and contiguous and held * windows * 64 <= budget:
        # whole K in one slot: unpadded rows, one bulk copy per operand ("slab" mode)
        return {**common, "chunk_windows": windows, "slots": 1, "slab": True, "shared_bytes": held * windows * 64 + tail}
    if held * row_bytes(windows) <= budget:
        chunk_windows, slots = windows, 1
    else:
        chunk_windows = max(1, (budget // 2 // held - 16) // 64)
        slots = 2
    return {**common, "chunk_windows": chunk_windows, "slots": slots, "slab": False,
            "shared_bytes": slots * held * row_bytes(chunk_windows) + tail}


def stream_splits(M: int, N: int, K: int, elem: int) -> int:
    """K slices for the bulk-stream GEMM.  One ring that wraps many times pays a round trip to memory per wrap
    (1536 x 6144 at 17 tokens: six chunks through two slots, 10.5 us); the same matrix as four slices side by
    side, each the shape of a 1536-wide product, has nothing to wait for twice.  Slices are used when the single
    ring would need more than four chunks and the sliced grid still fits three CTAs per SM."""
    if elem != 2 or M > 32:
        return 1
    t = stream_tiling(M, N, K, elem)
    if ceil_div(K * elem // 64, t["chunk_windows"]) <= 4:
        return 1
    for s in STREAM_SPLITS:
        if K % (s * 32) == 0 and ceil_div(N, 16) * s <= 3 * SM_COUNT:
            return s
    return 1


# ---- persistent block kernel (csrc/kernels/dit_block.cuh) ------------------------------------------------
DIT_TABLE_ORDER = ("to_q.weight", "to_q.bias", "to_k.weight", "to_k.bias", "to_v.weight", "to_v.bias", "to_out.weight",
                   "to_out.bias", "fc1.weight", "fc1.bias", "fc2.weight", "fc2.bias", "adaln", "context_k", "context_v")
DIT_SLOT_BYTES = 16 * (16 * 64 + 64)     # a ring slot: 16 weight rows x (1 KB + 64 bytes of padding)
DIT_HEADER_BYTES = 256
DIT_MAX_SPAN = 1536                      # K elements a consumer warp keeps as MMA B fragments
MAX_DYNAMIC_SHARED = 227 * 1024


def dit_block_span(mlp: int) -> int | None:
    """K span of the MLP down projection: the largest divisor of ``mlp`` that is a multiple of 32 and at most 1536."""
    return next((s for s in range(min(mlp, DIT_MAX_SPAN) // 32 * 32, 0, -32) if mlp % s == 0), None)


def dit_block_geometry(T: int, D: int, heads: int, head_dim: int, mlp: int, ctx: int, layers: int) -> dict[str, int] | None:
    """Shared-memory plan of the persistent block kernel, or None when the shape is outside its limits
    (mirrors ``ditb::exchange_bytes`` and ``ditb::attention_bytes``)."""
    span = dit_block_span(mlp)
    if (span is None or not 1 <= T <= 24 or D % 32 or D > DIT_MAX_SPAN or mlp % 16 or head_dim % 16 or head_dim > 64
            or heads * head_dim != D or not 1 <= layers <= 32 or ctx < 1):
        return None
    # then the attention tile (keys and values of a head)
    # the table's copy, the consumers' exchange area (partial tiles, row statistics), AdaLN scale | shift
    exchange = 32 * 16 * 8 + ceil_div(8 * 16 * (T | 1) * 4 + 2 * 8 * 24 * 4 + 64, 128) * 128 + 4 * DIT_MAX_SPAN
    keys = ceil_div(max(ctx, T), 16) * 16
    attention = ceil_div(max(2 * keys * (head_dim + 8) * 2, 8 * 16 * (head_dim + 2) * 4), 128) * 128
    region = exchange + attention
    slots = min(12, (MAX_DYNAMIC_SHARED - DIT_HEADER_BYTES - region) // DIT_SLOT_BYTES)
    if slots < 3:
        return None
    return {"slots": slots, "region": region, "shared_bytes": DIT_HEADER_BYTES + region + slots * DIT_SLOT_BYTES}


def grid_for(work_items: int, threads: int = 256, cap: int = SM_COUNT * 8) -> int:
    return max(1, min(cap, ceil_div(work_items, threads)))


@dataclass
class Profile:
    name: str
    inputs: list[dict[str, Any]] = field(default_factory=list)
    outputs: list[dict[str, Any]] = field(default_factory=list)
    launches: list[dict[str, Any]] = field(default_factory=list)
    graph_safe: bool = True


class RecipeBuilder:
    def __init__(self, weights: Mapping[str, tuple[str, Sequence[int]]], arch: str = "sm100",
                 counter_slots: int = (RESERVED - 64) // 4):
        """``counter_slots``: u32 slots cleared by every run's first launch (one per dynamic quantisation)."""
        self.arch = arch
        self.reserved = ceil_div(64 + 4 * counter_slots, ALIGN) * ALIGN
        self.weights = {k: (d, tuple(s)) for k, (d, s) in weights.items()}
        sizes = {k: math.prod(s) * CHECKPOINT_DTYPE_BYTES[d] for k, (d, s) in self.weights.items()}
        self.weight_offsets, self.weight_bytes = weight_layout(sizes)
        self.weight_sizes = sizes
        self._cursor = self.reserved
        self._high_water = self.reserved
        self._counter_cursor = 64          # counters live in [64, RESERVED); [0, 64) is the status area
        self.profiles: list[Profile] = []
        self.tactics: dict[tuple[str, str], dict[str, Any]] = {}
        self._profile: Profile | None = None
        # Split-K scratch of the tensor-core GEMMs lives outside the stack discipline of alloc/release:
        # its arrival counters must stay zero between launches for the whole life of the session.
        self._tc_scratch = (self.alloc(TC_SCRATCH_BYTES), self.alloc(TC_COUNTER_BYTES))
        self._dit_scratch: dict[tuple[int, int, int], tuple[Arena, Arena]] = {}

    # ---- address spaces -------------------------------------------------------------------
    def alloc(self, nbytes: int, align: int = ALIGN) -> Arena:
        at = ceil_div(self._cursor, align) * align
        self._cursor = at + max(nbytes, 1)
        self._high_water = max(self._high_water, self._cursor)
        return Arena(at)

    def mark(self) -> int:
        return self._cursor

    def release(self, mark: int) -> None:
        """Give back everything allocated since ``mark`` (stack discipline)."""
        self._cursor = mark

    def counter(self, words: int = 1) -> Arena:
        """A zero-at-run-start u32 slot (amax accumulators, flags)."""
        at = self._counter_cursor
        self._counter_cursor += 4 * words
        if self._counter_cursor > self.reserved:
            raise ValueError("out of per-run counter slots")
        return Arena(at)

    @property
    def arena_bytes(self) -> int:
        return ceil_div(self._high_water, ALIGN) * ALIGN

    # ---- profiles -------------------------------------------------------------------------
    def begin_profile(self, name: str, inputs: Sequence[dict[str, Any]], outputs: Sequence[dict[str, Any]],
                      graph_safe: bool = True) -> None:
        self._profile = Profile(name, [dict(i) for i in inputs], [dict(o) for o in outputs], [], graph_safe)
        self.profiles.append(self._profile)
        self._counter_cursor = 64          # every profile clears the counter area itself, so slots are per profile
        # prologue: clear status word and counters
        self.launch("agi_fill_u32", (1, 1, 1), (256, 1, 1), [Arena(0), U32(0), U32(self.reserved // 4)],
                    op="prologue", algorithm="fill_u32")

    def _encode(self, arg: Any) -> dict[str, Any]:
        if isinstance(arg, Tensor):
            return {"tensor": arg.name}
        if isinstance(arg, Arena):
            return {"arena_offset": arg.offset}
        if isinstance(arg, Weight):
            if arg.name not in self.weight_offsets:
                raise KeyError(f"recipe references unknown weight {arg.name!r}")
            if arg.byte_offset >= max(self.weight_sizes[arg.name], 1):
                raise ValueError(f"offset {arg.byte_offset} is outside weight {arg.name!r}")
            return {"weights_offset": self.weight_offsets[arg.name] + arg.byte_offset}
        if isinstance(arg, U32):
            return {"scalar_u32": int(arg.value)}
        if isinstance(arg, F32):
            return {"scalar_f32": float(arg.value)}
        raise TypeError(f"not a kernel argument: {arg!r}")

    def launch(self, kernel: str, grid: Sequence[int], block: Sequence[int], args: Sequence[Any], *,
               shared_bytes: int = 0, op: str | None = None, algorithm: str | None = None, **tactic: Any) -> None:
        assert self._profile is not None, "begin_profile first"
        self._profile.launches.append({"kernel": kernel, "grid": list(grid), "block": list(block),
                                       "shared_bytes": shared_bytes, "arguments": [self._encode(a) for a in args]})
        key = (op or kernel, algorithm or kernel)
        entry = self.tactics.setdefault(key, {"op": key[0], "algorithm": key[1], "kernel": kernel, "uses": 0, **tactic})
        entry["uses"] += 1

    def launch_count(self) -> int:
        assert self._profile is not None, "begin_profile first"
        return len(self._profile.launches)

    def drop_launches(self, first: int, kernel: str) -> None:
        """Remove the launches of ``kernel`` emitted since ``launch_count()`` returned ``first`` (measurement
        profiles that replay a sub-sequence of another profile's launches exactly as that profile emits them)."""
        assert self._profile is not None, "begin_profile first"
        self._profile.launches[first:] = [l for l in self._profile.launches[first:] if l["kernel"] != kernel]

    # ---- kernel families ------------------------------------------------------------------
    def export_status(self, out: Pointer) -> None:
        """Copy the status word (0 = every bounded wait succeeded) into a caller-visible I32 tensor."""
        self.launch("agi_copy_u32", (1, 1, 1), (32, 1, 1), [Arena(STATUS_WORD), out, U32(1)], op="export_status")

    def vector_add(self, left: Pointer, right: Pointer, out: Pointer, count: int) -> None:
        self.launch("vector_add_f32", (ceil_div(count, 256), 1, 1), (256, 1, 1), [left, right, out, U32(count)],
                    op="vector_add")

    def quantize_e4m3(self, x: Pointer, q: Pointer, scale_out: Pointer, count: int, amax: Pointer | None = None,
                      packed: tuple[int, int] | None = None) -> None:
        """amax -> scale = amax / 448 -> q = e4m3(x / scale); two launches sharing one counter, or one launch
        when the producer of ``x`` already folded max |x| into ``amax`` (a ``counter()`` slot).
        ``packed=(rows, cols)`` writes ``q`` in the packed operand layout of the bulk-copy GEMM
        (``recipes/layout.py``; ``q`` needs ``padded_token_rows(rows) * cols`` bytes)."""
        blocks = grid_for(count // 8 + 1, 256, SM_COUNT * 4)
        if amax is None:
            amax = self.counter()
            self.launch("agi_absmax_bf16", (blocks, 1, 1), (256, 1, 1), [x, U32(count), amax], op="absmax")
        if packed is not None:
            rows, cols = packed
            assert rows * cols == count and cols % 128 == 0
            self.launch("agi_quantize_e4m3_packed_bf16", (grid_for(count // 16, 256, SM_COUNT * 4), 1, 1), (256, 1, 1),
                        [x, q, amax, scale_out, U32(rows), U32(cols), U32(padded_token_rows(rows))],
                        op="quantize_e4m3_packed")
            return
        self.launch("agi_quantize_e4m3_bf16", (blocks, 1, 1), (256, 1, 1), [x, q, amax, scale_out, U32(count)],
                    op="quantize_e4m3")

    def rmsnorm(self, x: Pointer, gain: Pointer, y: Pointer, rows: int, cols: int, eps: float = 1e-6,
                x_stride: int | None = None, y_stride: int | None = None, amax: Pointer | None = None) -> None:
        """``amax``: a ``counter()`` slot that receives max |y| for a following ``quantize_e4m3(..., amax=)``."""
        assert cols % 8 == 0
        args = [x, gain, y, U32(rows), U32(cols), U32(x_stride or cols), U32(y_stride or cols), F32(eps)]
        self.launch("agi_rmsnorm_amax_bf16" if amax is not None else "agi_rmsnorm_bf16", (rows, 1, 1),
                    (min(1024, max(32, ceil_div(cols // 8, 32) * 32)), 1, 1), args + ([amax] if amax is not None else []),
                    op="rmsnorm_amax" if amax is not None else "rmsnorm")

    def layernorm(self, x: Pointer, y: Pointer, rows: int, cols: int, eps: float = 1e-5,
                  scale: Pointer | None = None, shift: Pointer | None = None,
                  x_stride: int | None = None, y_stride: int | None = None) -> None:
        assert cols % 8 == 0 and (scale is None) == (shift is None)
        dummy = Arena(0)
        self.launch("agi_layernorm_bf16", (rows, 1, 1), (min(1024, max(32, ceil_div(cols // 8, 32) * 32)), 1, 1),
                    [x, scale or dummy, shift or dummy, y, U32(rows), U32(cols), U32(x_stride or cols),
                     U32(y_stride or cols), F32(eps), U32(0 if scale is None else 1)],
                    op="layernorm_modulate" if scale is not None else "layernorm")

    def rope(self, x: Pointer, rows: int, heads: int, head_dim: int, row_stride: int, theta: float,
             pos_offset: int = 0) -> None:
        work = rows * heads * head_dim // 2
        self.launch("agi_rope_bf16", (grid_for(work), 1, 1), (256, 1, 1),
                    [x, U32(rows), U32(heads), U32(head_dim), U32(row_stride), F32(math.log2(theta)), U32(pos_offset)],
                    op="rope")

    def rope_pair(self, x0: Pointer, heads0: int, row_stride0: int, x1: Pointer, heads1: int, row_stride1: int,
                  rows: int, head_dim: int, theta: float, pos_offset: int = 0) -> None:
        """``rope`` over two tensors (queries and new keys in separate buffers) as one launch."""
        work = rows * (heads0 + heads1) * head_dim // 2
        self.launch("agi_rope_pair_bf16", (grid_for(work), 1, 1), (256, 1, 1),
                    [x0, U32(heads0), U32(row_stride0), x1, U32(heads1), U32(row_stride1), U32(rows), U32(head_dim),
                     F32(math.log2(theta)), U32(pos_offset)], op="rope")

    def mrope(self, x: Pointer, positions: Pointer, rows: int, heads: int, head_dim: int, row_stride: int,
              theta: float, sections: Sequence[int], ladder: int | None = None) -> None:
        """``ladder``: rotary pairs per frequency ladder (pair i turns at theta^(-(i mod ladder) / ladder));
        default head_dim / 2, the single ladder of a language model."""
        assert sum(sections) == head_dim // 2 and len(sections) == 3
        work = rows * heads * head_dim // 2
        self.launch("agi_mrope_bf16", (grid_for(work), 1, 1), (256, 1, 1),
                    [x, positions, U32(rows), U32(heads), U32(head_dim), U32(row_stride), F32(math.log2(theta)),
                     U32(sections[0]), U32(sections[1]), U32(ladder or head_dim // 2)], op="mrope")

    def attention(self, q: Pointer, k: Pointer, v: Pointer, o: Pointer, *, q_rows: int, kv_rows: int, q_heads: int,
                  kv_heads: int, head_dim: int, q_stride: int, k_stride: int, v_stride: int, o_stride: int,
                  mask: str = "none", mask_arg: int = 0, scale: float | None = None,
                  algorithm: str = "auto", amax: Pointer | None = None, kv_static: bool = False,
                  kv_static_rows: int | None = None) -> None:
        """``amax`` (a ``counter()`` slot; head widths 80 and 128, streaming tensor-core kernel only): the kernel
        also leaves max |o| there for a following ``quantize_e4m3(..., amax=)``.
        ``kv_static``: keys and values were written before the last ``agi_add_rows_bf16`` launch of the profile
        (which releases its successors only after its own wait), not by the launches since; the few-query-rows
        kernel then requests them before its grid-dependency wait.  ``kv_static_rows``: only that many leading rows
        (the prefix of a KV cache whose tail the previous launches just wrote)."""
        assert head_dim <= 128 and head_dim % 2 == 0 and q_heads % kv_heads == 0
        mode = {"none": 0, "causal": 1, "block": 2}[mask]
        args = [q, k, v, o, U32(q_rows), U32(kv_rows), U32(q_heads), U32(kv_heads), U32(head_dim), U32(q_stride),
                U32(k_stride), U32(v_stride), U32(o_stride), F32(scale if scale is not None else head_dim ** -0.5),
                U32(mode), U32(mask_arg)]
        # keys one block of 8 query rows can see: everything, or one diagonal block (plus alignment slack)
        span = kv_rows if mask != "block" else min(kv_rows, mask_arg * (1 + ceil_div(8, mask_arg)))
        span_pad = ceil_div(span, 32) * 32
        smem = span * (2 * head_dim + 2) * 2 + 16 + 8 * head_dim * 4 + 8 * span_pad * 4
        aligned = head_dim % 8 == 0 and k_stride % 8 == 0 and v_stride % 8 == 0
        rows_smem = (ceil_div(kv_rows * (head_dim + 2), 8) * 16 + kv_rows * head_dim * 2 + q_rows * head_dim * 4
                     + q_rows * ceil_div(kv_rows, 32) * 32 * 4 + 8 * q_rows * head_dim * 4 + 2 * 8 * q_rows * 4)
        kv16 = ceil_div(kv_rows, 16) * 16
        mma_smem = 2 * kv16 * (head_dim + 8) * 2 + 8 * 16 * (head_dim + 2) * 4
        if (aligned and q_rows <= 64 and head_dim <= 64 and head_dim % 16 == 0 and q_stride % 2 == 0 and o_stride % 2 == 0
                and mma_smem <= ATTN_SMEM_BUDGET and algorithm in ("auto", "mma")):
            # few query rows: one block per head, tensor-core scores and P.V
            if kv_static:
                args = args[:14] + [U32(mode | 0x100 | (min(kv_static_rows or 0, 0xffff) << 16)), args[15]]
            self.launch("agi_attention_mma_bf16", (q_heads, ceil_div(q_rows, 16), 1), (256, 1, 1), args, shared_bytes=mma_smem,
                        op=f"attention_{mask}", algorithm="mma_key_split" + ("_early_kv" if kv_static else ""))
            return
        wide_smem = max(2 * kv16 * (head_dim + 8) * 2, 8 * 16 * (head_dim + 2) * 4)
        if (aligned and q_rows <= 64 and 64 < head_dim <= 128 and head_dim % 16 == 0 and q_stride % 2 == 0 and o_stride % 2 == 0
                and wide_smem <= ATTN_SMEM_BUDGET and amax is None and algorithm in ("auto", "mma")):
            # few query rows, wide heads: the streaming kernel would give each of a handful of warps every key
            if kv_static:
                args = args[:14] + [U32(mode | 0x100 | (min(kv_static_rows or 0, 0xffff) << 16)), args[15]]
            self.launch("agi_attention_mma_bf16_d128", (q_heads, ceil_div(q_rows, 16), 1), (256, 1, 1), args,
                        shared_bytes=wide_smem, op=f"attention_{mask}",
                        algorithm="mma_key_split_d128" + ("_early_kv" if kv_static else ""))
            return
        # streaming tensor-core kernel: 4, 2 or 1 warps (64, 32 or 16 query rows) per block, the most rows that still
        # give the grid about one block per SM
        fa_warps = next((wp for wp in (4, 2, 1) if ceil_div(q_rows, 16 * wp) * q_heads >= 96), 1)
        if amax is not None:
            assert aligned and head_dim in (80, 128) and q_stride % 2 == 0 and o_stride % 2 == 0 and (q_rows > 64 or head_dim > 64)
            self.launch(f"agi_attention_fa_amax_bf16_d{head_dim}", (ceil_div(q_rows, 16 * fa_warps), q_heads, 1), (32 * fa_warps, 1, 1),
                        args + [amax], shared_bytes=4 * 64 * (head_dim + 8) * 2, op=f"attention_{mask}_amax",
                        algorithm="mma_streaming")
            return
        if (aligned and head_dim in FA_HEAD_DIMS and q_stride % 2 == 0 and o_stride % 2 == 0
                and algorithm in ("auto", "fa")):
            # many query rows: streaming softmax on tensor cores, 64 rows per block, keys in tiles of 64
            self.launch(f"agi_attention_fa_bf16_d{head_dim}", (ceil_div(q_rows, 16 * fa_warps), q_heads, 1), (32 * fa_warps, 1, 1), args,
                        shared_bytes=4 * 64 * (head_dim + 8) * 2, op=f"attention_{mask}", algorithm="mma_streaming")
            return
        if (aligned and q_rows <= 32 and head_dim <= 64 and rows_smem <= ATTN_SMEM_BUDGET
                and algorithm in ("auto", "key_split")):
            # few query rows: one block per head, warps split the keys
            self.launch("agi_attention_rows_bf16", (q_heads, 1, 1), (256, 1, 1), args, shared_bytes=rows_smem,
                        op=f"attention_{mask}", algorithm="key_split")
            return
        if aligned and smem <= ATTN_SMEM_BUDGET and algorithm != "warp_per_row":
            self.launch("agi_attention_smem_bf16", (ceil_div(q_rows, 8), q_heads, 1), (256, 1, 1), args + [U32(span)],
                        shared_bytes=smem, op=f"attention_{mask}", algorithm="keys_in_smem")
            return
        self.launch("agi_attention_bf16", (ceil_div(q_rows, 8), q_heads, 1), (256, 1, 1), args,
                    op=f"attention_{mask}", algorithm="warp_per_row")

    def swiglu(self, gate: Pointer, up: Pointer, out: Pointer, rows: int, cols: int, in_stride: int,
               out_stride: int | None = None, amax: Pointer | None = None) -> None:
        assert cols % 8 == 0
        args = [gate, up, out, U32(rows), U32(cols), U32(in_stride), U32(out_stride or cols)]
        self.launch("agi_swiglu_amax_bf16" if amax is not None else "agi_swiglu_bf16",
                    (grid_for(rows * cols // 8), 1, 1), (256, 1, 1), args + ([amax] if amax is not None else []),
                    op="swiglu_amax" if amax is not None else "swiglu")

    def gemm(self, x: Pointer, w: Pointer, y: Pointer, M: int, N: int, K: int, *, dtype: str = "bf16",
             bias: Pointer | None = None, residual: Pointer | None = None, act: str | None = None,
             scale_a: Pointer | None = None, scale_w: Pointer | None = None, ldx: int | None = None,
             ldy: int | None = None, out_f32: bool = False, tactic: str = "auto",
             splits: int | None = None, packed: bool = False) -> None:
        """Y[M, N] = epilogue(X[M, K] . W[N, K]^T); ``dtype`` names the operand type (bf16 or e4m3).
        ``packed`` (E4M3 only): both operands are in the packed layout of ``recipes/layout.py`` (weights packed
        at packaging time, activations by ``quantize_e4m3(..., packed=)``) and ring slots are filled by bulk copies."""
        if dtype == "bf16" and self.is_packed(w):
            assert not out_f32 and scale_a is None, "the packed bf16 GEMM writes bf16 and takes no scales"
            self.gemm_tcs(x, [(w, bias, N)], y, M, K, residual=residual, act=act, ldx=ldx, ldy=ldy)
            return
        if packed:
            assert dtype == "e4m3" and K % 128 == 0 and ldx is None
            t = tc_prefill_plan(M, N, K, 1)
            flags = ACT[act] | (FLAG_BIAS if bias else 0) | (FLAG_RESIDUAL if residual else 0) | \
                (FLAG_OUT_F32 if out_f32 else 0) | (FLAG_SCALED if scale_a else 0)
            dummy = Arena(0)
            # more 128 x TN output tiles than SMs: the persistent kernel (one CTA per SM walks the tiles, two
            # accumulators in tensor memory, epilogue of one tile under the multiplication of the next)
            # token tile: the split of M whose tile count divides best over the SMs (rounds x bytes per tile;
            # measured: a K block of 16 KB + TN * 128 B takes ~1 cycle per 40 bytes, the MMA 2 * TN cycles)
            m_tiles, TN, tiles = 0, 0, 0
            best_cost = None
            for mt in range(ceil_div(M, 256), ceil_div(M, 256) + PERSIST_TOKEN_SPLITS):
                tn = ceil_div(ceil_div(M, mt), 16) * 16
                if tn < 16:
                    break
                count = ceil_div(N, 128) * mt
                cost = ceil_div(count, SM_COUNT) * max((16384 + tn * 128) / 40, 2 * tn)
                if best_cost is None or cost < best_cost:
                    best_cost, m_tiles, TN, tiles = cost, mt, tn, count
            # also preferred over K slices while K is short (1280 x 3456, 512 tokens: 13.6 us against 18.6 us with two
            # slices); with 86 or more K blocks per tile the slices win (2048 x 11008, 288 tokens: 24.8 us against 32.5 us)
            # ... unless there are enough tokens for the tile loop to cover the SMs by itself (1024 tokens: 35.8 us against 42.3 us)
            short_k = t["splits"] > 1 and (K // 128 <= 48 or M >= 768)
            if tactic in ("auto", "persistent") and (tiles >= 2 * SM_COUNT or short_k or tactic == "persistent"):
                stage_bytes = 16384 + TN * 128
                stages = max(2, min(12, TC_SMEM_BUDGET // stage_bytes))
                self.launch("agi_gemm_tcq_e4m3", (min(tiles, SM_COUNT), 1, 1), (192, 1, 1),
                            [x, w, y, bias or dummy, residual or dummy, scale_a or dummy, scale_w or dummy,
                             Arena(STATUS_WORD), U32(M), U32(N), U32(K), U32(padded_token_rows(M)), U32(ldy or N),
                             U32(flags), U32(TN), U32(stages)], shared_bytes=stages * stage_bytes + 1024,
                            op="gemm_e4m3_packed", algorithm=f"tcgen05_persistent_128x{TN}_s{stages}")
                return
            partial, counters = self._tc_scratch
            wide = t["rows"] == 256
            self.launch("agi_gemm_tcp_wide_e4m3" if wide else "agi_gemm_tcp_e4m3", (t["n_tiles"], t["m_tiles"], t["splits"]),
                        (288 if wide else 160, 1, 1),
                        [x, w, y, bias or dummy, residual or dummy, scale_a or dummy, scale_w or dummy, partial, counters,
                         Arena(STATUS_WORD), U32(M), U32(N), U32(K), U32(padded_token_rows(M)), U32(ldy or N), U32(flags),
                         U32(t["TN"]), U32(t["stages"])], shared_bytes=t["shared_bytes"], op="gemm_e4m3_packed",
                        algorithm=f"tcgen05_bulk_{t['rows']}x{t['TN']}_s{t['stages']}_k{t['splits']}")
            return
        flags = ACT[act] | (FLAG_BIAS if bias else 0) | (FLAG_RESIDUAL if residual else 0) | \
            (FLAG_OUT_F32 if out_f32 else 0) | (FLAG_SCALED if scale_a else 0)
        assert (scale_a is None) == (scale_w is None)
        dummy = Arena(0)
        args = [x, w, y, bias or dummy, residual or dummy, scale_a or dummy, scale_w or dummy, U32(M), U32(N), U32(K),
                U32(ldx or K), U32(ldy or N), U32(flags)]
        elem = 1 if dtype == "e4m3" else 2
        aligned = ((ldx or K) * elem) % 16 == 0
        if tactic == "auto":
            # <= 64 tokens: weight-streaming kernel (whole 64-byte K windows); otherwise the tensor-core
            # kernel (whole 128-byte K blocks); anything else falls back to the CUDA-core kernel.
            if M <= 64 and (K * elem) % 64 == 0 and aligned:
                tactic = "stream"
                # 33-64 tokens: the weight-streaming kernel needs 5-8 token tiles of accumulators per warp and
                # slows down (50 tokens, 4096 x 1024: 18.8 us), while the tensor-core kernel with its K slices in
                # a thread-block cluster does not care about the token count (8.6 us)
                k_heavy = CLUSTER_K_RATIO > 0 and K >= CLUSTER_K_RATIO * N
                if (M > 32 or k_heavy) and tc_cluster_tiling(M, N, K, elem, dtype) is not None:
                    tactic = "cluster"
            elif (K * elem) % 128 == 0 and aligned:
                tactic = "tcgen05_plan" if M >= 128 else "tcgen05"
            else:
                tactic = "simt"
        if tactic == "stream":
            # both operands reach shared memory by bulk copies; K is cut into chunks of <= ~100 KB per slot
            if M > 64 or (K * elem) % 64 or not aligned:
                raise ValueError("stream GEMM needs M <= 64, K bytes % 64 == 0 and 16-byte aligned rows")
            S = stream_splits(M, N, K, elem) if dtype == "bf16" and not out_f32 and scale_a is None else 1
            if S > 1:
                t = stream_tiling(M, N, K, elem, splits=S)
                self.launch(f"agi_gemm_stream_bf16_t{t['tiles']}_k{S}", (t["grid"], 1, S), (t["threads"], 1, 1),
                            [x, w, y, bias or dummy, residual or dummy, Arena(STATUS_WORD), U32(M), U32(N), U32(K // S),
                             U32(ldx or K), U32(ldy or N), U32(flags), U32(t["rows"]), U32(t["chunk_windows"]), U32(K)],
                            shared_bytes=t["shared_bytes"], op="gemm_bf16",
                            algorithm=f"bulk_stream_r{t['rows']}_t{t['tiles']}_c{t['chunk_windows']}_k{S}")
                return
            t = stream_tiling(M, N, K, elem, contiguous=(ldx or K) == K)
            rows, chunk_windows, tiles = t["rows"], t["chunk_windows"], t["tiles"]
            if t["slab"]:
                args = args[:12] + [U32(flags | FLAG_SLAB)]
            self.launch(f"agi_gemm_stream_{dtype}_t{tiles}", (ceil_div(N, rows), 1, 1), (t["threads"], 1, 1),
                        args[:7] + [Arena(STATUS_WORD)] + args[7:] + [U32(rows), U32(chunk_windows)],
                        shared_bytes=t["shared_bytes"], op=f"gemm_{dtype}",
                        algorithm=f"bulk_stream_r{rows}_t{tiles}_c{chunk_windows}" + ("_slab" if t["slab"] else ""))
            return
        if tactic == "skinny":
            if M > 64 or (K * elem) % 64 or not aligned:
                raise ValueError("skinny GEMM needs M <= 64, K bytes % 64 == 0 and 16-byte aligned rows")
            rows = 16 if ceil_div(N, 16) >= SM_COUNT else 8
            tiles = next(t for t in (1, 2, 3, 4, 6, 8) if 8 * t >= M)
            self.launch(f"agi_gemm_skinny_{dtype}_t{tiles}", (ceil_div(N, rows), 1, 1), (256, 1, 1), args + [U32(rows)],
                        op=f"gemm_{dtype}", algorithm=f"skinny_stream_r{rows}_t{tiles}")
            return
        if tactic == "simt":
            self.launch(f"agi_gemm_simt_{dtype}", (ceil_div(N, 64), ceil_div(M, 64), 1), (256, 1, 1), args,
                        op=f"gemm_{dtype}", algorithm="simt_64x64x16")
            return
        if tactic == "cluster":
            # tcgen05 with the K slices of a tile forming a thread-block cluster; partial sums meet in
            # distributed shared memory (no global scratch, no atomics)
            t = tc_cluster_tiling(M, N, K, elem, dtype)
            if t is None:
                raise ValueError("cluster split-K needs M <= 64, whole 128-byte K blocks and a usable cluster size")
            self.launch(f"agi_gemm_tc_{dtype}_c{t['cluster']}", (t["n_tiles"], 1, t["cluster"]), (160, 1, 1),
                        args[:7] + [dummy, dummy, Arena(STATUS_WORD)] + args[7:] + [U32(t["TN"]), U32(t["stages"])],
                        shared_bytes=t["shared_bytes"], op=f"gemm_{dtype}",
                        algorithm=f"tcgen05_128x{t['TN']}_s{t['stages']}_cluster{t['cluster']}")
            return
        if tactic not in ("tcgen05", "tcgen05_wide", "tcgen05_plan"):
            raise ValueError(f"unknown GEMM tactic {tactic!r}")
        if (K * elem) % 128 or ((ldx or K) * elem) % 16:
            raise ValueError("tcgen05 GEMM needs K bytes % 128 == 0 and 16-byte aligned rows")
        partial, counters = self._tc_scratch
        tc_args = args[:7] + [partial, counters, Arena(STATUS_WORD)] + args[7:]
        if tactic in ("tcgen05_wide", "tcgen05_plan"):
            if tactic == "tcgen05_plan":
                t = tc_prefill_plan(M, N, K, elem)
            else:   # explicit: 256 rows, the largest token tile, K sliced only on request
                m_tiles = ceil_div(M, 256)
                TN = ceil_div(ceil_div(M, m_tiles), 16) * 16
                k_blocks = K * elem // 128
                per = ceil_div(k_blocks, max(1, min(splits or 1, 8, k_blocks)))
                stage_bytes = 32768 + TN * 128
                stages = max(3, min(12, TC_SMEM_BUDGET // stage_bytes, max(per, 3)))
                t = {"rows": 256, "TN": TN, "m_tiles": m_tiles, "n_tiles": ceil_div(N, 256),
                     "splits": ceil_div(k_blocks, per), "stages": stages, "shared_bytes": stages * stage_bytes + 1024}
                assert t["splits"] == 1 or t["splits"] * M * t["n_tiles"] * 256 * 4 <= TC_SCRATCH_BYTES
            wide = t["rows"] == 256
            self.launch(f"agi_gemm_tc_wide_{dtype}" if wide else f"agi_gemm_tc_{dtype}",
                        (t["n_tiles"], t["m_tiles"], t["splits"]), (288 if wide else 160, 1, 1),
                        tc_args + [U32(t["TN"]), U32(t["stages"])], shared_bytes=t["shared_bytes"], op=f"gemm_{dtype}",
                        algorithm=f"tcgen05_{t['rows']}x{t['TN']}_s{t['stages']}_k{t['splits']}")
            return
        t = tc_tiling(M, N, K, elem, splits)
        while t["splits"] > 1 and t["splits"] * M * t["n_tiles"] * 128 * 4 > TC_SCRATCH_BYTES:
            t = tc_tiling(M, N, K, elem, t["splits"] // 2)
        assert t["tiles"] * 4 <= TC_COUNTER_BYTES
        self.launch(f"agi_gemm_tc_{dtype}", (t["n_tiles"], t["m_tiles"], t["splits"]), (160, 1, 1),
                    args[:7] + [partial, counters, Arena(STATUS_WORD)] + args[7:] + [U32(t["TN"]), U32(t["stages"])],
                    shared_bytes=t["shared_bytes"], op=f"gemm_{dtype}",
                    algorithm=f"tcgen05_128x{t['TN']}_s{t['stages']}_k{t['splits']}")

    def gemm_group(self, x: Pointer, parts: Sequence[tuple[Pointer, Pointer | None, Pointer | None, Pointer, int, int]],
                   M: int, K: int, *, dtype: str = "bf16", scale_a: Pointer | None = None, ldx: int | None = None,
                   act: str | None = None, packed: bool = False) -> None:
        """Up to three GEMMs over one activation matrix in one tensor-core launch (Q | K | V, gate | up).
        ``parts``: ``(weight, bias or None, weight scale or None, y, N, ldy)``; either every part has a bias
        or none has; with ``scale_a`` every part brings its weight scale."""
        assert 1 <= len(parts) <= 3
        elem = 1 if dtype == "e4m3" else 2
        if (K * elem) % 128 or ((ldx or K) * elem) % 16:
            raise ValueError("grouped tcgen05 GEMM needs K bytes % 128 == 0 and 16-byte aligned rows")
        has_bias = parts[0][1] is not None
        assert all((p[1] is not None) == has_bias for p in parts)
        assert all((p[2] is not None) == (scale_a is not None) for p in parts)
        flags = ACT[act] | (FLAG_BIAS if has_bias else 0) | (FLAG_SCALED if scale_a else 0)
        t = tc_group_tiling(M, sum(ceil_div(p[4], 128) for p in parts), K, elem)
        dummy = Arena(0)
        assert not packed or (dtype == "e4m3" and ldx is None)
        args: list[Any] = [x, scale_a or dummy, Arena(STATUS_WORD), U32(M), U32(K),
                           U32(padded_token_rows(M) if packed else (ldx or K)), U32(flags), U32(t["TN"]), U32(t["stages"])]
        for i in range(3):
            if i < len(parts):
                w, bias, sw, y, N, ldy = parts[i]
                args += [w, bias or dummy, sw or dummy, y, U32(N), U32(ldy)]
            else:
                args += [dummy, dummy, dummy, dummy, U32(0), U32(0)]
        grid_x = sum(ceil_div(p[4], 128) for p in parts)
        if dtype == "bf16" and not packed and M <= 64:
            # few tokens: too few tiles to fill the SMs, so the K slices of every tile form a cluster (as `cluster`
            # does for one matrix) and the projections that share the activations still share the launch
            c = tc_cluster_tiling(M, 128 * grid_x, K, elem, dtype, sizes=(2, 4, 8))
            if c is not None:
                args[7:9] = [U32(c["TN"]), U32(c["stages"])]
                self.launch(f"agi_gemm_tc_bf16_x3_c{c['cluster']}", (grid_x, 1, c["cluster"]), (160, 1, 1), args,
                            shared_bytes=c["shared_bytes"], op="gemm_bf16_group",
                            algorithm=f"tcgen05_128x{c['TN']}_s{c['stages']}_cluster{c['cluster']}_x{len(parts)}")
                return
        self.launch(f"agi_gemm_tcp_{dtype}_x3" if packed else f"agi_gemm_tc_{dtype}_x3", (grid_x, t["m_tiles"], 1),
                    (160, 1, 1), args, shared_bytes=t["shared_bytes"], op=f"gemm_{dtype}_group" + ("_packed" if packed else ""),
                    algorithm=f"tcgen05_{'bulk_' if packed else ''}128x{t['TN']}_s{t['stages']}_x{len(parts)}")

    def gemm_batch(self, x: Pointer, parts: Sequence[tuple[Pointer, Pointer]], y: Pointer, M: int, N: int, K: int,
                   seg_stride: int, ldx: int | None = None) -> None:
        """Up to 16 bf16 GEMMs ``y[s] = x . W_s^T + b_s`` over the same ``x`` in one tensor-core launch;
        ``y[s]`` starts ``seg_stride`` elements after ``y[s - 1]``."""
        assert 1 <= len(parts) <= 16 and (K * 2) % 128 == 0
        t = tc_tiling(M, N, K, 2, 1)
        dummy = Arena(0)
        ws = [p[0] for p in parts] + [dummy] * (16 - len(parts))
        bs = [p[1] for p in parts] + [dummy] * (16 - len(parts))
        self.launch("agi_gemm_tc_bf16_x16", (len(parts) * t["n_tiles"], t["m_tiles"], 1), (160, 1, 1),
                    [x, y, Arena(STATUS_WORD), U32(M), U32(N), U32(K), U32(ldx or K), U32(N), U32(FLAG_BIAS), U32(t["TN"]),
                     U32(t["stages"]), U32(seg_stride), *ws, *bs], shared_bytes=t["shared_bytes"], op="gemm_bf16_batch",
                    algorithm=f"tcgen05_128x{t['TN']}_s{t['stages']}_x{len(parts)}")

    def is_packed(self, w: Pointer) -> bool:
        """True for a checkpoint matrix stored in the packed layout of ``recipes/layout.py`` ([K blocks, rows, 64])."""
        return isinstance(w, Weight) and len(self.weights.get(w.name, ("", ()))[1]) == 3

    def gemm_tcs(self, x: Pointer, parts: Sequence[tuple[Pointer, Pointer | None, int]], y: Pointer, M: int, K: int, *,
                 residual: Pointer | None = None, act: str | None = None, ldx: int | None = None,
                 ldy: int | None = None, cluster: int | None = None, groups: int | None = None,
                 kb: int | None = None) -> None:
        """``y[:, blocks] = epilogue(x . [W0 | W1 | W2]^T)`` with packed bf16 weights and M <= 32: the
        weight-streaming tensor-core kernel (every CTA requests its whole weight slab before the grid-dependency
        wait).  ``parts``: up to three ``(packed weight, bias or None, N_i)``, N_i multiples of 128."""
        assert 1 <= len(parts) <= 3 and all(n % 128 == 0 for _, _, n in parts)
        assert len({b is None for _, b, _ in parts}) == 1 and ((ldx or K) * 2) % 16 == 0
        total = sum(n for _, _, n in parts)
        t = tcs_tiling(M, total // 128, K, cluster, groups, kb)
        if t is None:
            raise ValueError("the weight-streaming tensor-core GEMM needs M <= 32 and K in whole 64-element blocks")
        partial, counters = self._tc_scratch
        assert t["slices"] * M * total * 4 <= TC_SCRATCH_BYTES and total // 128 * 8 * 4 <= TC_COUNTER_BYTES
        flags = ACT[act] | (FLAG_BIAS if parts[0][1] is not None else 0) | (FLAG_RESIDUAL if residual else 0)
        dummy = Arena(0)
        ws = [p[0] for p in parts] + [dummy] * (3 - len(parts))
        bs = [(p[1] or dummy) for p in parts] + [dummy] * (3 - len(parts))
        ns = [p[2] for p in parts] + [0] * (3 - len(parts))
        C, G = t["cluster"], t["groups"]
        kernel = "agi_gemm_tcs_bf16" if C == 1 else f"agi_gemm_tcs_bf16_c{C}"
        grid = (total // 128, 1, t["slices"]) if C == 1 else (total // 128, G, C)
        self.launch(kernel, grid, (160, 1, 1),
                    [x, *ws, y, *bs, residual or dummy, partial, counters, Arena(STATUS_WORD), U32(M), *map(U32, ns),
                     U32(K), U32(ldx or K), U32(ldy or total), U32(flags), U32(t["kb"])],
                    shared_bytes=t["shared_bytes"], op="gemm_bf16_packed",
                    algorithm=f"tcgen05_stream_kb{t['kb']}_c{C}_g{G}_x{len(parts)}")

    def fused_linear(self, x: Pointer, parts: Sequence[tuple[Pointer, Pointer | None, int]], y: Pointer, M: int, K: int,
                     *, ln: dict[str, Any] | None = None, ln_scratch: Pointer | None = None,
                     residual: Pointer | None = None, act: str | None = None, ldx: int | None = None,
                     ldy: int | None = None, fuse: bool = True, fuse_ln: bool = False) -> None:
        """``y[:, blocks] = epilogue(LN?(x) . [W0 | W1 | W2]^T)`` for bf16 and M <= 64.

        ``parts``: up to three ``(weight, bias or None, N_i)``; outputs land in consecutive column blocks of
        ``y``.  ``ln``: ``{"eps": e}`` for LayerNorm without affine, plus ``"scale"``/``"shift"`` pointers for
        AdaLN modulation.  The weight matrices share one launch of the fused bulk-stream kernel.  The LayerNorm
        is a launch of its own (into ``ln_scratch``) unless ``fuse_ln`` is set and the whole K range of a CTA
        fits one ring slot: measured inside the action-head recipe, the in-kernel prologue (every CTA
        normalising all rows again) costs more than the 2.8 us of the separate kernel.  ``fuse=False`` gives
        one launch per weight matrix."""
        total = sum(n for _, _, n in parts)
        ldy = ldy or total
        if all(self.is_packed(w) for w, _, _ in parts):
            src = x
            if ln is not None:
                assert ln_scratch is not None, "a separate LayerNorm needs a buffer for the normalised activations"
                self.layernorm(x, ln_scratch, M, K, ln["eps"], scale=ln.get("scale"), shift=ln.get("shift"), x_stride=ldx)
                src, ldx = ln_scratch, None
            self.gemm_tcs(src, parts, y, M, K, residual=residual, act=act, ldx=ldx, ldy=ldy)
            return
        t = stream_tiling(M, total, K, 2, contiguous=(ldx or K) == K)
        rows = t["rows"]
        fits = (M <= 64 and (K * 2) % 64 == 0 and len(parts) <= 3 and all(n % rows == 0 for _, _, n in parts)
                and (ln is None or (t["slots"] == 1 and K <= 1536))
                and len({b is None for _, b, _ in parts}) == 1)
        if fuse and fits and ln is not None and not fuse_ln:
            assert ln_scratch is not None, "a separate LayerNorm needs a buffer for the normalised activations"
            self.layernorm(x, ln_scratch, M, K, ln["eps"], scale=ln.get("scale"), shift=ln.get("shift"), x_stride=ldx)
            x, ldx, ln = ln_scratch, None, None
        if not (fuse and fits):
            src = x
            if ln is not None:
                assert ln_scratch is not None, "fallback needs a buffer for the normalised activations"
                self.layernorm(x, ln_scratch, M, K, ln["eps"], scale=ln.get("scale"), shift=ln.get("shift"),
                               x_stride=ldx)
                src, ldx = ln_scratch, None
            col = 0
            for w, b, n in parts:
                self.gemm(src, w, y + col * 2 if col else y, M, n, K, bias=b, residual=(residual + col * 2 if col else
                          residual) if residual is not None else None, act=act, ldx=ldx, ldy=ldy)
                col += n
            return
        flags = ACT[act] | (FLAG_BIAS if parts[0][1] is not None else 0) | (FLAG_RESIDUAL if residual else 0)
        if ln is not None:
            flags |= FLAG_LAYERNORM | (FLAG_LN_MODULATE if "scale" in ln else 0)
        if t["slab"]:
            flags |= FLAG_SLAB
        dummy = Arena(0)
        ws = [p[0] for p in parts] + [dummy] * (3 - len(parts))
        bs = [(p[1] or dummy) for p in parts] + [dummy] * (3 - len(parts))
        ns = [p[2] for p in parts] + [0] * (3 - len(parts))
        tiles = t["tiles"]
        family = "lnfused" if ln is not None else "fused"
        self.launch(f"agi_gemm_stream_{family}_bf16_t{tiles}", (t["grid"], 1, 1), (t["threads"], 1, 1),
                    [x, *ws, y, *bs, residual or dummy, (ln or {}).get("scale", dummy), (ln or {}).get("shift", dummy),
                     Arena(STATUS_WORD), U32(M), *map(U32, ns), U32(K), U32(ldx or K), U32(ldy), U32(flags), U32(rows),
                     U32(t["chunk_windows"]), F32((ln or {}).get("eps", 0.0))],
                    shared_bytes=t["shared_bytes"], op="fused_linear_bf16",
                    algorithm=f"bulk_stream_r{rows}_t{tiles}_x{len(parts)}" + ("_ln" if ln else ""))

    # ---- persistent block kernel ----------------------------------------------------------
    def store_pointers(self, table: Arena, first: int, pointers: Sequence[Pointer]) -> None:
        """Write device addresses into consecutive 8-byte slots of an arena table, 16 per launch: how a
        persistent kernel receives more pointers than a parameter list should carry."""
        dummy = Arena(0)
        for i in range(0, len(pointers), 16):
            batch = list(pointers[i:i + 16])
            self.launch("agi_store_pointers16", (1, 1, 1), (32, 1, 1),
                        [table, U32(first + i), U32(len(batch)), *batch, *([dummy] * (16 - len(batch)))],
                        op="pointer_table", algorithm="store16")

    def dit_scratch(self, T: int, D: int, mlp: int) -> tuple[Arena, Arena]:
        """Scratch of the persistent block kernel: K-span partial sums of the MLP down projection and the arrival
        counters of its feature groups (zero between launches for the life of the session, like the split-K
        counters).  Outside the stack discipline of alloc/release: call it before the first ``mark`` of a recipe
        that releases arena space between profiles."""
        scratch = self._dit_scratch.get((T, D, mlp))
        if scratch is None:
            span = dit_block_span(mlp)
            scratch = (self.alloc((mlp // span) * T * D * 4), self.alloc(D // 16 * 4))
            self._dit_scratch[(T, D, mlp)] = scratch
        return scratch

    def dit_blocks(self, table: Arena, seq: Pointer, qkv: Pointer, attn: Pointer, ff: Pointer, *, layers: int, T: int,
                   D: int, heads: int, head_dim: int, mlp: int, ctx: int, cross_mask: int, mod_offset: int,
                   eps: float, scale: float | None = None) -> None:
        """A stack of DiT blocks as ONE launch of the persistent block kernel (``agi_coop_dit_blocks_bf16_t*``):
        one CTA per SM walks every block; the weight stream runs ahead of the compute through a shared-memory
        ring and never stops at a phase boundary.  ``table``: 16 pointers per block (``DIT_TABLE_ORDER``),
        written earlier in the profile with ``store_pointers``.  ``mod_offset``: elements from a block's AdaLN
        pointer to this step's (scale | shift) row.  ``seq`` [T, D] is updated in place."""
        span = dit_block_span(mlp)
        geometry = dit_block_geometry(T, D, heads, head_dim, mlp, ctx, layers)
        if geometry is None or span is None:
            raise ValueError("shape is outside what the persistent block kernel covers")
        partial, group_counters = self.dit_scratch(T, D, mlp)
        tiles = 2 if T <= 16 else 3
        self.launch(f"agi_coop_dit_blocks_bf16_t{tiles}", (SM_COUNT, 1, 1), (384, 1, 1),
                    [table, seq, qkv, attn, ff, partial, group_counters, self.counter(), Arena(STATUS_WORD), U32(layers),
                     U32(T), U32(D), U32(heads), U32(head_dim), U32(mlp), U32(span), U32(ctx), U32(cross_mask),
                     U32(mod_offset), U32(geometry["slots"]), F32(eps), F32(scale if scale is not None else head_dim ** -0.5)],
                    shared_bytes=geometry["shared_bytes"], op="dit_blocks",
                    algorithm=f"persistent_ring{geometry['slots']}_span{span}_x{layers}")

    # ---- outputs --------------------------------------------------------------------------
    def plan(self) -> dict[str, Any]:
        return {
            "cuda_arch": self.arch,
            "arena_bytes": self.arena_bytes,
            "workspace_bytes": 0,
            "shape_dispatch": [{"profile": p.name, "inputs": p.inputs, "outputs": p.outputs, "launches": p.launches}
                               for p in self.profiles],
            "cuda_graph_templates": [{"profile": p.name} for p in self.profiles if p.graph_safe],
        }

    def tactic_database(self) -> dict[str, Any]:
        return {"cuda_arch": self.arch, "tactics": sorted(self.tactics.values(), key=lambda t: (t["op"], t["algorithm"]))}


def io(name: str, dtype: str, shape: Sequence[int]) -> dict[str, Any]:
    return {"name": name, "dtype": dtype, "shape": list(shape)}

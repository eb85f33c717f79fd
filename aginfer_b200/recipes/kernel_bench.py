"""Time one kernel family in isolation through the packaged path (AIM -> loader -> CUDA graph).

    python -m aginfer_b200.recipes.kernel_bench --case gemm_fc1 --tactic stream [--pdl] [--reps 64] [--iters 20]

Each profile is ``reps`` launches of one kernel back to back; GEMM cases rotate over 16 distinct weight
matrices of the DiT action head's shapes (17 tokens, hidden 1536, MLP 6144) so that consecutive launches
do not find their weights in L2 by accident (16 x 18.9 MB for the MLP shapes; the 4.7 MB projection
rotates inside L2, which is noted in the output).  Prints microseconds per launch and, for GEMMs, the
weight-streaming rate.  Used for the per-kernel numbers under ``profiles/`` and as the small, bounded
workload for ``ncu`` captures.
"""
from __future__ import annotations

import argparse
import tempfile
from pathlib import Path

D, T, MLP, LAYERS = 1536, 17, 6144, 16
GEMM_SHAPES = {"gemm_q": (D, D), "gemm_fc1": (MLP, D), "gemm_fc2": (D, MLP),
               # the (N, K) grid of the FP8 GEMM sweep
               "gemm_2048x2048": (2048, 2048), "gemm_11008x2048": (11008, 2048), "gemm_2048x11008": (2048, 11008),
               "gemm_2560x2048": (2560, 2048), "gemm_1536x1536": (1536, 1536), "gemm_6144x1536": (6144, 1536),
               # vision tower and 7B-shaped backbone
               "gemm_3840x1280": (3840, 1280), "gemm_3456x1280": (3456, 1280), "gemm_1280x3456": (1280, 3456),
               "gemm_1024x1024": (1024, 1024), "gemm_512x1024": (512, 1024), "gemm_4096x1024": (4096, 1024),
               "gemm_1024x4096": (1024, 4096),     # action expert
               "gemm_3584x3584": (3584, 3584), "gemm_18944x3584": (18944, 3584), "gemm_3584x18944": (3584, 18944)}
CASES = ("empty", "layernorm", "attn_self", "attn_cross", "attn_prefill", "attn_vision", "attn_expert", "group_qkv",
         "group_expert_qkv", "batch_kv",
         "quantize_packed", "rmsnorm_amax", "mrope", "swiglu_amax", "dit_blocks", *GEMM_SHAPES)


def build(case: str, tactic: str, reps: int, tokens: int, stages: int = 4, dtype: str = "bf16", packed: bool = False,
          tcs: tuple[int, int, int] | None = None):
    import torch

    from . import Arena, RecipeBuilder, Tensor, U32, Weight, io
    from .package import describe

    weights = {"bias": torch.zeros(MLP, dtype=torch.bfloat16)}
    if case in GEMM_SHAPES:
        n, k = GEMM_SHAPES[case]
        g = torch.Generator().manual_seed(0)
        for l in range(LAYERS):
            w = torch.randn(n, k, generator=g) * 0.02
            weights[f"l{l}.w"] = w.to(torch.bfloat16) if dtype == "bf16" else w.clamp(-0.08, 0.08).mul(448 / 0.08).to(
                torch.float8_e4m3fn)
            if packed:
                from .layout import pack_kblock_swizzled
                weights[f"l{l}.w"] = pack_kblock_swizzled(weights[f"l{l}.w"])
        weights["w_scale"] = torch.tensor(0.08 / 448, dtype=torch.float32)
    if case == "group_qkv":       # decoder Q | K | V (2048 | 256 | 256 rows, K = 2048) as one grouped tensor-core launch
        from .layout import pack_kblock_swizzled
        g = torch.Generator().manual_seed(0)
        for l in range(LAYERS):
            for part, n in (("q", 2048), ("k", 256), ("v", 256)):
                w = (torch.randn(n, 2048, generator=g) * 0.02).clamp(-0.08, 0.08).mul(448 / 0.08).to(torch.float8_e4m3fn)
                weights[f"l{l}.{part}"] = pack_kblock_swizzled(w) if packed else w
        weights["w_scale"] = torch.tensor(0.08 / 448, dtype=torch.float32)
    if case == "group_expert_qkv":
        g = torch.Generator().manual_seed(0)
        for l in range(LAYERS):
            for part, n in (("q", 1024), ("k", 512), ("v", 512)):
                weights[f"l{l}.{part}"] = (torch.randn(n, 1024, generator=g) * 0.02).to(torch.bfloat16)
    if case == "batch_kv":        # the action head's cross-attention K / V projections: 16 x (1536 x 2048) bf16, one launch
        g = torch.Generator().manual_seed(0)
        for l in range(LAYERS):
            weights[f"l{l}.w"] = (torch.randn(D, 2048, generator=g) * 0.02).to(torch.bfloat16)
    if case in ("rmsnorm_amax",):
        weights["gain"] = torch.ones(2048, dtype=torch.bfloat16)
    r = RecipeBuilder(describe(weights))
    r.begin_profile("default", [io("token", "I32", [1])], [io("status", "I32", [1])])
    big = (max(tokens, 64) + 512) * 18944 * 2     # room for the padded rows of packed activations
    x, y, scale_a = r.alloc(big), r.alloc(big), r.alloc(4)
    attn_bytes = max(tokens, 300) * 2048 * 2       # the widest attention operand of any case
    kbuf, vbuf, q = r.alloc(attn_bytes), r.alloc(attn_bytes), r.alloc(attn_bytes)
    for i in range(reps):
        if case == "empty":
            r.launch("agi_fill_u32", (1, 1, 1), (256, 1, 1), [Arena(64), U32(0), U32(16)])
        elif case == "layernorm":
            r.layernorm(x, y, tokens, D, 1e-5)
        elif case in ("attn_self", "attn_cross"):
            kv_rows = tokens if case == "attn_self" else 300
            r.attention(q, kbuf, vbuf, y, q_rows=tokens, kv_rows=kv_rows, q_heads=32, kv_heads=32, head_dim=48,
                        q_stride=D, k_stride=D, v_stride=D, o_stride=D,
                        algorithm=tactic if tactic in ("warp_per_row", "keys_in_smem", "mma") else "auto")
        elif case == "attn_expert":       # action expert: `tokens` queries over a 256-row prefix + themselves, 8 / 4 heads of 128
            r.attention(q, kbuf, vbuf, y, q_rows=tokens, kv_rows=256 + tokens, q_heads=8, kv_heads=4, head_dim=128,
                        q_stride=1024, k_stride=512, v_stride=512, o_stride=1024,
                        algorithm=tactic if tactic in ("warp_per_row", "keys_in_smem", "mma") else "auto")
        elif case == "group_expert_qkv":  # action expert Q | K | V (1024 | 512 | 512 rows, K = 1024, bf16) as one launch
            r.gemm_group(x, [(Weight(f"l{i % LAYERS}.q"), None, None, y, 1024, 2048),
                             (Weight(f"l{i % LAYERS}.k"), None, None, y + 1024 * 2, 512, 2048),
                             (Weight(f"l{i % LAYERS}.v"), None, None, y + 1536 * 2, 512, 2048)], tokens, 1024)
        elif case == "attn_prefill":      # decoder prefill: `tokens` causal rows, 16 query / 2 KV heads of 128
            r.attention(q, kbuf, vbuf, y, q_rows=tokens, kv_rows=tokens, q_heads=16, kv_heads=2, head_dim=128,
                        q_stride=2048, k_stride=256, v_stride=256, o_stride=2048, mask="causal")
        elif case == "group_qkv":
            dummy_bias = None
            r.gemm_group(x, [(Weight(f"l{i % LAYERS}.q"), dummy_bias, Weight("w_scale"), y, 2048, 2560),
                             (Weight(f"l{i % LAYERS}.k"), dummy_bias, Weight("w_scale"), y + 2048 * 2, 256, 2560),
                             (Weight(f"l{i % LAYERS}.v"), dummy_bias, Weight("w_scale"), y + 2304 * 2, 256, 2560)],
                         tokens, 2048, dtype="e4m3", scale_a=scale_a, packed=packed)
        elif case == "batch_kv":
            r.gemm_batch(x, [(Weight(f"l{j}.w"), Weight("bias")) for j in range(LAYERS)], y, tokens, D, 2048,
                         seg_stride=tokens * D)
        elif case == "quantize_packed":   # amax is taken as already folded by the producer (one launch)
            r.quantize_e4m3(x, y, scale_a, tokens * 2048, amax=r.counter() if i == 0 else Arena(64), packed=(tokens, 2048))
        elif case == "rmsnorm_amax":
            r.rmsnorm(x, Weight("gain"), y, tokens, 2048, 1e-6, amax=Arena(64))
        elif case == "mrope":
            r.mrope(x, kbuf, tokens, 16, 128, 2048, 1e6, (16, 24, 24))
        elif case == "swiglu_amax":
            r.swiglu(x, x + 11008 * 2, y, tokens, 11008, 2 * 11008, amax=Arena(64))
        elif case == "attn_vision":       # vision tower: `tokens` patch rows, 16 heads of 80, 64-token windows
            r.attention(q, kbuf, vbuf, y, q_rows=tokens, kv_rows=tokens, q_heads=16, kv_heads=16, head_dim=80,
                        q_stride=1280, k_stride=1280, v_stride=1280, o_stride=1280, mask="block", mask_arg=64)
        else:
            n, k = GEMM_SHAPES[case]
            if dtype == "bf16" and packed:    # weight-streaming tensor-core kernel; geometry from --tcs or the builder
                c, g, kb = tcs or (None, None, None)
                r.gemm_tcs(x, [(Weight(f"l{i % LAYERS}.w"), None, n)], y, tokens, k, cluster=c, groups=g, kb=kb)
            elif dtype == "bf16":
                r.gemm(x, Weight(f"l{i % LAYERS}.w"), y, tokens, n, k, tactic=tactic)
            else:   # activations taken as already quantised bytes; scales are whatever the arena holds
                r.gemm(x, Weight(f"l{i % LAYERS}.w"), y, tokens, n, k, dtype="e4m3", scale_a=scale_a,
                       scale_w=Weight("w_scale"), tactic=tactic, packed=packed)
    r.export_status(Tensor("status"))
    return weights, r


def main() -> None:
    import torch

    from .. import runtime as rt
    from ..runner import Runner
    from .package import build_aim

    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="gemm_fc1", choices=CASES)
    ap.add_argument("--tactic", default="auto")
    ap.add_argument("--reps", type=int, default=64)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=T)
    ap.add_argument("--pdl", action="store_true")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "e4m3"])
    ap.add_argument("--packed", action="store_true", help="packed weights (and, for e4m3, activations), bulk-copy producers")
    ap.add_argument("--tcs", default=None, help="packed bf16 only: cluster,groups,blocks-per-slice of the weight-streaming "
                                                "tensor-core kernel (default: the builder's choice)")
    ap.add_argument("--stages", type=int, default=4, help="K partitions of the bulk-stream GEMM (1-4)")
    ap.add_argument("--layers", type=int, default=2, help="blocks in the stack of the dit_blocks case")
    args = ap.parse_args()

    profile = ""
    if args.case == "dit_blocks":
        # the persistent block kernel over `--layers` blocks of the action head's shape: the recipe's own
        # measurement profile (pointer table + one launch); --reps does not apply
        from . import dit
        cfg = dit.DitConfig(layers=args.layers)
        weights = dit.synthetic_weights(cfg, seed=2)
        recipe = dit.build_recipe(cfg, stream_profile=True, block_kernel=True)
        profile, args.reps = "blocks_1", 1
    else:
        weights, recipe = build(args.case, args.tactic, args.reps, args.tokens, args.stages, args.dtype, args.packed,
                                tuple(map(int, args.tcs.split(","))) if args.tcs else None)
    with tempfile.TemporaryDirectory() as tmp:
        aim = build_aim(Path(tmp), weights, recipe)
        runner = Runner(aim, profile=profile, flags=rt.PROGRAMMATIC_LAUNCH if args.pdl else 0)
        token = torch.zeros(1, dtype=torch.int32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            for _ in range(3):
                runner.run({"token": token}, {"status": status}, stream=stream)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record(stream)
            for _ in range(args.iters):
                runner.run({"token": token}, {"status": status}, stream=stream)
            end.record(stream)
            torch.cuda.synchronize()
        if args.case == "dit_blocks":
            from . import dit
            alg, _ = dit.stream_profile_bytes(cfg)
            ms = start.elapsed_time(end) / args.iters
            print(f"dit_blocks layers={args.layers}: {ms * 1000:.1f} us per profile replay (pointer table + one launch), "
                  f"{alg / ms / 1e6:.0f} GB/s of algorithmic bytes, status={status.item()}")
            return
        us = start.elapsed_time(end) * 1000.0 / args.iters / (args.reps + 2)
        line = (f"{args.case} tactic={args.tactic} tokens={args.tokens} pdl={args.pdl} packed={args.packed}"
                + (f" tcs={args.tcs}" if args.tcs else "") + f": {us:.2f} us/launch")
        if args.case in GEMM_SHAPES:
            n, k = GEMM_SHAPES[args.case]
            elem = 2 if args.dtype == "bf16" else 1
            line += f" dtype={args.dtype}, {n * k * elem / us / 1e3:.0f} GB/s of weights"
            line += f", {2.0 * args.tokens * n * k / us / 1e6:.1f} TFLOP/s"
            line += " (L2-resident rotation)" if n * k * elem * LAYERS < 126e6 else " (rotation larger than L2)"
        print(line + f", status={status.item()}")


if __name__ == "__main__":
    main()

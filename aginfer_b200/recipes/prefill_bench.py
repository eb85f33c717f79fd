"""Time the Qwen2.5-VL-shaped FP8 prefill recipe (vision tower + merger + 36 decoder layers, 288 tokens).

    python -m aginfer_b200.recipes.prefill_bench [--iters 20] [--pdl] [--v-layers 32] [--layers 36] [--vocab 151936]
                                                 [--check-against oracle_outputs.pt]

Builds the synthetic checkpoint (seed 3), packages it, loads it through the runtime and replays the
profile.  Prints ms per prefill (CUDA events around ``iters`` replays), the fraction of the FP8 weight stream
against the HBM peak and the achieved FLOP/s.  ``--save-inputs DIR`` writes the weights and inputs so that a
CPU oracle run elsewhere can check the outputs saved with ``--save-outputs``.
"""
from __future__ import annotations

import argparse
import json
import shutil
import tempfile
import time
from pathlib import Path

import torch

from aginfer_b200 import runtime as rt
from aginfer_b200.recipes import qwen_vl
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--pdl", action="store_true")
    ap.add_argument("--v-layers", type=int, default=32)
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--tactic", default="auto")
    ap.add_argument("--packed", action="store_true", help="packed weights / activations, bulk-copy GEMM producers")
    ap.add_argument("--save-outputs", default=None, help="write hidden_out / kv_cache / status as a .pt file")
    args = ap.parse_args()
    full = tuple(i for i in (7, 15, 23, 31) if i < args.v_layers) or (args.v_layers - 1,)
    cfg = qwen_vl.VlConfig(v_layers=args.v_layers, v_full_layers=full, layers=args.layers, vocab=args.vocab)
    t0 = time.time()
    weights, inputs = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
    if args.packed:
        weights = qwen_vl.pack_checkpoint(weights)
    recipe = qwen_vl.build_recipe(cfg, describe(weights), gemm_tactic=args.tactic, packed=args.packed)
    scratch = Path("/dev/shm") if Path("/dev/shm").is_dir() else None      # 2 x 4 GB of files: prefer memory
    tmp = Path(tempfile.mkdtemp(prefix="agi_prefill_", dir=scratch))
    try:
        aim = build_aim(tmp, weights, recipe)
        t1 = time.time()
        runner = Runner(aim, flags=rt.PROGRAMMATIC_LAUNCH if args.pdl else 0)
        stream = torch.cuda.Stream()
        dev = {k: v.cuda() for k, v in inputs.items()}
        out = runner.empty_outputs()
        with torch.cuda.stream(stream):
            for _ in range(3):
                runner.run(dev, out, stream=stream)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            start.record(stream)
            for _ in range(args.iters):
                runner.run(dev, out, stream=stream)
            end.record(stream)
            torch.cuda.synchronize()
        ms = start.elapsed_time(end) / args.iters
        alg = qwen_vl.algorithmic(cfg)
        stats = runner.stats()
        print(json.dumps({
            "workload": f"qwen2.5-vl-shaped fp8 prefill, {cfg.v_layers} vision blocks + {cfg.layers} decoder layers, "
                        f"{cfg.patches} patches, {cfg.tokens} tokens",
            "ms_per_prefill": ms, "launches": int(stats["launches_per_enqueue"]), "pdl": args.pdl, "packed": args.packed,
            "fp8_weight_gb": alg["fp8_weight_bytes"] / 1e9, "weight_stream_gbs": alg["fp8_weight_bytes"] / ms / 1e6,
            "tflops": alg["flops"] / ms / 1e9, "status": int(out["status"].item()),
            "setup_s": {"weights_and_package": t1 - t0, "load_and_first_runs": time.time() - t1 - ms * args.iters / 1e3},
        }))
        if args.save_outputs:
            torch.save({k: v.cpu() for k, v in out.items()}, args.save_outputs)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()

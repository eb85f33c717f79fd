"""Time the Qwen2.5-VL-shaped FP8 prefill recipe (vision tower + merger + 36 decoder layers, 288 tokens), or
the LingBot-VLA-shaped episode (7B-shaped prefill + 18-layer action expert, 10 Euler steps) with --episode.

    python -m aginfer_b200.recipes.prefill_bench [--episode] [--packed] [--iters 20] [--pdl] [--v-layers 32]
                                                 [--layers N] [--vocab 151936] [--save-outputs out.pt]

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
from aginfer_b200.recipes import lingbot, qwen_vl
from aginfer_b200.recipes.package import build_aim, describe
from aginfer_b200.runner import Runner


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--pdl", action="store_true")
    ap.add_argument("--v-layers", type=int, default=32)
    ap.add_argument("--layers", type=int, default=None, help="decoder layers (default 36, or 28 with --episode)")
    ap.add_argument("--episode", action="store_true", help="LingBot-shaped episode: 7B-shaped prefill + action expert")
    ap.add_argument("--e-layers", type=int, default=18)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--tactic", default="auto")
    ap.add_argument("--packed", action="store_true", help="packed weights / activations, bulk-copy GEMM producers")
    ap.add_argument("--save-outputs", default=None, help="write hidden_out / kv_cache / status as a .pt file")
    ap.add_argument("--load-timing", action="store_true",
                    help="also time the package load (integrity hashing) and the weight upload, pinned double-buffered "
                         "against one blocking copy from the file mapping")
    args = ap.parse_args()
    full = tuple(i for i in (7, 15, 23, 31) if i < args.v_layers) or (args.v_layers - 1,)
    t0 = time.time()
    if args.episode:
        import dataclasses
        backbone = dataclasses.replace(lingbot.BACKBONE_7B, v_layers=args.v_layers, v_full_layers=full,
                                       layers=args.layers or 28, vocab=args.vocab)
        ecfg = lingbot.EpisodeConfig(backbone=backbone, e_layers=args.e_layers, steps=args.steps)
        cfg = backbone
        weights, inputs = lingbot.synthetic_weights(ecfg), lingbot.synthetic_inputs(ecfg)
        if args.packed:
            weights = qwen_vl.pack_checkpoint(weights)
        recipe = lingbot.build_recipe(ecfg, describe(weights), packed=args.packed)
    else:
        cfg = qwen_vl.VlConfig(v_layers=args.v_layers, v_full_layers=full, layers=args.layers or 36, vocab=args.vocab)
        weights, inputs = qwen_vl.synthetic_weights(cfg), qwen_vl.synthetic_inputs(cfg)
        if args.packed:
            weights = qwen_vl.pack_checkpoint(weights)
        recipe = qwen_vl.build_recipe(cfg, describe(weights), gemm_tactic=args.tactic, packed=args.packed)
    need = 3 * sum(v.numel() * v.element_size() for v in weights.values())     # checkpoint + package + slack
    shm = Path("/dev/shm")
    scratch = shm if shm.is_dir() and shutil.disk_usage(shm).free > need else None   # two big files: prefer memory
    tmp = Path(tempfile.mkdtemp(prefix="agi_prefill_", dir=scratch))
    try:
        aim = build_aim(tmp, weights, recipe)
        load_timing = None
        if args.load_timing:
            load_timing = {"aim_bytes": aim.stat().st_size}
            a = time.time()
            rt.Model.load(aim)                               # mmap + whole-file and per-section SHA-256
            load_timing["model_load_seconds"] = time.time() - a
            for label, flag in (("pinned_double_buffered", 0), ("blocking_from_mapping", rt.BLOCKING_UPLOAD)):
                probe = Runner(aim, flags=flag | rt.NO_GRAPH_REPLAY)
                probe.run({k: v.cuda() for k, v in inputs.items()}, probe.empty_outputs())
                torch.cuda.synchronize()
                load_timing[f"upload_seconds_{label}"] = probe.stats()["upload_seconds"]
                del probe
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
        what = f"{cfg.v_layers} vision blocks + {cfg.layers} decoder layers, {cfg.patches} patches, {cfg.tokens} tokens"
        if args.episode:
            e = lingbot.algorithmic(ecfg)
            what = (f"lingbot-shaped episode: {what}; expert {ecfg.e_layers} layers x {ecfg.steps} steps "
                    f"({e['expert_weight_bytes_per_episode'] / 1e9:.2f} GB of bf16 weights streamed)")
        else:
            what = "qwen2.5-vl-shaped fp8 prefill, " + what
        print(json.dumps({
            "workload": what,
            "ms_per_prefill": ms, "launches": int(stats["launches_per_enqueue"]), "pdl": args.pdl, "packed": args.packed,
            "fp8_weight_gb": alg["fp8_weight_bytes"] / 1e9, "weight_stream_gbs": alg["fp8_weight_bytes"] / ms / 1e6,
            "tflops": alg["flops"] / ms / 1e9, "status": int(out["status"].item()),
            "setup_s": {"weights_and_package": t1 - t0, "load_and_first_runs": time.time() - t1 - ms * args.iters / 1e3},
            **({"load_timing": load_timing} if load_timing else {}),
        }))
        if args.save_outputs:
            torch.save({k: v.cpu() for k, v in out.items()}, args.save_outputs)
    finally:
        shutil.rmtree(tmp, ignore_errors=True)


if __name__ == "__main__":
    main()

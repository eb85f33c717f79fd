"""Benchmark of the AIM launch-recipe hot path on B200: action chunks per second at batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (``config.workload``): the GR00T-N1.5-shaped flow-matching DiT action head of the
baseline's third configuration: 16 blocks x 1536, 17 tokens, cross-attention to 300 backbone
tokens, 4 Euler steps, BF16 weights ~N(0, 0.02) seed 2, synthetic N(0, 1) inputs.  A "step" of
this benchmark is one action chunk = one ``Session::Enqueue`` of the packaged recipe (505 kernel
launches replayed as one CUDA graph).  The real model's checkpoint is not available offline;
seeded synthetic tensors of its shapes stand in.

One process per GPU; replicas only (independent episodes, replicated weights, no collective):
``value`` is total chunks/s over all ranks, timed on the device with CUDA events, max over ranks.
Every chunk re-streams ~0.9 GB of weights, far more than the 126 MB L2, so no L2 flush is needed
between iterations.

``--impl reference``: the reference has no CPU (or any) implementation of the arithmetic, so the
reference arm times the CPU oracle port (PyTorch fp32, all host threads) on the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "action_chunks_per_s"
UNIT = "chunks/s"
WORKLOAD = "groot_n1_5_dit_action_head_b1 (16x1536, 17 tok, 300 ctx tok, 4 Euler steps, bf16)"


def peaks() -> tuple[float, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock / throttle samples every 100 ms while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", gpu_id, f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            import threading
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        rows = [l.split(", ") for t, l in self.lines if t0 <= t <= t1 + 0.15] or [l.split(", ") for _, l in self.lines]
        sm, reasons, top = [], set(), None
        for r in rows:
            try:
                sm.append(float(r[0]))
                top = float(r[1])
            except (ValueError, IndexError):
                continue
            for name, flag in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if flag.strip() == "Active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": top, "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_oracle_rate(cfg, weights, inputs, budget_s: float, max_chunks: int) -> tuple[float, int, float]:
    """Chunks per second of the CPU oracle (all host threads); returns (rate, chunks timed, seconds)."""
    import torch
    from oracle import dit as oracle_dit
    torch.set_num_threads(os.cpu_count() or 1)
    oracle_dit.forward(cfg, weights, inputs["backbone_features"], inputs["state"], inputs["noise"])  # warm-up
    done, t0 = 0, time.perf_counter()
    while done < max_chunks and (done == 0 or time.perf_counter() - t0 < budget_s):
        oracle_dit.forward(cfg, weights, inputs["backbone_features"], inputs["state"], inputs["noise"])
        done += 1
    seconds = time.perf_counter() - t0
    return done / seconds, done, seconds


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from aginfer_b200.recipes import dit
    cfg = dit.DitConfig()
    weights, inputs = dit.synthetic_weights(cfg, seed=2), dit.synthetic_inputs(cfg, seed=2)
    rate, chunks, seconds = cpu_oracle_rate(cfg, weights, inputs, budget_s=90.0, max_chunks=max(1, args.steps))
    cores = os.cpu_count() or 1
    sample = f"{chunks} whole action chunks of the same workload in {seconds:.1f} s (time-bounded at 90 s)"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": chunks,
        "warmup": 1, "ms_per_step": 1000.0 / rate, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "device": "host cpu"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def run_ours(args) -> None:
    import torch

    from aginfer_b200.build import build_all
    from aginfer_b200.recipes import dit
    from aginfer_b200.recipes.package import build_aim
    from aginfer_b200.runner import Runner

    from aginfer_b200.replicas import ReplicaGroup
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the recipe has no CPU execution path")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    group = ReplicaGroup.from_env("nccl")
    world, rank, local = group.world, group.rank, group.local_rank
    group.rank0_first(build_all)

    cfg = dit.DitConfig()
    weights, inputs = dit.synthetic_weights(cfg, seed=2), dit.synthetic_inputs(cfg, seed=2)
    tmp = tempfile.TemporaryDirectory(prefix=f"agi_bench_r{rank}_")
    recipe = dit.build_recipe(cfg, stream_profile=True)
    aim = build_aim(Path(tmp.name), weights, recipe, steps=cfg.steps, action_horizon=cfg.horizon,
                    state_length=cfg.state_dim)
    from aginfer_b200 import runtime as rt
    session_flags = 0 if args.no_pdl else rt.PROGRAMMATIC_LAUNCH
    runner = Runner(aim, profile="default", flags=session_flags)
    stream = torch.cuda.Stream()
    dev_in = {k: v.cuda() for k, v in inputs.items()}
    out = runner.empty_outputs()

    def barrier():
        torch.cuda.synchronize()
        group.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters: int) -> float:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        with torch.cuda.stream(stream):
            start.record(stream)
            for _ in range(iters):
                fn()
            end.record(stream)
        barrier()
        return start.elapsed_time(end)

    uuid = str(torch.cuda.get_device_properties(local).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None

    # ---- device-resident leg: inputs already in HBM --------------------------------------------------
    chunk = lambda: runner.run(dev_in, out, stream=stream)
    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            chunk()
    t0 = time.time()
    ms = timed(chunk, args.steps)
    t1 = time.time()

    if args.legs == "device":
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": group.whole_job_rate(args.steps, ms), "unit": UNIT,
                              "n_gpus": world, "steps": args.steps, "ms_per_step": ms / args.steps, "legs": "device"}))
        if sampler is not None:
            sampler.stop(t0, t1)
        group.close()
        tmp.cleanup()
        return

    # ---- end-to-end leg: pinned host inputs in, actions out, every chunk --------------------------------
    host_in = {k: v.pin_memory() for k, v in inputs.items()}
    host_out = torch.empty(out["actions"].shape, dtype=out["actions"].dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for v in host_in.values())
    d2h = host_out.numel() * host_out.element_size()

    def chunk_e2e():
        for k, v in host_in.items():
            dev_in[k].copy_(v, non_blocking=True)
        runner.run(dev_in, out, stream=stream)
        host_out.copy_(out["actions"], non_blocking=True)
        stream.synchronize()   # the caller needs the actions before it can act

    with torch.cuda.stream(stream):
        for _ in range(3):
            chunk_e2e()
    e2e_steps = args.steps
    ms_e2e = timed(chunk_e2e, e2e_steps)
    clocks = sampler.stop(t0, t1) if sampler is not None else None

    # ---- the same chunk as plain launches (no graph replay): what a loader without graph templates would do ----
    plain = Runner(aim, profile="default", flags=session_flags | rt.NO_GRAPH_REPLAY)
    plain_chunk = lambda: plain.run(dev_in, out, stream=stream)
    with torch.cuda.stream(stream):
        for _ in range(3):
            plain_chunk()
    plain_steps = max(3, min(args.steps, 50))
    ms_plain = timed(plain_chunk, plain_steps) / plain_steps
    del plain

    ms, ms_e2e, ms_plain = group.max_over_ranks([ms, ms_e2e, ms_plain])
    stats = runner.stats()

    result = None
    if rank == 0:
        peak, peak_kind = peaks()
        acc = dit.algorithmic_bytes(cfg)
        value = group.whole_job_rate(args.steps, ms)
        result = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch": 1, "replicas": world, "parallelism": f"replicas x{world}",
                       "l2": "inputs larger than L2: each chunk streams %.2f GB of weights" % (acc["per_chunk"] / 1e9),
                       "launch_mode": "one CUDA graph per chunk, built by the loader on the first Enqueue; "
                                      + ("plain edges" if args.no_pdl else "programmatic dependent launch edges")},
            "latency_ms_per_action_chunk": ms / args.steps,
            "latency_ms_per_action_chunk_plain_launches": ms_plain,
            "chunk_weight_bytes": acc["per_chunk"],
            "chunk_hbm_frac_of_%s" % peak_kind: acc["per_chunk"] / (ms / args.steps / 1000.0) / 1e9 / peak,
            "e2e": {"value": group.whole_job_rate(e2e_steps, ms_e2e), "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / e2e_steps},
            "gpu_launches": int(stats["launches_per_enqueue"]) * args.steps,
            "launches_per_chunk": int(stats["launches_per_enqueue"]),
            "clocks": clocks,
        }

    # ---- roofline of the dominant kernel family (agi_gemm_stream_bf16_t*), rank 0 only ----------------------
    if rank == 0:
        probe = Runner(aim, profile="gemm_stream", flags=session_flags)
        token = torch.zeros(1, dtype=torch.int32, device="cuda")
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        stream_chunk = lambda: probe.run({"token": token}, {"status": status}, stream=stream)
        with torch.cuda.stream(stream):
            for _ in range(5):
                stream_chunk()
        reps = 50
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        with torch.cuda.stream(stream):
            start.record(stream)
            for _ in range(reps):
                stream_chunk()
            end.record(stream)
        torch.cuda.synchronize()
        stream_ms = start.elapsed_time(end) / reps
        total_bytes, launches = dit.stream_profile_bytes(cfg)
        achieved = total_bytes / (stream_ms / 1000.0) / 1e9
        result["roofline"] = {
            "bound": "hbm", "kernel": "agi_gemm_stream_bf16_t3 / agi_gemm_stream_fused_bf16_t3", "achieved": achieved,
            "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
            "traffic": DRAM_BYTES_PER_ALGORITHMIC_BYTE * total_bytes / launches,
            "traffic_how": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the 6144x1536 and 1536x6144 launches "
                           "(profiles/gemm_stream_bf16_dit_mlp.md) over their algorithmic bytes, times this "
                           "profile's algorithmic bytes per launch",
            "launches": launches, "avg_launch_us": stream_ms * 1000.0 / launches,
            "algorithmic_bytes_per_launch": total_bytes / launches,
            "how": "the GEMM launches of one denoising step replayed back to back (profile gemm_stream), CUDA events",
            "status_word": int(status.item()),
        }
        if world == 1 and not args.no_cpu_baseline:
            rate, chunks, seconds = cpu_oracle_rate(cfg, weights, inputs, budget_s=15.0, max_chunks=1000)
            result["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                      "sample": f"{chunks} whole action chunks of the same workload in {seconds:.1f} s"}
        print(json.dumps(result))
    group.close()
    tmp.cleanup()


# DRAM bytes per algorithmic byte of the bulk-stream GEMM, from one ncu capture per MLP shape at 17 tokens:
# 18.953 MB read / 19.148 MB (6144 x 1536) and 19.110 MB / 19.139 MB (1536 x 6144), no DRAM writes (outputs
# stay in L2 until the next kernel reads them).
DRAM_BYTES_PER_ALGORITHMIC_BYTE = 0.994


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=1000)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-pdl", action="store_true", help="launch without programmatic stream serialization")
    parser.add_argument("--legs", default="all", choices=["all", "device"],
                        help="'device' runs only the device-resident timed leg (small profiler captures)")
    args = parser.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

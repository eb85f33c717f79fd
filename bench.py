"""Benchmark of the AIM launch-recipe hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--configs all|3]

Headline workload (``config.workload``, the JSON line's ``metric`` / ``value`` / ``e2e`` / ``roofline``): the
GR00T-N1.5-shaped flow-matching DiT action head of the baseline's third configuration: 16 blocks x 1536,
17 tokens, cross-attention to 300 backbone tokens, 4 Euler steps, BF16 weights ~N(0, 0.02) seed 2, synthetic
N(0, 1) inputs.  A "step" of this benchmark is one action chunk = one ``Session::Enqueue`` of the packaged
recipe, replayed as one CUDA graph.  The real model's checkpoint is not available offline; seeded synthetic
tensors of its shapes stand in.

The same line also carries, under ``configs`` and ``kernels``, what the baseline quotes on its other
configurations, measured in this run: the LingBot-VLA-shaped episode of configuration 5 (7B-shaped FP8 prefill
+ BF16 action expert, 10 Euler steps) as episodes/s over all ranks (the baseline's scaling metric), and at one
GPU the Qwen2.5-VL-3B-shaped FP8 prefill of configuration 4, the 1024-token FP8 tensor-core GEMM and the
17-token weight-streaming GEMM in isolation.

One process per GPU; replicas only (independent episodes, replicated weights, no collective): rates are totals
over all ranks, timed on the device with CUDA events, max over ranks.  Every chunk re-streams ~0.9 GB of
weights per Euler step, far more than the 126 MB L2, so no L2 flush is needed between iterations.

``--impl reference``: the reference has no CPU (or any) implementation of the arithmetic, so the reference arm
times the CPU oracle port (PyTorch fp32, all host threads) on the headline workload.
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
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
NOMINAL_FP8_TFLOPS = 4500.0       # dense FP8, B200 data sheet
SPREAD_REPEATS = 4                # further timed repeats of the --steps loop, for min / median / max


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


def measured_traffic_ratio() -> float | None:
    """DRAM bytes per algorithmic byte of the weight-streaming GEMM, from the committed ncu figures."""
    path = ROOT / "profiles" / "gemm_stream_dram_traffic.txt"
    if not path.exists():
        return None
    rows = dict(line.split()[:2] for line in path.read_text().splitlines() if line.strip() and not line.startswith("#"))
    dram = float(rows["fc1_dram_bytes"]) + float(rows["fc2_dram_bytes"])
    return dram / (float(rows["fc1_algorithmic_bytes"]) + float(rows["fc2_algorithmic_bytes"]))


class ClockSampler:
    """nvidia-smi clock / throttle samples every 100 ms while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_id: str):
        self.proc = None
        self.lines: list[tuple[float, str]] = []
        self.windows: list[tuple[float, float]] = []
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

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        inside = [l.split(", ") for t, l in self.lines if any(a <= t <= b + 0.15 for a, b in self.windows)]
        rows = inside or [l.split(", ") for _, l in self.lines]
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
    if hasattr(os, "sched_setaffinity"):
        try:
            os.sched_setaffinity(0, range(os.cpu_count() or 1))     # undo any pinning done by a communication library
        except OSError:
            pass
    torch.set_num_threads(os.cpu_count() or 1)
    oracle_dit.forward(cfg, weights, inputs["backbone_features"], inputs["state"], inputs["noise"])  # warm-up
    done, t0 = 0, time.perf_counter()
    while done < max_chunks and (done == 0 or time.perf_counter() - t0 < budget_s):
        oracle_dit.forward(cfg, weights, inputs["backbone_features"], inputs["state"], inputs["noise"])
        done += 1
    seconds = time.perf_counter() - t0
    return done / seconds, done, seconds


def cpu_baseline_in_a_fresh_process(budget_s: float) -> dict:
    """The CPU oracle timed by a child process with a clean environment: this process has by now initialised CUDA
    and, under torch.distributed.run, a communication library and a one-thread OpenMP default, all of which were
    seen to slow the host leg down by more than an order of magnitude when it ran in-process at N > 1."""
    drop = ("OMP_NUM_THREADS", "MKL_NUM_THREADS", "RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK",
            "ROLE_RANK", "MASTER_ADDR", "MASTER_PORT", "TORCHELASTIC_RUN_ID", "CUDA_VISIBLE_DEVICES")
    env = {k: v for k, v in os.environ.items() if k not in drop}
    env["CUDA_VISIBLE_DEVICES"] = ""
    done = subprocess.run([sys.executable, str(Path(__file__).resolve()), "--impl", "reference", "--steps", "1000",
                           "--reference-budget", str(budget_s)], env=env, capture_output=True, text=True, timeout=600)
    if done.returncode != 0:
        raise RuntimeError("the CPU baseline leg failed: " + done.stderr[-400:])
    return json.loads(done.stdout.strip().splitlines()[-1])["cpu_baseline"]


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from aginfer_b200.recipes import dit
    cfg = dit.DitConfig()
    weights, inputs = dit.synthetic_weights(cfg, seed=2), dit.synthetic_inputs(cfg, seed=2)
    rate, chunks, seconds = cpu_oracle_rate(cfg, weights, inputs, budget_s=args.reference_budget, max_chunks=max(1, args.steps))
    cores = os.cpu_count() or 1
    sample = (f"{chunks} whole action chunks of the same workload in {seconds:.1f} s "
              f"(time-bounded at {args.reference_budget:.0f} s)")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": chunks,
        "warmup": 1, "ms_per_step": 1000.0 / rate, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD, "device": "host cpu"},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


class Harness:
    """Timing helpers shared by the legs: CUDA events on the launching stream, barriers on both sides."""

    def __init__(self, group, stream, sampler):
        self.group, self.stream, self.sampler = group, stream, sampler

    def barrier(self):
        import torch
        torch.cuda.synchronize()
        self.group.barrier()
        torch.cuda.synchronize()

    def timed(self, fn, iters: int) -> float:
        """Milliseconds for ``iters`` calls of ``fn`` on this rank."""
        import torch
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        t0 = time.time()
        with torch.cuda.stream(self.stream):
            start.record(self.stream)
            for _ in range(iters):
                fn()
            end.record(self.stream)
        self.barrier()
        if self.sampler is not None:
            self.sampler.windows.append((t0, time.time()))
        return start.elapsed_time(end)

    def warm(self, fn, iters: int) -> None:
        import torch
        with torch.cuda.stream(self.stream):
            for _ in range(iters):
                fn()
        torch.cuda.synchronize()


def shared_scratch(tag: str) -> Path:
    """A directory every rank of this job derives the same way (memory-backed when there is room)."""
    base = Path("/dev/shm") if Path("/dev/shm").is_dir() else Path(tempfile.gettempdir())
    return base / f"agi_bench_{os.environ.get('MASTER_PORT', 'single')}_{os.getppid() if 'RANK' in os.environ else os.getpid()}_{tag}"


def bench_action_head(args, group, harness, session_flags) -> tuple[dict, dict]:
    """Configuration 3: the headline.  Returns (fields of the JSON line, context for the roofline leg)."""
    import torch

    from aginfer_b200 import runtime as rt
    from aginfer_b200.recipes import dit
    from aginfer_b200.recipes.package import build_aim
    from aginfer_b200.runner import Runner
    from oracle import dit as oracle_dit
    from oracle import ops

    cfg = dit.DitConfig()
    weights, inputs = dit.synthetic_weights(cfg, seed=2), dit.synthetic_inputs(cfg, seed=2)
    tmp = tempfile.TemporaryDirectory(prefix=f"agi_bench_r{group.rank}_")
    recipe = dit.build_recipe(cfg, stream_profile=True)
    aim = build_aim(Path(tmp.name), weights, recipe, steps=cfg.steps, action_horizon=cfg.horizon,
                    state_length=cfg.state_dim)
    runner = Runner(aim, profile="default", flags=session_flags)
    stream = harness.stream
    dev_in = {k: v.cuda() for k, v in inputs.items()}
    out = runner.empty_outputs()
    warmup = max(args.warmup, 3) if args.legs != "device" else args.warmup

    # ---- device-resident leg: inputs already in HBM; exactly --steps chunks between the barriers ----
    chunk = lambda: runner.run(dev_in, out, stream=stream)
    harness.warm(chunk, warmup)
    ms = harness.timed(chunk, args.steps)
    if args.legs == "device":      # small profiler captures: nothing but the device-resident leg
        ms, = group.max_over_ranks([ms])
        line = {"metric": METRIC, "value": group.whole_job_rate(args.steps, ms), "unit": UNIT, "n_gpus": group.world,
                "steps": args.steps, "ms_per_step": ms / args.steps}
        return line, {"tmp": tmp}
    spread = [harness.timed(chunk, args.steps) / args.steps for _ in range(SPREAD_REPEATS)]

    # ---- end-to-end leg: pinned host inputs in, actions out, every chunk ----
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

    harness.warm(chunk_e2e, 3)
    ms_e2e = harness.timed(chunk_e2e, args.steps)

    # ---- the same chunk as plain launches (no graph replay): what a loader without graph templates would do ----
    plain = Runner(aim, profile="default", flags=session_flags | rt.NO_GRAPH_REPLAY)
    plain_chunk = lambda: plain.run(dev_in, out, stream=stream)
    harness.warm(plain_chunk, 3)
    plain_steps = max(3, min(args.steps, 50))
    ms_plain = harness.timed(plain_chunk, plain_steps) / plain_steps
    del plain

    # ---- two and three independent sessions of the same package on one GPU, each on its own stream ----
    # (an extra figure, not the headline: a chunk's latency stays what it is, but a GPU that one batch-1 episode
    #  keeps at a fifth of its HBM bandwidth can serve several episodes at once)
    concurrent = {}
    for sessions in (2, 3):
        lanes = []
        for _ in range(sessions):
            lane_stream = torch.cuda.Stream()
            lane_runner = Runner(aim, profile="default", flags=session_flags)
            lane_in, lane_out = {k: v.clone() for k, v in dev_in.items()}, lane_runner.empty_outputs()
            lanes.append((lane_runner, lane_stream, lane_in, lane_out))

        def all_lanes():
            for lane_runner, lane_stream, lane_in, lane_out in lanes:
                lane_runner.run(lane_in, lane_out, stream=lane_stream)

        for _ in range(3):
            all_lanes()
        torch.cuda.synchronize()
        marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in lanes]
        harness.barrier()
        first = torch.cuda.Event(enable_timing=True)
        first.record(lanes[0][1])
        rounds = max(10, args.steps // 4)
        for _ in range(rounds):
            all_lanes()
        for (_, lane_stream, _, _), (_, done) in zip(lanes, marks):
            done.record(lane_stream)
        harness.barrier()
        lane_ms = max(first.elapsed_time(done) for _, done in marks)
        concurrent[f"{sessions}_sessions"] = {"chunks_per_s": sessions * rounds / (lane_ms / 1e3) * group.world,
                                              "ms_per_round": lane_ms / rounds}
        del lanes

    # ---- after the timed regions: the chunk that was timed is the right one ----
    chunk()
    torch.cuda.synchronize()
    status_word = int(out["status"].item())
    want = oracle_dit.forward(cfg, weights, inputs["backbone_features"], inputs["state"], inputs["noise"])
    cosine = ops.cosine(out["actions"].cpu(), want)
    if status_word != 0 or cosine < 0.999:
        raise SystemExit(f"bench: the timed recipe is wrong (status {status_word:#x}, cosine against the oracle {cosine:.6f})")

    ms, ms_e2e, ms_plain, *spread = group.max_over_ranks([ms, ms_e2e, ms_plain, *spread])
    per_chunk = [ms / args.steps, *spread]
    acc = dit.algorithmic_bytes(cfg)
    stats = runner.stats()
    line = {
        "metric": METRIC, "value": group.whole_job_rate(args.steps, ms), "unit": UNIT, "n_gpus": group.world,
        "steps": args.steps, "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch": 1, "replicas": group.world, "parallelism": f"replicas x{group.world}",
                   "l2": "inputs larger than L2: each chunk streams %.2f GB of weights" % (acc["per_chunk"] / 1e9),
                   "launch_mode": "one CUDA graph per chunk, built by the loader on the first Enqueue; "
                                  + ("plain edges" if args.no_pdl else "programmatic dependent launch edges")},
        "latency_ms_per_action_chunk": ms / args.steps,
        "latency_ms_per_action_chunk_repeats": {"each": per_chunk, "median": statistics.median(per_chunk),
                                                "min": min(per_chunk), "max": max(per_chunk),
                                                "how": f"{1 + SPREAD_REPEATS} timed regions of {args.steps} chunks each"},
        "latency_ms_per_action_chunk_plain_launches": ms_plain,
        "chunk_weight_bytes": acc["per_chunk"],
        "e2e": {"value": group.whole_job_rate(args.steps, ms_e2e), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps},
        "gpu_launches": int(stats["launches_per_enqueue"]) * args.steps,
        "launches_per_chunk": int(stats["launches_per_enqueue"]),
        "check": {"status_word": status_word, "cosine_vs_cpu_oracle": cosine},
        "concurrent_sessions_per_gpu": {**concurrent, "how": "independent sessions of the same package on separate streams "
                                        "of one GPU, device-resident inputs; this rank's figure times the number of ranks"},
    }
    context = {"aim": aim, "cfg": cfg, "weights": weights, "inputs": inputs, "tmp": tmp, "per_chunk_bytes": acc["per_chunk"]}
    return line, context


def roofline_of_stream_gemm(context, harness, session_flags, peak) -> dict:
    """The dominant kernel family of the headline: weight-streaming GEMMs of one denoising step, back to back."""
    import torch

    from aginfer_b200.recipes import dit
    from aginfer_b200.runner import Runner
    stream = harness.stream
    probe = Runner(context["aim"], profile="gemm_stream", flags=session_flags)
    token = torch.zeros(1, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    run = lambda: probe.run({"token": token}, {"status": status}, stream=stream)
    harness.warm(run, 5)
    reps = 50
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        start.record(stream)
        for _ in range(reps):
            run()
        end.record(stream)
    torch.cuda.synchronize()
    stream_ms = start.elapsed_time(end) / reps
    total_bytes, launches = dit.stream_profile_bytes(context["cfg"])
    achieved = total_bytes / (stream_ms / 1000.0) / 1e9
    ratio = measured_traffic_ratio()
    return {
        "bound": "hbm", "kernel": "agi_gemm_stream_bf16_t3 / agi_gemm_stream_bf16_t3_k4 / agi_gemm_stream_fused_bf16_t3", "achieved": achieved,
        "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": achieved / peak["hbm_gbs"], "peak_kind": f"of {peak['kind']}",
        "traffic": None if ratio is None else ratio * total_bytes / launches,
        "traffic_how": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the 6144x1536 and 1536x6144 launches "
                       "(profiles/gemm_stream_dram_traffic.txt) over their algorithmic bytes, times this profile's "
                       "algorithmic bytes per launch",
        "launches": launches, "avg_launch_us": stream_ms * 1000.0 / launches,
        "algorithmic_bytes_per_launch": total_bytes / launches,
        "how": "the weight-streaming GEMM launches of one denoising step replayed back to back, without the other "
               "kernels of the step (profile gemm_stream), CUDA events",
        "status_word": int(status.item()),
    }


def bench_episode(args, group, harness, session_flags, peak) -> dict:
    """Configuration 5 on every rank: LingBot-VLA-shaped episodes per second (the baseline's scaling metric)."""
    import torch

    from aginfer_b200.recipes import lingbot, qwen_vl
    from aginfer_b200.recipes.package import build_aim, describe
    from aginfer_b200.runner import Runner
    cfg = lingbot.EpisodeConfig()
    folder = shared_scratch("cfg5")
    t0 = time.time()
    if group.rank == 0:
        shutil.rmtree(folder, ignore_errors=True)
        folder.mkdir(parents=True)
        weights = qwen_vl.pack_checkpoint(lingbot.synthetic_weights(cfg))
        build_aim(folder, weights, lingbot.build_recipe(cfg, describe(weights), packed=True))
        shutil.rmtree(folder / "checkpoint", ignore_errors=True)
        del weights
    group.barrier()
    built_s = time.time() - t0
    try:
        runner = Runner(folder / "model.aim", flags=session_flags)
        inputs = lingbot.synthetic_inputs(cfg)
        dev = {k: v.cuda() for k, v in inputs.items()}
        out = runner.empty_outputs()
        stream = harness.stream
        episode = lambda: runner.run(dev, out, stream=stream)
        harness.warm(episode, 3)
        iters = max(5, min(args.steps, 20))
        ms = harness.timed(episode, iters)
        host_in = {k: v.pin_memory() for k, v in inputs.items()}
        host_actions = torch.empty(out["actions"].shape, dtype=out["actions"].dtype).pin_memory()

        def episode_e2e():
            for k, v in host_in.items():
                dev[k].copy_(v, non_blocking=True)
            runner.run(dev, out, stream=stream)
            host_actions.copy_(out["actions"], non_blocking=True)
            stream.synchronize()

        harness.warm(episode_e2e, 2)
        ms_e2e = harness.timed(episode_e2e, iters)
        torch.cuda.synchronize()
        status_word = int(out["status"].item())
        finite = bool(torch.isfinite(out["actions"]).all())
        stats = runner.stats()
        del runner
    finally:
        group.barrier()
        if group.rank == 0:
            shutil.rmtree(folder, ignore_errors=True)
    ms, ms_e2e = group.max_over_ranks([ms, ms_e2e])
    alg = lingbot.algorithmic(cfg)
    per = ms / iters
    weight_bytes = alg["backbone_fp8_weight_bytes"] + alg["expert_weight_bytes_per_episode"]
    flops = alg["backbone_flops"] + alg["expert_flops"]
    return {
        "workload": "lingbot_vla_episode_b1 (7B-shaped fp8 prefill: 32 vision blocks + 28 layers x 3584, 256 tokens; "
                    "bf16 action expert 18 x 1024, 50 x 14 actions, 10 Euler steps; full depth, packed fp8 operands)",
        "episodes_per_s": group.whole_job_rate(iters, ms), "episode_ms": per, "episodes_timed_per_rank": iters,
        "e2e_episodes_per_s": group.whole_job_rate(iters, ms_e2e), "e2e_episode_ms": ms_e2e / iters,
        "h2d_bytes_per_episode": sum(v.numel() * v.element_size() for v in host_in.values()),
        "d2h_bytes_per_episode": host_actions.numel() * host_actions.element_size(),
        "launches_per_episode": int(stats["launches_per_enqueue"]), "status_word": status_word, "actions_finite": finite,
        "roofline": {"weight_bytes_per_episode": weight_bytes, "flops_per_episode": flops,
                     "hbm_floor_ms": weight_bytes / peak["hbm_gbs"] / 1e6, "hbm_frac": weight_bytes / per / 1e6 / peak["hbm_gbs"],
                     "peak_kind": f"of {peak['kind']}", "achieved_tflops": flops / per / 1e9},
        "setup_seconds": built_s,
    }


def bench_prefill(harness, session_flags, peak) -> dict:
    """Configuration 4 on one GPU: the Qwen2.5-VL-3B-shaped FP8 prefill, full depth."""
    import torch

    from aginfer_b200.recipes import qwen_vl
    from aginfer_b200.recipes.package import build_aim, describe
    from aginfer_b200.runner import Runner
    cfg = qwen_vl.VlConfig()
    folder = shared_scratch("cfg4")
    shutil.rmtree(folder, ignore_errors=True)
    folder.mkdir(parents=True)
    out_line = {}
    try:
        weights = qwen_vl.synthetic_weights(cfg)
        inputs = qwen_vl.synthetic_inputs(cfg)
        dev = {k: v.cuda() for k, v in inputs.items()}
        alg = qwen_vl.algorithmic(cfg)
        for label, packed in (("packed", True), ("row_major", False)):
            w = qwen_vl.pack_checkpoint(weights) if packed else weights
            sub = folder / label
            aim = build_aim(sub, w, qwen_vl.build_recipe(cfg, describe(w), packed=packed))
            shutil.rmtree(sub / "checkpoint", ignore_errors=True)
            runner = Runner(aim, flags=session_flags)
            out = runner.empty_outputs()
            prefill = lambda: runner.run(dev, out, stream=harness.stream)
            harness.warm(prefill, 3)
            ms = harness.timed(prefill, 20) / 20
            torch.cuda.synchronize()
            out_line[label] = {"prefill_ms": ms, "launches": int(runner.stats()["launches_per_enqueue"]),
                               "status_word": int(out["status"].item()),
                               "hbm_frac": alg["fp8_weight_bytes"] / ms / 1e6 / peak["hbm_gbs"],
                               "achieved_tflops": alg["flops"] / ms / 1e9}
            del runner, out
            shutil.rmtree(sub, ignore_errors=True)
        out_line["workload"] = ("qwen2_5_vl_3b_prefill_b1 (32 vision blocks + 36 layers x 2048, 2 images, 288 tokens, "
                                "fp8 e4m3 linears with per-tensor scales; full depth)")
        out_line["fp8_weight_bytes"] = alg["fp8_weight_bytes"]
        out_line["flops"] = alg["flops"]
        out_line["hbm_floor_ms"] = alg["fp8_weight_bytes"] / peak["hbm_gbs"] / 1e6
        out_line["fp8_floor_ms_nominal"] = alg["flops"] / NOMINAL_FP8_TFLOPS / 1e9
        out_line["peak_kind"] = f"of {peak['kind']}"
    finally:
        shutil.rmtree(folder, ignore_errors=True)
    return out_line


def bench_kernels(harness, session_flags, peak) -> dict:
    """Two kernels in isolation, through the packaged path, weights rotating through more than L2."""
    import torch

    from aginfer_b200.recipes import kernel_bench
    from aginfer_b200.recipes.package import build_aim
    from aginfer_b200.runner import Runner
    found = {}
    cases = (("fp8_gemm_1024x11008x2048", "gemm_11008x2048", 1024, "e4m3", True),
             ("stream_gemm_17x6144x1536_bf16", "gemm_fc1", 17, "bf16", False))
    for label, case, tokens, dtype, packed in cases:
        reps = 32
        weights, recipe = kernel_bench.build(case, "auto", reps, tokens, dtype=dtype, packed=packed)
        with tempfile.TemporaryDirectory(prefix="agi_kernel_") as tmp:
            runner = Runner(build_aim(Path(tmp), weights, recipe), flags=session_flags)
            token = torch.zeros(1, dtype=torch.int32, device="cuda")
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            run = lambda: runner.run({"token": token}, {"status": status}, stream=harness.stream)
            harness.warm(run, 3)
            iters = 20
            us = harness.timed(run, iters) * 1000.0 / iters / (reps + 2)
            n, k = kernel_bench.GEMM_SHAPES[case]
            elem = 1 if dtype == "e4m3" else 2
            entry = {"us_per_launch": us, "status_word": int(status.item()), "tokens": tokens, "N": n, "K": k,
                     "kernel": sorted({l["kernel"] for l in recipe.plan()["shape_dispatch"][0]["launches"]
                                       if l["kernel"].startswith("agi_gemm")})}
            if dtype == "e4m3":
                tflops = 2.0 * tokens * n * k / us / 1e6
                entry.update({"pflops": tflops / 1e3, "frac_of_twice_measured_bf16": tflops / (2 * peak["bf16_tflops"]),
                              "frac_of_nominal_fp8": tflops / NOMINAL_FP8_TFLOPS})
            else:
                gbs = (n * k * elem + tokens * k * elem + tokens * n * 2 + n * 2) / us / 1e3
                entry.update({"gbs": gbs, "frac_of_hbm": gbs / peak["hbm_gbs"]})
            found[label] = entry
            del runner
    found["peak_kind"] = f"of {peak['kind']}"
    return found


def run_ours(args) -> None:
    import torch

    from aginfer_b200 import runtime as rt
    from aginfer_b200.build import build_all
    from aginfer_b200.replicas import ReplicaGroup
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the recipe has no CPU execution path")
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    group = ReplicaGroup.from_env("nccl")
    rank, local = group.rank, group.local_rank
    group.rank0_first(build_all)
    session_flags = 0 if args.no_pdl else rt.PROGRAMMATIC_LAUNCH
    uuid = str(torch.cuda.get_device_properties(local).uuid)
    sampler = ClockSampler(uuid if uuid.startswith("GPU-") else "GPU-" + uuid) if rank == 0 else None
    harness = Harness(group, torch.cuda.Stream(), sampler)
    peak = peaks()

    line, context = bench_action_head(args, group, harness, session_flags)
    if args.legs == "device":
        if rank == 0:
            print(json.dumps({k: line[k] for k in ("metric", "value", "unit", "n_gpus", "steps", "ms_per_step")} | {"legs": "device"}))
        if sampler is not None:
            sampler.stop()
        group.close()
        context["tmp"].cleanup()
        return
    line["chunk_hbm_frac_%s" % peak["kind"]] = context["per_chunk_bytes"] / (line["ms_per_step"] / 1e3) / 1e9 / peak["hbm_gbs"]
    if rank == 0:
        line["roofline"] = roofline_of_stream_gemm(context, harness, session_flags, peak)
    context["tmp"].cleanup()

    if args.configs == "all":
        episode = bench_episode(args, group, harness, session_flags, peak)      # every rank takes part
        line["configs"] = {"cfg5_episode": episode, "headline": "config 3 action chunks (metric / value); config 5 "
                           "episodes/s is the baseline's scaling figure, in configs.cfg5_episode.episodes_per_s"}
        if rank == 0 and group.world == 1:
            line["configs"]["cfg4_prefill"] = bench_prefill(harness, session_flags, peak)
            line["kernels"] = bench_kernels(harness, session_flags, peak)

    if rank == 0:
        line["clocks"] = sampler.stop() if sampler is not None else None
    # the GPU part is over: the other ranks leave now, so that nobody spins in a barrier on the host's cores while
    # rank 0 times the CPU oracle on them
    group.close()
    if rank == 0:
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_in_a_fresh_process(budget_s=15.0)
        print(json.dumps(line))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--configs", default="all", choices=["all", "3"],
                        help="'3': only the headline (configuration 3); 'all': also configurations 5 (every rank) "
                             "and, on one GPU, 4 and the isolated kernels")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--reference-budget", type=float, default=90.0,
                        help="--impl reference: stop after this many seconds of CPU work even if --steps is not reached")
    parser.add_argument("--no-pdl", action="store_true", help="launch without programmatic stream serialization")
    parser.add_argument("--legs", default="all", choices=["all", "device"],
                        help="'device' runs only the device-resident timed leg (small profiler captures)")
    args = parser.parse_args()
    if int(os.environ.get("RANK", "0")) == 0:
        # torch.distributed.run exports OMP_NUM_THREADS=1 to every rank; rank 0 also times the CPU oracle, which is
        # meant to use every host thread (torch is imported only after this point)
        for name in ("OMP_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[name] = str(os.cpu_count() or 1)
        # ... and NCCL pins the thread that initialises it to the cores next to its GPU; the worker threads of the
        # CPU leg would inherit that mask
        os.environ.setdefault("NCCL_IGNORE_CPU_AFFINITY", "1")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

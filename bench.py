#!/usr/bin/env python3
"""Headline benchmark: ``soap_step`` milliseconds per step on one 8192 x 8192 fp32 parameter.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Configuration (the reference's strong-scaling harness, ``scripts/slurm/frontier/
submit_soap_tp_scaling.sh:56-60`` and ``scripts/run_soap_tp_timing_gpu.py:126-209``, at the
benchmark shape): one 8192 x 8192 fp32 parameter, column shards (``shard_dim=1``), block size 128,
most-square process grid ((1,1), (1,2), (2,2), (2,4)), gradients i.i.d. N(0, 1) * 1e-2 seeded per
step, betas (0.95, 0.95), basis refresh every 10 steps.  STRONG scaling: the parameter is fixed
while N grows.  The first call (basis initialisation) is part of the warm-up.

Reported in one JSON line on rank 0:

* ``value``  -- device time of K ``soap_step`` calls whose gradients are resident on the GPU
  (CUDA events, barrier + synchronise on both sides, maximum over ranks) / K;
* ``e2e``    -- the same K calls through the public API where every step first copies its gradient
  shard from pinned host memory to the device and ends with a device-to-host read of the update
  norm (host wall clock around barrier + synchronise, maximum over ranks) / K;
* ``median_steady_ms``, ``refresh_step_ms``, ``init_ms`` -- from one CUDA-event pair per step (maximum over
  ranks per step): the median step without a refresh, the mean step with one, and the first call (both
  eigenbases), which is outside the timed region;
* ``host_enqueue_ms_median_steady`` -- host time the launching thread spends inside one steady ``soap_step`` call;
* ``check`` -- correctness figures computed after the timed region (``--no-check`` skips them): orthogonality
  of both bases, both Gram matrices against a float64 EMA of the same gradient sequence, and a 2048 x 2048
  side problem on the same grid against the single-GPU pipeline (``soap_tp_b200/bench/checks.py``).

For N > 1 the script expects one process per GPU (``python -m torch.distributed.run
--nproc-per-node N ...``); started without that environment it re-launches itself that way.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

# load every kernel of every module when the module is loaded: a first launch in the middle of the timed region
# would otherwise pay the lazy loading of that kernel's code (must be set before CUDA is initialised)
os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
ROOT = Path(__file__).resolve().parent
SIZE, BLOCK, SHARD_DIM, REFRESH = 8192, 128, 1, 10
GRAD_SCALE = 1e-2
METRIC = "soap_step ms/step, 8192^2 fp32 (device time, max over ranks; refresh every 10 steps included)"


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--size", type=int, default=SIZE, help="matrix size (the metric of record is 8192)")
    parser.add_argument("--block-size", type=int, default=BLOCK)
    parser.add_argument("--shard-dim", type=int, choices=(0, 1), default=SHARD_DIM)
    parser.add_argument("--refresh-interval", type=int, default=REFRESH)
    parser.add_argument("--basis-implementation", default=None)
    parser.add_argument("--stage-timing", action="store_true", help="also print per-stage device times (stderr)")
    parser.add_argument("--check", dest="check", action="store_true", default=True,
                        help="after the timed region, report correctness figures of the state it left (default)")
    parser.add_argument("--no-check", dest="check", action="store_false")
    args = parser.parse_args()
    if args.warmup < 1:
        parser.error("--warmup must be at least 1 (the first call initialises the bases)")
    return args


class ClockSampler:
    """Samples SM clocks and throttle reasons with ``nvidia-smi`` while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int) -> None:
        self.device_index = device_index
        self.lines: list[str] = []
        self.proc: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, maxima, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            fields = [f.strip() for f in line.split(",")]
            if len(fields) < 8:
                continue
            try:
                clocks.append(float(fields[1]))
                maxima.append(float(fields[2]))
                power.append(float(fields[3]))
            except ValueError:
                continue
            for name, flag in zip(names, fields[4:8]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "power_w_max": max(power) if power else None,
            "reasons": sorted(reasons),
            "samples": len(clocks),
        }


def relaunch_under_torchrun(args: argparse.Namespace) -> int:
    import socket

    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), str(Path(__file__).resolve()), *sys.argv[1:]]
    return subprocess.call(command)


def gradient_for(step: int, rank: int, shape, device, generator_cache: dict):
    """Seeded per step (and rank): i.i.d. N(0, 1) * 1e-2."""
    import torch

    generator = generator_cache.setdefault("g", torch.Generator(device=device))
    generator.manual_seed(1_000_003 * step + rank)
    return torch.randn(shape, generator=generator, dtype=torch.float32, device=device) * GRAD_SCALE


def run(args: argparse.Namespace) -> int:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)

    sys.path.insert(0, str(ROOT))
    from soap_tp_b200.layout import most_square_grid

    size = args.size
    grid = most_square_grid(world)
    if size % world:
        raise SystemExit(f"size {size} must be divisible by {world} ranks")
    shard_shape = (size // world, size) if args.shard_dim == 0 else (size, size // world)

    status_wait_seconds = lambda: 0.0
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline"))
        import reference_arm

        step_fn, launches, basis = reference_arm.make_step(
            size=size, block_size=args.block_size, shard_dim=args.shard_dim, grid=grid,
            refresh_interval=args.refresh_interval, device=device)
    else:
        from soap_tp_b200 import soap_step
        from soap_tp_b200.engine import kernels

        basis = args.basis_implementation or "householder"
        state: dict = {}

        def make_step(side: int, target: dict):
            return lambda gradient: soap_step(
                gradient, target, global_shape=(side, side), shard_dim=args.shard_dim, block_size=args.block_size,
                process_grid_shape=grid, basis_refresh_interval=args.refresh_interval, basis_implementation=basis)

        step_fn = make_step(size, state)

        launches = kernels.total_launches
        status_wait_seconds = lambda: kernels._StatusMonitor.waited_seconds
        if args.stage_timing:
            from soap_tp_b200.profiling import GLOBAL_STAGE_TIMER

            GLOBAL_STAGE_TIMER.enabled = True

    def fence() -> None:
        dist.barrier()
        torch.cuda.synchronize(device)

    cache: dict = {}
    pool = 4  # distinct resident gradients cycled through the timed region
    counter = 0
    history: list[int] = []      # gradient index of every call so far (for the checks after the timed region)

    def max_over_ranks(values) -> list[float]:
        tensor = torch.tensor(list(values), dtype=torch.float64, device=device)
        dist.all_reduce(tensor, op=dist.ReduceOp.MAX)
        return [float(v) for v in tensor.tolist()]

    def step_summary(per_step_ms: list[float], first_call_index: int) -> dict:
        """Median of the steps without a refresh and mean of those with one (call c refreshes when c % interval == 0)."""
        steady = [t for i, t in enumerate(per_step_ms) if (first_call_index + i) % args.refresh_interval]
        refresh = [t for i, t in enumerate(per_step_ms) if (first_call_index + i) % args.refresh_interval == 0]
        return {
            "median_steady_ms": round(statistics.median(steady), 4) if steady else None,
            "refresh_step_ms": round(sum(refresh) / len(refresh), 4) if refresh else None,
            "refresh_steps_timed": len(refresh),
            "step_ms": [round(t, 3) for t in per_step_ms],
        }

    # ---- warm-up (first call = basis initialisation) ----
    init_start = time.perf_counter()
    init_events = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    for _ in range(args.warmup):
        if counter == 0:
            fence()
            init_events[0].record()
        step_fn(gradient_for(counter, rank, shard_shape, device, cache))
        history.append(counter)
        counter += 1
        if counter == 1:
            init_events[1].record()
            fence()
            init_seconds = time.perf_counter() - init_start
            init_ms = max_over_ranks([init_events[0].elapsed_time(init_events[1])])[0]
    fence()

    # ---- device-timed region ----
    # The reference arm needs seconds per steady step and minutes per refresh step at the size of record,
    # so it runs ONE loop (the end-to-end one below) and takes both numbers from it: CUDA events around that
    # loop give the device time (the prefetched copy and the 4-byte read-back are under 1 % of its step).
    single_loop = args.impl == "reference"
    budget_seconds = float(os.environ.get("SOAP_TP_REFERENCE_BUDGET_SECONDS", "1200"))
    # Everything allocated so far (modules, workspaces, caches) is permanent: keep the cyclic collector from walking
    # it again in the middle of a launch-bound refresh step (both arms; a full collection of a process that has
    # imported torch takes tens of milliseconds).
    import gc

    gc.collect()
    gc.freeze()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = launches()
    device_ms = None
    if not single_loop:
        if args.impl == "ours" and args.stage_timing:
            GLOBAL_STAGE_TIMER.reset()
        resident = [gradient_for(counter + i, rank, shard_shape, device, cache) for i in range(pool)]
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
        fence()
        marks[0].record()
        host_ms = []
        for i in range(args.steps):
            host_begin, waited = time.perf_counter(), status_wait_seconds()
            step_fn(resident[i % pool])
            host_ms.append((time.perf_counter() - host_begin - (status_wait_seconds() - waited)) * 1e3)
            marks[i + 1].record()
        fence()
        history.extend(counter + i % pool for i in range(args.steps))
        device_ms = torch.tensor([marks[0].elapsed_time(marks[-1])], dtype=torch.float64, device=device)
        dist.all_reduce(device_ms, op=dist.ReduceOp.MAX)
        per_step = max_over_ranks(marks[i].elapsed_time(marks[i + 1]) for i in range(args.steps))
        summary = step_summary(per_step, len(history) - args.steps)
        # host time to enqueue one step (rank 0's median over the steps without a refresh), without the wait for the
        # previous step's status word: far below the device time means the device, not the launching thread, sets
        # the pace
        first = len(history) - args.steps
        steady_host = [t for i, t in enumerate(host_ms) if (first + i) % args.refresh_interval]
        summary["host_enqueue_ms_median_steady"] = round(statistics.median(steady_host), 3) if steady_host else None
        refresh_host = [t for i, t in enumerate(host_ms) if (first + i) % args.refresh_interval == 0]
        summary["host_enqueue_ms_refresh"] = round(sum(refresh_host) / len(refresh_host), 3) if refresh_host else None
        launches_timed = launches() - launches_before
        if args.impl == "ours" and args.stage_timing:
            stages = GLOBAL_STAGE_TIMER.summary()
            GLOBAL_STAGE_TIMER.enabled = False
            if rank == 0:
                print(json.dumps({"stage_ms_per_step_max_over_ranks":
                                  {n: round(v / args.steps, 3) for n, v in stages.items()}}), file=sys.stderr)
        clocks = sampler.stop() if rank == 0 else {}
        counter += args.steps

    # ---- end-to-end region: pinned host -> device every step, metric back to the host ----
    host_pool = [torch.empty(shard_shape, dtype=torch.float32).pin_memory() for _ in range(pool)]
    for i, buffer in enumerate(host_pool):
        buffer.copy_(gradient_for(counter + i, rank, shard_shape, device, cache))
    # Every step's input crosses PCIe inside the timed region; the copy of step i + 1 is issued on a copy
    # stream while step i computes (two device buffers), as an input pipeline would do it.
    device_buffers = [torch.empty(shard_shape, dtype=torch.float32, device=device) for _ in range(2)]
    copy_stream = torch.cuda.Stream(device=device)
    arrived = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]
    used = [False, False]
    # the step's metric comes back into pinned memory every step; the host reads it one step later, as a
    # training loop that logs its loss without stalling the device does
    metric_host = torch.empty(2, dtype=torch.float32).pin_memory()
    metric_ready = [torch.cuda.Event() for _ in range(2)]
    metrics_read = []

    def prefetch(index: int) -> None:
        slot = index % 2
        with torch.cuda.stream(copy_stream):
            if used[slot]:
                copy_stream.wait_event(consumed[slot])
            device_buffers[slot].copy_(host_pool[index % pool], non_blocking=True)
            arrived[slot].record(copy_stream)

    # warm the machinery of this loop that the device-timed loop never used (copy stream, pinned transfers in both
    # directions, the norm kernel) without taking an optimizer step
    with torch.cuda.stream(copy_stream):
        device_buffers[1].copy_(host_pool[0], non_blocking=True)
    copy_stream.synchronize()
    metric_host[0:1].copy_(torch.linalg.vector_norm(device_buffers[1]).reshape(1), non_blocking=True)
    fence()
    loop_start, loop_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    loop_marks = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    e2e_first_call = len(history)
    e2e_start = time.perf_counter()
    loop_start.record()
    loop_marks[0].record()
    prefetch(0)
    steps_done = 0
    e2e_host_ms: list[float] = []
    for i in range(args.steps):
        slot = i % 2
        if i + 1 < args.steps:
            prefetch(i + 1)
        torch.cuda.current_stream().wait_event(arrived[slot])
        host_begin, waited = time.perf_counter(), status_wait_seconds()
        update = step_fn(device_buffers[slot])
        e2e_host_ms.append(round((time.perf_counter() - host_begin - (status_wait_seconds() - waited)) * 1e3, 3))
        consumed[slot].record()
        used[slot] = True
        metric_host[slot:slot + 1].copy_(torch.linalg.vector_norm(update).reshape(1), non_blocking=True)
        metric_ready[slot].record()
        if i > 0:
            metric_ready[1 - slot].synchronize()
            metrics_read.append(float(metric_host[1 - slot]))
        steps_done += 1
        loop_marks[steps_done].record()
        history.append(counter + i % pool)
        if single_loop:
            # every rank must take the same decision: agree on the slowest rank's clock
            elapsed = torch.tensor([time.perf_counter() - e2e_start], dtype=torch.float64, device=device)
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
            if float(elapsed.item()) > budget_seconds and steps_done < args.steps:
                break
    loop_stop.record()
    if steps_done:
        metric_ready[(steps_done - 1) % 2].synchronize()
        metrics_read.append(float(metric_host[(steps_done - 1) % 2]))
    fence()
    e2e_ms = torch.tensor([(time.perf_counter() - e2e_start) * 1e3], dtype=torch.float64, device=device)
    dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_step_ms = [round(t, 3) for t in max_over_ranks(loop_marks[i].elapsed_time(loop_marks[i + 1]) for i in range(steps_done))]
    if single_loop:
        device_ms = torch.tensor([loop_start.elapsed_time(loop_stop)], dtype=torch.float64, device=device)
        dist.all_reduce(device_ms, op=dist.ReduceOp.MAX)
        launches_timed = launches() - launches_before
        clocks = sampler.stop() if rank == 0 else {}
        per_step = max_over_ranks(loop_marks[i].elapsed_time(loop_marks[i + 1]) for i in range(steps_done))
        summary = step_summary(per_step, e2e_first_call)
        if steps_done < args.steps:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  f"the unmodified reference did not finish {args.steps} steps within "
                                  f"{budget_seconds:.0f} s at {world} GPU(s): {steps_done} steps took "
                                  f"{float(e2e_ms.item()) / 1e3:.0f} s (refresh steps run Python index planning "
                                  "over every matrix element)"}), flush=True)
            dist.destroy_process_group()
            return 0

    check: dict | None = None
    if args.impl == "ours":
        from soap_tp_b200.engine import kernels

        kernels.check_status()
        if args.stage_timing and rank == 0:
            print(json.dumps({"launch_counts": kernels.LAUNCH_COUNTS}), file=sys.stderr)
        if args.check:
            from soap_tp_b200.bench import checks

            def full_gradient(index: int):
                shards = [gradient_for(index, r, shard_shape, device, cache) for r in range(world)]
                return shards[0] if world == 1 else torch.cat(shards, dim=args.shard_dim)

            check = {
                "left_basis_max_abs_QtQ_minus_I": checks.basis_orthogonality(state["left_basis"], size, args.block_size, grid),
                "right_basis_max_abs_QtQ_minus_I": checks.basis_orthogonality(state["right_basis"], size, args.block_size, grid),
                "gram_relative_error_vs_float64": checks.gram_error(state, full_gradient, history, (size, size),
                                                                    args.block_size, grid, 0.95),
                "steps_behind_the_state": len(history),
            }
            side = min(2048, size)
            if world > 1 and side % world == 0:
                side_state: dict = {}
                check["side_problem_vs_single_gpu_pipeline"] = checks.side_problem_against_one_gpu(
                    lambda: make_step(side, side_state), side, args.block_size, grid, args.shard_dim,
                    steps=args.refresh_interval + 2, interval=args.refresh_interval, implementation=basis, state=side_state)
            else:
                check["side_problem_vs_single_gpu_pipeline"] = None    # one rank: the two paths are the same code
            kernels.check_status()

    ms_per_step = float(device_ms.item()) / args.steps
    e2e_per_step = float(e2e_ms.item()) / args.steps
    shard_bytes = shard_shape[0] * shard_shape[1] * 4
    if rank == 0:
        line = {
            "metric": METRIC,
            "value": round(ms_per_step, 4),
            "unit": "ms/step",
            "impl": args.impl,
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": False,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "fp32 state; 3xTF32 tcgen05 products (fp32-class accuracy)" if args.impl == "ours" else "fp32",
            "data": "synthetic: gradients i.i.d. N(0,1)*1e-2 seeded per step; random-init state from the first gradient",
            "config": {
                "model": f"one {size}x{size} fp32 parameter (SOAP-TP state: L, R, Q_L, Q_R, momentum, variance)",
                "global_batch": None,
                "seq_len": None,
                "parallelism": f"tp{world} column shards, 2-D block-cyclic grid {grid[0]}x{grid[1]}, block {args.block_size}",
                "shard_dim": args.shard_dim,
                "basis_refresh_interval": args.refresh_interval,
                "l2": "no flush: each step streams > 1 GiB of operand planes and state per GPU (L2 is 126 MB); "
                      f"{pool} distinct resident gradients are cycled",
            },
            # per-arm facts, kept out of `config` so that both arms print the same workload description
            "run_info": {
                "basis_implementation": basis,
                "initialization_seconds": round(init_seconds, 3),
                "timed_loop": ("one loop: device events around the end-to-end loop" if single_loop
                               else "device loop on resident gradients, then a separate end-to-end loop"),
            },
            "init_ms": round(init_ms, 2),
            **summary,
            "check": check,
            "clocks": clocks,
            "e2e": {
                "value": round(e2e_per_step, 4),
                "unit": "ms/step",
                "h2d_bytes_per_step": shard_bytes,
                "d2h_bytes_per_step": 4,
                "step_ms": e2e_step_ms,
                "host_ms_rank0": e2e_host_ms,     # host time inside each call (without the status-word wait)
            },
            "gpu_launches": int(launches_timed),
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
    return 0


def main() -> int:
    args = parse_args()
    if args.impl == "reference" and not (ROOT / "baseline" / "_ref" / "soap_tp").exists():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed "
                          "(python -m pip install --no-index --no-build-isolation --target baseline/_ref "
                          "<checkout of the reference>)"}), flush=True)
        return 0
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        return relaunch_under_torchrun(args)
    return run(args)


if __name__ == "__main__":
    raise SystemExit(main())

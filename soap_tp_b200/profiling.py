"""Tracing and timing protocols.

Two line-oriented JSON protocols of the reference are kept byte-compatible so that existing
log tooling keeps working:

* ``SOAP_PROFILE {json}`` -- value taps emitted by rank 0 when the environment variable
  ``SOAP_PROFILE`` is one of ``1/true/yes`` (optionally restricted to the comma-separated step
  list ``SOAP_PROFILE_STEPS``); fields ``impl, step, stage, shape, dtype, values`` with compact
  separators (``src/soap_tp/soap.py:26-57``).  A disabled tap costs one environment lookup and
  no collective (``soap.py:66,84``).
* ``SOAP_TIMING {json}`` -- benchmark events with sorted keys
  (``scripts/run_soap_tp_timing_gpu.py:31-37``).

Added here: per-stage device timers (CUDA events, reported as the maximum over ranks) and NVTX
ranges, both off unless ``SOAP_STAGE_TIMING=1``.
"""
from __future__ import annotations

import contextlib
import json
import os
from collections import defaultdict
from typing import Dict, List, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

PROFILE_PREFIX = "SOAP_PROFILE "
TIMING_PREFIX = "SOAP_TIMING "


def profile_enabled(step: int) -> bool:
    if os.environ.get("SOAP_PROFILE", "").lower() not in {"1", "true", "yes"}:
        return False
    requested = os.environ.get("SOAP_PROFILE_STEPS")
    if not requested:
        return True
    return step in {int(item.strip()) for item in requested.split(",") if item.strip()}


def emit_profile_tensor(stage: str, step: int, tensor: Tensor, impl: str = "tp") -> None:
    if dist.is_initialized() and dist.get_rank() != 0:
        return
    detached = tensor.detach()
    print(
        PROFILE_PREFIX
        + json.dumps(
            {
                "impl": impl,
                "step": step,
                "stage": stage,
                "shape": list(detached.shape),
                "dtype": str(detached.dtype).removeprefix("torch."),
                "values": detached.cpu().reshape(-1).tolist(),
            },
            separators=(",", ":"),
        ),
        flush=True,
    )


def profile_tp_shard(stage: str, step: int, tensor: Tensor, shard_dim: int) -> None:
    """Tap a tensor-parallel shard: all ranks gather, rank 0 prints the full matrix."""
    if not profile_enabled(step):
        return
    from .ops import _hostpath as host

    source = tensor.detach().contiguous()
    if source.is_cuda and dist.get_backend() == "gloo":
        source = source.cpu()
    emit_profile_tensor(stage, step, host.gather_tp_shards(source, shard_dim))


def profile_block_cyclic(stage: str, step: int, tensor: Tensor, global_shape, block_size: int, grid) -> None:
    """Tap a packed block-cyclic buffer."""
    if not profile_enabled(step):
        return
    from .ops import _hostpath as host

    source = tensor.detach()
    if source.is_cuda and dist.get_backend() == "gloo":
        source = source.cpu()
    emit_profile_tensor(stage, step, host.gather_block_cyclic(source, tuple(global_shape), block_size, grid))


def emit_timing(event: str, **values: object) -> None:
    """Rank 0 prints one ``SOAP_TIMING`` line (keys sorted, as the reference's driver does)."""
    if dist.is_initialized() and dist.get_rank() != 0:
        return
    print(TIMING_PREFIX + json.dumps({"event": event, **values}, sort_keys=True), flush=True)


class StageTimer:
    """Accumulates per-stage device time with CUDA events (host clock on CPU tensors).

    ``with timer.stage("rotate_forward"): ...`` records a start/stop event pair on the current
    stream; :meth:`summary` synchronises once, sums the pairs per stage and reduces with MAX
    over ranks so the figure reported is that of the slowest rank.
    """

    def __init__(self, enabled: bool | None = None) -> None:
        if enabled is None:
            enabled = os.environ.get("SOAP_STAGE_TIMING", "") in {"1", "true", "yes"}
        self.enabled = enabled
        self._pairs: Dict[str, List[Tuple[object, object]]] = defaultdict(list)

    @contextlib.contextmanager
    def stage(self, name: str, device: torch.device | None = None):
        if not self.enabled:
            yield
            return
        if device is not None and device.type == "cuda":
            torch.cuda.nvtx.range_push(name)
            start = torch.cuda.Event(enable_timing=True)
            stop = torch.cuda.Event(enable_timing=True)
            start.record()
            try:
                yield
            finally:
                stop.record()
                torch.cuda.nvtx.range_pop()
                self._pairs[name].append((start, stop))
        else:
            import time

            begin = time.perf_counter()
            try:
                yield
            finally:
                self._pairs[name].append((begin, time.perf_counter()))

    def summary(self, reduce_over_ranks: bool = True) -> Dict[str, float]:
        """Milliseconds per stage (sum over calls), max over ranks."""
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        totals: Dict[str, float] = {}
        for name, pairs in self._pairs.items():
            total = 0.0
            for start, stop in pairs:
                if isinstance(start, float):
                    total += (stop - start) * 1e3
                else:
                    total += start.elapsed_time(stop)
            totals[name] = total
        if reduce_over_ranks and dist.is_initialized() and dist.get_world_size() > 1 and totals:
            names = sorted(totals)
            values = torch.tensor([totals[n] for n in names], dtype=torch.float64)
            if dist.get_backend() == "nccl":
                values = values.cuda()
            dist.all_reduce(values, op=dist.ReduceOp.MAX)
            totals = dict(zip(names, values.cpu().tolist()))
        return totals

    def reset(self) -> None:
        self._pairs.clear()


GLOBAL_STAGE_TIMER = StageTimer()

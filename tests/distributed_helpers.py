"""Launch helpers for multi-rank tests: real processes, gloo (CPU) control plane, 127.0.0.1."""
from __future__ import annotations

import datetime
import os
import socket
import traceback
from typing import Callable

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def _entry(rank: int, world_size: int, port: int, backend: str, fn: Callable, args: tuple, errors,
           pg_timeout: float = 0.0) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world_size), LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank % torch.cuda.device_count())
        elif torch.cuda.is_available():
            torch.cuda.set_device(rank % torch.cuda.device_count())
        extra = {"timeout": datetime.timedelta(seconds=pg_timeout)} if pg_timeout > 0 else {}
        dist.init_process_group(backend, rank=rank, world_size=world_size, **extra)
        fn(rank, world_size, *args)
    except Exception:
        errors.put((rank, traceback.format_exc()))
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn: Callable, world_size: int, *args, backend: str = "gloo", timeout: float = 300.0,
                    pg_timeout: float = 0.0) -> None:
    """Run ``fn(rank, world_size, *args)`` in ``world_size`` processes; raise on any failure.
    ``pg_timeout`` > 0 sets the process group's collective timeout in seconds (failure-detection tests)."""
    ctx = mp.get_context("spawn")
    errors = ctx.SimpleQueue()
    port = free_port()
    procs = [
        ctx.Process(target=_entry, args=(rank, world_size, port, backend, fn, args, errors, pg_timeout))
        for rank in range(world_size)
    ]
    for proc in procs:
        proc.start()
    failed = []
    for proc in procs:
        proc.join(timeout)
        if proc.is_alive():
            proc.terminate()
            proc.join(5)
            failed.append(f"pid {proc.pid} timed out")
    messages = []
    while not errors.empty():
        rank, text = errors.get()
        messages.append(f"--- rank {rank} ---\n{text}")
    for proc in procs:
        if proc.exitcode not in (0, None) and not messages:
            failed.append(f"pid {proc.pid} exit code {proc.exitcode}")
    if messages or failed:
        raise AssertionError("\n".join(messages + failed))

"""Symmetric-memory communicator: the data plane of the multi-GPU engine.

One :class:`Communicator` per process (default world, row-major ``Pr x Pc`` grid).  It owns

* **symmetric segments** -- device buffers that exist with the same size and meaning on every
  rank, exported with CUDA IPC and mapped by every peer, so this package's kernels read a peer's
  buffer with plain global loads over NVLink (``csrc/comm.cu``);
* a **barrier**: a device-side flag barrier with a bounded spin when every rank has its own GPU,
  or a host-side barrier (stream synchronise + control-plane barrier) when ranks share a GPU,
  because kernels that wait on one another must never be separate launches on one device;
* a **control plane** for small host-side exchanges (IPC handles, shape checks): a gloo group,
  created next to an NCCL default group when necessary.

The reference has two rank-matched worlds instead -- ``torch.distributed`` for its Python ops and
``MPI_COMM_WORLD`` inside SLATE/ELPA (``src/soap_tp/ops/factorizations.py:85-101``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
from torch import Tensor



from ..engine.kernels import SoapCommTimeout  # noqa: E402  (re-exported: a bounded device-side wait on a peer ran out)


class _RawBuffer:
    """Expose a raw device allocation to torch through the CUDA array interface."""

    def __init__(self, ptr: int, numel: int, typestr: str) -> None:
        self.__cuda_array_interface__ = {
            "shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 2,
        }


@dataclass
class SymmetricSegment:
    name: str
    numel: int
    dtype: torch.dtype
    local: Tensor            # this rank's buffer (flat)
    peer_ptrs: List[int]     # base address of every rank's buffer in this process's address space
    peer_table: Tensor       # int64 device tensor of the same addresses (kernel argument)


def default_barrier_timeout() -> float:
    """Budget of one device-side barrier spin in seconds (``SOAP_TP_BARRIER_TIMEOUT_S``, default 30).

    The spin only has to cover the skew between ranks that are all running device work; waits that can be
    long by design (a leader rank factoring a whole matrix, a rank that saves a checkpoint) are taken on the
    host first, see :meth:`Communicator.barrier`.  When the budget runs out the kernel sets the status word and
    the next ``soap_step`` raises :class:`SoapCommTimeout`.
    """
    return float(os.environ.get("SOAP_TP_BARRIER_TIMEOUT_S", "30"))


class Communicator:
    CHANNELS = 4     # independent barrier channels: barriers issued on different streams use different channels

    def __init__(self, device: torch.device, *, group=None, barrier_timeout_s: Optional[float] = None) -> None:
        """``group``: the process group whose ranks form the grid (default: the world).  Every rank of the group
        must construct its communicator at the same point of the program."""
        from ..engine import kernels

        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialized first.")
        self._C = kernels._C
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.barrier_timeout_s = default_barrier_timeout() if barrier_timeout_s is None else float(barrier_timeout_s)
        # Control plane for small host-side exchanges.  A gloo-capable group serves as it is; for an NCCL-only
        # world a gloo twin is created (collective over the world, which is where a world communicator is built);
        # an NCCL-only sub-group is used directly -- object collectives and barriers work there through the device.
        backend = str(dist.get_backend(group))
        whole_world = group is None or group is dist.group.WORLD
        if "gloo" in backend:
            self.control = dist.group.WORLD if whole_world else group
        elif whole_world:
            self.control = dist.new_group(backend="gloo")
        else:
            self.control = group
        self.control_on_device = "gloo" not in str(dist.get_backend(self.control))
        self.segments: Dict[str, SymmetricSegment] = {}
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        identity = (os.uname().nodename, bytes(self._C.device_uuid(index)))
        everyone: List[Optional[tuple]] = [None] * self.world
        dist.all_gather_object(everyone, identity, group=self.control)
        self.exclusive_gpus = len(set(everyone)) == self.world
        if len({host for host, _ in everyone}) != 1:
            raise RuntimeError("the CUDA IPC communicator needs all ranks on one node.")
        self.use_device_barrier = self.exclusive_gpus and os.environ.get("SOAP_TP_HOST_BARRIER", "0") != "1"
        self._channel_stride = max(self.world, 64)
        self._pads = self.segment("signal_pads", self.CHANNELS * self._channel_stride, torch.int32) if self.world > 1 else None
        self._epochs = [0] * self.CHANNELS
        self.barrier_count = 0

    # ---- symmetric segments ------------------------------------------------------------------
    def segment(self, name: str, numel: int, dtype: torch.dtype = torch.float32) -> SymmetricSegment:
        """Create (collectively) or fetch the symmetric segment ``name``.

        Every rank must request the same names with the same sizes in the same order.
        """
        existing = self.segments.get(name)
        if existing is not None:
            if existing.numel < numel or existing.dtype != dtype:
                raise ValueError(f"segment {name!r} exists with {existing.numel} x {existing.dtype}.")
            return existing
        itemsize = torch.empty((), dtype=dtype).element_size()
        with torch.cuda.device(self.device):
            ptr, handle = self._C.ipc_alloc(max(1, numel) * itemsize)
            handles: List[Optional[tuple]] = [None] * self.world
            dist.all_gather_object(handles, (numel, bytes(handle)), group=self.control)
            if any(h[0] != numel for h in handles):
                raise ValueError(f"segment {name!r}: sizes differ across ranks: {[h[0] for h in handles]}.")
            peer_ptrs = [ptr if r == self.rank else self._C.ipc_open(handles[r][1]) for r in range(self.world)]
        typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.int64: "<i8"}[dtype]
        local = torch.as_tensor(_RawBuffer(ptr, max(1, numel), typestr), device=self.device)
        table = torch.tensor(peer_ptrs, dtype=torch.int64, device=self.device)
        seg = SymmetricSegment(name, numel, dtype, local, peer_ptrs, table)
        self.segments[name] = seg
        dist.barrier(group=self.control)
        return seg

    # ---- ordering ----------------------------------------------------------------------------
    def barrier(self, *, after_long_work: bool = False, channel: int = 0) -> None:
        """All work enqueued so far on every rank's current stream happens-before anything
        enqueued after this call on any rank.

        ``channel``: barriers that run on different streams at the same time must use different channels (each has
        its own flags and epoch counter); every rank issues the barriers of a channel in the same order.

        ``after_long_work``: some rank has just enqueued work that may take longer than the device barrier's
        spin budget (a dense factorisation on a leader rank).  Every rank then first drains its own stream and
        meets the others on the control plane, so the device-side spin that follows only covers microseconds
        and cannot run out while a peer is still computing.
        """
        if self.world == 1:
            return
        self.barrier_count += 1
        if self.use_device_barrier and after_long_work:
            torch.cuda.current_stream().synchronize()
            dist.barrier(group=self.control)
        if self.use_device_barrier:
            from ..engine import kernels

            self._epochs[channel] += 1
            self._C.device_barrier(self._pads.peer_table.data_ptr(), self.rank, self.world, self._epochs[channel],
                                   kernels.status_word(self.device).data_ptr(), float(self.barrier_timeout_s),
                                   torch.cuda.current_stream().cuda_stream, channel * self._channel_stride)
            kernels._count("barrier_kernel")
        else:
            torch.cuda.current_stream().synchronize()
            dist.barrier(group=self.control)

    def check(self) -> None:
        """Synchronise and raise if a device-side wait timed out on this rank."""
        from ..engine import kernels

        kernels.check_status(self.device)

    def gather_ints(self, values: List[int]) -> List[List[int]]:
        """The integer lists of every rank, in rank order (control plane)."""
        everyone: List[Optional[List[int]]] = [None] * self.world
        dist.all_gather_object(everyone, [int(v) for v in values], group=self.control)
        return [list(v) for v in everyone]

    def all_equal(self, values: Tensor) -> bool:
        """True if the int64 tensor is identical on every rank (control plane)."""
        if self.world == 1:
            return True
        if self.control_on_device:
            values = values.to(self.device)
        low, high = values.clone(), values.clone()
        dist.all_reduce(low, op=dist.ReduceOp.MIN, group=self.control)
        dist.all_reduce(high, op=dist.ReduceOp.MAX, group=self.control)
        return bool(torch.equal(low, high))


_COMMUNICATORS: Dict[tuple, Communicator] = {}


def group_key(group) -> int:
    """Identity of a process group for caches (0: the world)."""
    return 0 if group is None or group is dist.group.WORLD else id(group)


def get_communicator(device: torch.device, group=None) -> Communicator:
    key = (str(torch.device(device)), group_key(group))
    comm = _COMMUNICATORS.get(key)
    if comm is None:
        comm = Communicator(torch.device(device), group=group)
        _COMMUNICATORS[key] = comm
    return comm


def reset_communicators() -> None:
    _COMMUNICATORS.clear()

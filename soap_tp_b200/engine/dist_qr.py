"""Householder QR spread over the ranks of a grid.

The reference factors a packed matrix with ``slate::geqrf`` + ``unmqr`` over all MPI ranks
(``src/soap_tp/csrc/slate_bindings.cpp:125-189``).  Here the work of one factorisation is divided by what
bounds it.  The chain of panel factorisations (128 Householder columns each) is a sequence of short,
latency-bound steps whose partial sums are exchanged through one GPU's L2; sending those exchanges over NVLink
would only lengthen it, so one rank -- the job's *leader* -- runs the chain together with the trailing-matrix
updates that the next panel depends on.  The other two thirds of the arithmetic, the accumulation of the explicit
orthogonal factor ``Q^T <- H_p^T Q^T``, depends on the chain only through each panel's reflectors.  It is done
by the other ranks of the job's group (*workers*), each owning a slice of the columns of ``Q^T``:

    leader   gather A[:, order] from all ranks -> panel p -> Z_p = T_p V_p^T -> publish (V_p, Z_p), flag p
             -> trailing update -> panel p+1 ...
    worker   wait flag p -> pull V_p, Z_p from the leader's memory (NVLink) -> W = V_p^T Q^T[j0:, slice]
             -> Q^T[j0:, slice] -= Z_p^T W     (3xTF32 tcgen05 GEMMs; pulls of panel p+1 overlap the products of p)
    all      pull the tiles of Q they own in the packed layout from the workers' slices

Two factorisations (left and right basis of a refresh) use disjoint halves of the ranks and run at the same
time.  Progress is announced by a flag in the leader's symmetric memory that workers poll from the device
with a time budget; when ranks share a GPU (tests) the announcement travels over the host control plane instead,
because kernels that wait for one another must not be separate launches on one device.  Groups of one rank
(two ranks in all) fall back to the single-GPU factorisation on the leader.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import owned_indices
from . import kernels as k
from . import qr as qr_driver

_C = k._C
PANEL = qr_driver.PANEL


def _planes_in(buffer: Tensor, start: int, depth: int, cols: int) -> Tuple[k.Planes, int]:
    """Operand planes of a ``depth x cols`` matrix laid out in ``buffer`` from element ``start``."""
    ld = max(4, k.round_up(depth, 4))
    count = max(1, cols) * ld
    hi = buffer[start:start + count].view(max(1, cols), ld)
    lo = buffer[start + count:start + 2 * count].view(max(1, cols), ld)
    return k.Planes(hi, lo, depth, cols, ld), start + 2 * count


def group_of(job: int, jobs: int, world: int) -> Tuple[int, List[int]]:
    """Leader and workers of factorisation ``job`` of ``jobs`` concurrent ones."""
    first, last = (job * world) // jobs, ((job + 1) * world) // jobs
    return first, list(range(first + 1, last))


def worker_slices(n: int, workers: int) -> List[Tuple[int, int]]:
    """Column ranges of ``Q^T`` (rows of ``Q``), multiples of the panel width, one per worker."""
    blocks = -(-n // PANEL)
    bounds = [min(n, PANEL * ((blocks * w) // workers)) for w in range(workers)] + [n]
    return [(bounds[w], bounds[w + 1]) for w in range(workers)]


class _Publication:
    """The leader's reflectors in a symmetric segment: ``V`` (n x n planes) and one ``Z_p`` slot per panel."""

    def __init__(self, e, job: int, n: int) -> None:
        self.e, self.job, self.n = e, job, n
        self.panels = -(-n // PANEL)
        ldn = max(4, k.round_up(n, 4))
        self.v_numel = 2 * n * ldn
        self.z_slot = 2 * n * PANEL
        self.segment = e.comm.segment(f"qr_publication{job}:{n}", self.v_numel + self.panels * self.z_slot)
        self.V, _ = _planes_in(self.segment.local, 0, n, n)
        self.flags = e.comm.segment("qr_flags", 64, torch.int32)
        self.base = 0
        self.workers: List[int] = []
        self._addresses: Dict[int, Tensor] = {}

    def flag_value(self, p: int) -> int:
        """Announcement number of panel ``p`` of the current call as a signed 32-bit value; consumers compare by
        wrapping difference, so the numbers may wrap around."""
        value = (self.base + p + 1) & 0xFFFFFFFF
        return value - (1 << 32) if value >= (1 << 31) else value

    def addresses(self, leader: int) -> Tensor:
        """Device table of the plane addresses in ``leader``'s copy of the segment: V hi, V lo, then (Z_p hi, Z_p lo)."""
        table = self._addresses.get(leader)
        if table is None:
            base = self.segment.peer_ptrs[leader]
            entries = [base, base + 4 * (self.v_numel // 2)]
            for p in range(self.panels):
                z_base = base + 4 * (self.v_numel + p * self.z_slot)
                entries += [z_base, z_base + 4 * (self.z_slot // 2)]
            table = self._addresses[leader] = torch.tensor(entries, dtype=torch.int64, device=self.e.device)
        return table

    def z(self, p: int) -> k.Planes:
        planes, _ = _planes_in(self.segment.local, self.v_numel + p * self.z_slot, PANEL, self.n)
        return planes

    def announce(self, p: int) -> None:
        if self.e.comm.use_device_barrier:
            _C.signal_flag(self.flags.local[self.job:].data_ptr(), self.flag_value(p), k._stream())
            k._count("signal_flag_kernel")
        else:
            torch.cuda.current_stream().synchronize()
            token = torch.tensor([self.base + p + 1], dtype=torch.int64)
            for worker in self.workers:
                dist.send(token, dst=worker, group=self.e.comm.control)


def _copy_from(table_entry: int, pitch: int, cols_total: int, row0: int, col0: int, out: Tensor, rows: int, cols: int) -> None:
    """``out[:rows, :cols] <- peer_plane[row0:, col0:]`` for a column-major plane of pitch ``pitch`` in a peer's
    memory; ``table_entry`` is the device address of the int64 that holds the plane's address.  The plane is
    described to the pull kernel as a one-rank block-cyclic matrix (block size 4 keeps its 16-byte path open)."""
    d_j = out.stride(0)      # planes are stored [col][depth]
    _C.dist_gather(table_entry, 0, pitch, cols_total, 4, 4, 1, 1, 1, 0, 1, 1, row0, 0, 0, 1, 1, col0, 0, 0, 0, 0, 0,
                   out.data_ptr(), 0, 1, d_j, rows, cols, k._stream())
    k._count("dist_gather_kernel")


class _Worker:
    """One worker's buffers for one (job, n): its slice of ``Q^T`` and double-buffered copies of (V_p, Z_p)."""

    def __init__(self, e, n: int, width: int) -> None:
        device = e.device
        self.qt = k.Planes.empty(n, width, device)
        self.v = [k.Planes.empty(n, PANEL, device) for _ in range(2)]
        self.z = [k.Planes.empty(PANEL, n, device) for _ in range(2)]
        self.w = k.Planes.empty(PANEL, width, device)
        self.scratch = {"partials": torch.empty(16 * PANEL * max(width, PANEL), dtype=torch.float32, device=device)}
        self.pull_stream = torch.cuda.Stream(device=device)
        self.landed = [torch.cuda.Event() for _ in range(2)]
        self.consumed = [torch.cuda.Event() for _ in range(2)]


_WORKERS: Dict[tuple, _Worker] = {}
_PUBLICATIONS: Dict[tuple, _Publication] = {}


def publication(e, job: int, n: int) -> _Publication:
    key = (id(e), job, n)
    if key not in _PUBLICATIONS:
        _PUBLICATIONS[key] = _Publication(e, job, n)
    return _PUBLICATIONS[key]


def out_segment(e, job: int, n: int, workers: int):
    widest = max(c1 - c0 for c0, c1 in worker_slices(n, workers))
    return e.comm.segment(f"qr_rows{job}:{n}:{workers}", max(1, widest) * n)


def prepare(e, jobs_sizes: List[int]) -> None:
    """Create (collectively) every segment and workspace the factorisations of these sizes need."""
    count = len(jobs_sizes)
    for job, n in enumerate(jobs_sizes):
        leader, workers = group_of(job, count, e.world)
        if not workers:
            continue
        pub = publication(e, job, n)
        out_segment(e, job, n, len(workers))
        if e.rank == leader:
            qr_driver._workspace(n, e.device, 0)
        elif e.rank in workers:
            c0, c1 = worker_slices(n, len(workers))[workers.index(e.rank)]
            if c1 > c0:
                _worker_buffers(e, job, n, c1 - c0)
                pub.addresses(leader)


def _worker_buffers(e, job: int, n: int, width: int) -> _Worker:
    key = (id(e), job, n, width)
    if key not in _WORKERS:
        _WORKERS[key] = _Worker(e, n, width)
    return _WORKERS[key]


def _run_worker(e, pub: _Publication, leader: int, c0: int, c1: int, out_rows: Tensor) -> None:
    n, width = pub.n, c1 - c0
    buffers = _worker_buffers(e, pub.job, n, width)
    main = torch.cuda.current_stream(e.device)
    status = k.status_word(e.device).data_ptr()
    addresses = pub.addresses(leader).data_ptr()
    ldn = pub.V.ld
    flag_address = pub.flags.peer_ptrs[leader] + 4 * pub.job
    _C.identity_planes(buffers.qt.hi.data_ptr(), buffers.qt.lo.data_ptr(), buffers.qt.ld, n, width, k._stream(), c0)
    k._count("identity_planes_kernel")
    start = torch.cuda.Event()
    start.record(main)
    buffers.pull_stream.wait_event(start)
    panels = list(range(0, n, PANEL))
    for p, j0 in enumerate(panels):
        slot = p % 2
        bw, r = min(PANEL, n - j0), n - j0
        if not e.comm.use_device_barrier:
            token = torch.zeros(1, dtype=torch.int64)
            dist.recv(token, src=leader, group=e.comm.control)
            if int(token) != pub.base + p + 1:
                raise RuntimeError(f"QR worker expected announcement {pub.base + p + 1}, got {int(token)}")
        with torch.cuda.stream(buffers.pull_stream):
            if p >= 2:
                buffers.pull_stream.wait_event(buffers.consumed[slot])
            if e.comm.use_device_barrier:
                _C.wait_flag(flag_address, pub.flag_value(p), status, float(e.comm.barrier_timeout_s), k._stream())
                k._count("wait_flag_kernel")
            v, z = buffers.v[slot], buffers.z[slot]
            _copy_from(addresses, ldn, n, j0, j0, v.hi, r, bw)
            _copy_from(addresses + 8, ldn, n, j0, j0, v.lo, r, bw)
            _copy_from(addresses + 8 * (2 + 2 * p), PANEL, n, 0, 0, z.hi, bw, r)
            _copy_from(addresses + 8 * (3 + 2 * p), PANEL, n, 0, 0, z.lo, bw, r)
            buffers.landed[slot].record(buffers.pull_stream)
        main.wait_event(buffers.landed[slot])
        block = buffers.qt.sub(j0, 0, r, width)
        w = buffers.w.sub(0, 0, bw, width)
        qr_driver._skinny_product(buffers.scratch, buffers.v[slot].sub(0, 0, r, bw), block, w)      # W = V^T Q^T
        k.gemm(buffers.z[slot].sub(0, 0, bw, r), w, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0)
        buffers.consumed[slot].record(main)
    # planes column c of Q^T is row c0 + c of Q: write the slice as contiguous rows
    _C.planes_sum(buffers.qt.hi.data_ptr(), buffers.qt.lo.data_ptr(), buffers.qt.ld, out_rows.data_ptr(), n, n, width,
                  k._stream())
    k._count("planes_sum_kernel")


def qr_jobs(e, jobs, stage_and_gather) -> bool:
    """Factor ``jobs`` = ``[(packed matrix, packed Q, size, column_order), ...]`` concurrently, every job on its
    own group of ranks.  ``stage_and_gather(index, planes)`` fills ``planes`` on the calling (leader) rank with
    the column-permuted dense input of job ``index`` (all inputs are staged and a barrier has passed).  Returns
    ``False`` without doing anything when the groups have no workers (the caller then uses the leader-only path).
    """
    from ..ops.basis import count_qr_call

    count = len(jobs)
    groups = [group_of(index, count, e.world) for index in range(count)]
    if any(not workers for _, workers in groups):
        return False
    epoch = e.comm.qr_epoch = getattr(e.comm, "qr_epoch", 0) + 1     # one counter per communicator: it owns the flags
    outs = []
    for index, (matrix, output, n, order) in enumerate(jobs):
        leader, workers = groups[index]
        pub = publication(e, index, n)
        pub.base = epoch * 65536
        slices = worker_slices(n, len(workers))
        pub.workers = [rank for rank, (c0, c1) in zip(workers, slices) if c1 > c0]
        segment = out_segment(e, index, n, len(workers))
        outs.append((segment, workers, slices))
        if e.rank == leader:
            ws = qr_driver._workspace(n, e.device, 0)     # a rank leads at most one of the concurrent jobs
            stage_and_gather(index, ws["C"])
            for _ in qr_driver._factorisation_steps(None, None, None, 0, publisher=pub, size=n, device=e.device):
                pass
        elif e.rank in pub.workers:
            c0, c1 = slices[workers.index(e.rank)]
            _run_worker(e, pub, leader, c0, c1, segment.local)
        count_qr_call()
    e.comm.barrier()
    # every rank pulls the rows of Q it owns, slice by slice, from the workers
    for (matrix, output, n, order), (segment, workers, slices) in zip(jobs, outs):
        lr, lc = e.rows_of(n), e.cols_of(n)
        if not (lr and lc):
            continue
        mine = owned_indices(n, e.nb, e.pr, e.Pr)          # global rows of my local rows, increasing
        for worker, (c0, c1) in zip(workers, slices):
            if c1 <= c0:
                continue
            l0 = int(torch.searchsorted(mine, c0))
            l1 = int(torch.searchsorted(mine, c1))
            if l1 <= l0:
                continue
            table = e.leader_table(segment, worker)
            target = output[l0:l1, :lc]
            d_j = target.stride(1) if target.shape[1] > 1 else max(1, output.shape[0])
            _C.dist_gather(table.data_ptr(), 1, c1 - c0, n, 1, 1, 1, 1, 1,
                           e.pr, e.Pr, e.nb, -c0, 0, e.pc, e.Pc, e.nb, 0, 0, 0, 0, l0, 0,
                           target.data_ptr(), 0, 1, d_j, l1 - l0, lc, k._stream())
            k._count("dist_gather_kernel")
        k.mark_written(output)
    e.comm.barrier()
    return True

"""Reference arm of ``bench.py``: the UNMODIFIED reference package, installed under
``baseline/_ref``, driven through its own public API (``soap_tp.soap_step``).

The reference reaches its distributed GEMM/QR through an injectable binding object
(``slate_binding=``; ``src/soap_tp/ops/factorizations.py:18-30,114``) because its real bindings need
SLATE/ELPA/MPI, whose sources are not vendored in the checkout and cannot be fetched or rebuilt
offline.  The harness therefore injects a library stand-in that implements the six binding entry
points with nothing but ``torch.distributed`` collectives, cuBLAS (``torch.mm``) and cuSOLVER
(``torch.linalg.qr``), and selects ``basis_implementation="eigh"`` (``torch.linalg.eigh`` on rank 0).
Everything else -- redistribution, Gram updates, permutations, Adam, the step logic -- is the
reference's own stock Python.  None of this repository's kernels, engine or ops is imported here.
"""
from __future__ import annotations

import sys
from pathlib import Path

import torch
import torch.distributed as dist

REF_ROOT = Path(__file__).resolve().parent / "_ref"


class _Raw:
    def __init__(self, ptr: int, shape) -> None:
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (ptr, False), "version": 2}


class LibraryBinding:
    """``slate_bindings`` look-alike built from NCCL + cuBLAS + cuSOLVER (library baseline)."""

    def __init__(self, device: torch.device, block_cyclic_indices) -> None:
        self.device = device
        self._indices = block_cyclic_indices
        self.kernel_launch_estimate = 0

    def compiled_gpu_backend(self) -> str:
        return "cuda"

    def mpi_world_rank_and_size(self):
        return dist.get_rank(), dist.get_world_size()

    def _index(self, n, nb, p, P):
        return torch.tensor(self._indices(n, nb, p, P), dtype=torch.long, device=self.device)

    def _local(self, ptr, ld, rows, cols):
        flat = torch.as_tensor(_Raw(ptr, (max(1, cols), ld)), device=self.device)
        return flat.T[:rows, :cols]

    def _gather(self, ptr, ld, shape, nb, Pr, Pc):
        rank = dist.get_rank()
        pr, pc = rank // Pc, rank % Pc
        ri, ci = self._index(shape[0], nb, pr, Pr), self._index(shape[1], nb, pc, Pc)
        local = self._local(ptr, ld, len(ri), len(ci))
        full = torch.zeros(shape, dtype=torch.float32, device=self.device)
        if len(ri) and len(ci):
            full[ri[:, None], ci] = local
        if dist.get_world_size() > 1:
            dist.all_reduce(full)
        return full, local, ri, ci

    def _rotation(self, ql, x, qr, rows, cols, ldql, ldx, ldqr, nb, Pr, Pc, forward):
        QL, *_ = self._gather(ql, ldql, (rows, rows), nb, Pr, Pc)
        QR, *_ = self._gather(qr, ldqr, (cols, cols), nb, Pr, Pc)
        X, local, ri, ci = self._gather(x, ldx, (rows, cols), nb, Pr, Pc)
        Y = torch.mm(torch.mm(QL.T, X), QR) if forward else torch.mm(torch.mm(QL, X), QR.T)
        if len(ri) and len(ci):
            local.copy_(Y[ri[:, None], ci])

    def slate_forward_rotation_float(self, *args):
        self._rotation(*args, True)

    def slate_backward_rotation_float(self, *args):
        self._rotation(*args, False)

    def slate_symmetric_multiply_float(self, a, q, w, n, lda, nb, Pr, Pc):
        A, *_ = self._gather(a, lda, (n, n), nb, Pr, Pc)
        Q, *_ = self._gather(q, lda, (n, n), nb, Pr, Pc)
        _, local, ri, ci = self._gather(w, lda, (n, n), nb, Pr, Pc)
        if len(ri) and len(ci):
            local.copy_(torch.mm(A, Q)[ri[:, None], ci])

    def slate_qr_float(self, m, q, n, ldm, ldq, nb, Pr, Pc):
        M, *_ = self._gather(m, ldm, (n, n), nb, Pr, Pc)
        _, local, ri, ci = self._gather(q, ldq, (n, n), nb, Pr, Pc)
        factor, _ = torch.linalg.qr(M)
        if len(ri) and len(ci):
            local.copy_(factor[ri[:, None], ci])


def make_step(*, size: int, block_size: int, shard_dim: int, grid, refresh_interval: int, device: torch.device):
    """Return ``(step_fn(gradient) -> update, launch_counter, basis_name)`` for ``bench.py``."""
    sys.path.insert(0, str(REF_ROOT))
    import soap_tp  # the installed reference
    from soap_tp.ops._utils import block_cyclic_indices

    torch.backends.cuda.matmul.allow_tf32 = False
    binding = LibraryBinding(device, block_cyclic_indices)
    state: dict = {}

    def step_fn(gradient):
        return soap_tp.soap_step(
            gradient, state, global_shape=(size, size), shard_dim=shard_dim, block_size=block_size,
            process_grid_shape=grid, basis_refresh_interval=refresh_interval, basis_implementation="eigh",
            slate_binding=binding,
        )

    return step_fn, (lambda: 0), "eigh"

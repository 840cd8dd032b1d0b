"""Pointer-level entry points with the calling convention of the reference's native modules.

The reference reaches its distributed GEMM/QR and its eigensolver through two pybind11 modules whose functions
take raw addresses, leading dimensions and grid parameters (``src/soap_tp/csrc/slate_bindings.cpp:317-389``,
``src/soap_tp/csrc/elpa_bindings.cpp:200-236``), and every op accepts a replacement object for them
(``slate_binding=``, ``elpa_binding=``; ``src/soap_tp/ops/factorizations.py:18-30``) -- its own tests wrap the
module in a proxy that counts QR calls (``tests/unit/test_soap.py:402-412``).  This module keeps that seam usable:

* :func:`slate_bindings_for` / :func:`elpa_bindings_for` return objects with the reference's entry points
  (``slate_forward_rotation_float``, ``slate_backward_rotation_float``, ``slate_symmetric_multiply_float``,
  ``slate_qr_float``, ``elpa_eigenvectors_2d_block_cyclic_double``, ``compiled_gpu_backend``,
  ``mpi_world_rank_and_size``) implemented by this package's own ops on the buffers behind the pointers;
* an object handed to an op as ``slate_binding=`` / ``elpa_binding=`` is CALLED for that op's heavy step, with the
  reference's argument order, instead of the built-in path -- so proxies, fakes and third-party bindings work.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch
import torch.distributed as dist

from .layout import local_2d_block_cyclic_shape


def _view(pointer: int, ld: int, rows: int, cols: int, device: torch.device, dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Column-major ``rows x cols`` tensor (pitch ``ld``) over raw memory at ``pointer``."""
    itemsize = 8 if dtype == torch.float64 else 4
    numel = max(1, ld) * max(1, cols)
    if device.type == "cuda":
        typestr = "<f8" if dtype == torch.float64 else "<f4"

        class _Raw:
            __cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (pointer, False), "version": 2}

        flat = torch.as_tensor(_Raw(), device=device)
    else:
        ctype = ctypes.c_double if dtype == torch.float64 else ctypes.c_float
        flat = torch.frombuffer((ctype * numel).from_address(pointer), dtype=dtype)
    del itemsize
    return flat.view(max(1, cols), max(1, ld)).T[: max(1, rows), : max(1, cols)]


class _Bindings:
    def __init__(self, device) -> None:
        self.device = torch.device(device)

    def compiled_gpu_backend(self) -> str:
        return "cuda" if self.device.type == "cuda" else "none"

    def mpi_world_rank_and_size(self) -> Tuple[int, int]:
        return dist.get_rank(), dist.get_world_size()

    def _local(self, shape, nb, Pr, Pc):
        return local_2d_block_cyclic_shape(shape, nb, (Pr, Pc), dist.get_rank())


class SlateBindings(_Bindings):
    """The four SLATE entry points of the reference, served by this package's rotation, product and QR ops."""

    def _rotation(self, ql, x, qr, rows, cols, ldql, ldx, ldqr, nb, Pr, Pc, direction):
        from .ops import rotate_2d_block_cyclic_

        lr, lc = self._local((rows, cols), nb, Pr, Pc)
        llr, llc = self._local((rows, rows), nb, Pr, Pc)
        rlr, rlc = self._local((cols, cols), nb, Pr, Pc)
        rotate_2d_block_cyclic_(_view(x, ldx, lr, lc, self.device), _view(ql, ldql, llr, llc, self.device),
                                _view(qr, ldqr, rlr, rlc, self.device), (rows, cols), nb, (Pr, Pc), direction=direction)

    def slate_forward_rotation_float(self, ql, x, qr, rows, cols, ldql, ldx, ldqr, nb, Pr, Pc):
        self._rotation(ql, x, qr, rows, cols, ldql, ldx, ldqr, nb, Pr, Pc, "forward")

    def slate_backward_rotation_float(self, ql, x, qr, rows, cols, ldql, ldx, ldqr, nb, Pr, Pc):
        self._rotation(ql, x, qr, rows, cols, ldql, ldx, ldqr, nb, Pr, Pc, "backward")

    def slate_symmetric_multiply_float(self, a, q, w, n, lda, nb, Pr, Pc):
        from .ops import estimated_eigenvalue_order_2d_block_cyclic_

        lr, lc = self._local((n, n), nb, Pr, Pc)
        views = [_view(p, lda, lr, lc, self.device) for p in (a, q, w)]
        estimated_eigenvalue_order_2d_block_cyclic_(*views, n, nb, (Pr, Pc))      # leaves P Q in `w`

    def slate_qr_float(self, m, q, n, ldm, ldq, nb, Pr, Pc):
        from .ops import qr_2d_block_cyclic_

        lr, lc = self._local((n, n), nb, Pr, Pc)
        qr_2d_block_cyclic_(_view(m, ldm, lr, lc, self.device), _view(q, ldq, lr, lc, self.device), n, nb, (Pr, Pc))


class ElpaBindings(_Bindings):
    """The ELPA entry point of the reference (fp64 buffers, ascending eigenvalues), served by this package's
    eigensolvers: the fp64 input is rounded to fp32, solved, and the result widened again."""

    def elpa_eigenvectors_2d_block_cyclic_double(self, a, eigenvalues, q, n, local_rows, local_cols, nb, Pr, Pc, gpu_id):
        from .layout import empty_2d_block_cyclic_like_shape
        from .ops import initialize_basis_2d_block_cyclic_

        ld = max(1, local_rows)
        A64 = _view(a, ld, local_rows, local_cols, self.device, torch.float64)
        Q64 = _view(q, ld, local_rows, local_cols, self.device, torch.float64)
        values64 = _view(eigenvalues, n, n, 1, self.device, torch.float64)[:, 0]
        make = lambda: empty_2d_block_cyclic_like_shape(local_rows, local_cols, device=self.device)
        P, Q, work = make(), make(), make()
        P.copy_(A64)
        values = torch.empty(n, dtype=torch.float32, device=self.device)
        initialize_basis_2d_block_cyclic_(P, Q, work, values, n, nb, (Pr, Pc), implementation="householder")
        # descending -> ascending, as ELPA returns them
        order = torch.arange(n - 1, -1, -1, device=self.device)
        from .ops import permute_2d_block_cyclic_

        permute_2d_block_cyclic_(Q, (n, n), torch.arange(n, device=self.device), order, nb, (Pr, Pc))
        Q64.copy_(Q)
        values64.copy_(values.flip(0))


def slate_bindings_for(device) -> SlateBindings:
    return SlateBindings(device)


def elpa_bindings_for(device) -> ElpaBindings:
    return ElpaBindings(device)


slate_bindings = SlateBindings("cpu")
elpa_bindings = ElpaBindings("cpu")

__all__ = ["ElpaBindings", "SlateBindings", "elpa_bindings", "elpa_bindings_for", "slate_bindings", "slate_bindings_for"]

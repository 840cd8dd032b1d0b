"""Symmetric eigensolver by Householder tridiagonalisation on one GPU.

``symmetric_eigenbasis(P, Q, work, values)`` has the contract of :mod:`.jacobi` (orthonormal eigenvectors in
``Q``, eigenvalues in ``values``, both descending) and is what the names ``"householder"``, ``"elpa"`` and
``"eigh"`` select on CUDA tensors.  It is the method behind the reference's default basis initialisation
(ELPA's one-stage solver, ``src/soap_tp/csrc/elpa_bindings.cpp:61-196``), built from this package's kernels:

    reduce     A = Q_h T Q_h^T, 32 reflectors per launch of the cooperative panel kernel (``csrc/tridiag.cu``),
               deferred rank-64 update of the trailing matrix as one 3xTF32 tcgen05 GEMM per panel
    solve      eigenvalues of T by bisection, eigenvectors by twisted factorisation, both in float64
    transform  X = Q_h Z: the panels' block reflectors applied to Z by the products of the QR driver
    polish     one Newton-Schulz step (orthogonality to fp32 rounding) and Rayleigh quotients

Eigenvalues that float64 bisection cannot tell apart (exactly repeated ones: an identity, a matrix with
repeated diagonal blocks) would make the twisted factorisation return the same vector several times.  Such inputs
are detected after the bisection and handed to the Jacobi solver, which has no such restriction.
"""
from __future__ import annotations

from typing import Dict

import torch
from torch import Tensor

from . import jacobi
from . import kernels as k
from . import qr as qr_driver

_C = k._C
TB = _C.TRIDIAG_PANEL
_WORKSPACES: Dict[tuple, dict] = {}
MIN_SIZE = 3            # below this the matrix is handed to the Jacobi solver


def _workspace(n: int, device) -> dict:
    key = (n, str(device))
    ws = _WORKSPACES.get(key)
    if ws is None:
        panels = -(-(n - 1) // TB)
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        f32 = dict(dtype=torch.float32, device=device)
        f64 = dict(dtype=torch.float64, device=device)
        ws = dict(
            vw=torch.zeros(n * 2 * TB, **f32), x=torch.zeros(n, **f32), y=torch.zeros(n, **f32),
            partial=torch.zeros(sms * (2 * TB + 8), **f32), d=torch.zeros(n, **f64), e=torch.zeros(max(1, n - 1), **f64),
            tau=torch.zeros(n, **f32), barrier=torch.zeros(4, dtype=torch.int32, device=device),
            za=k.Planes.empty(2 * TB, n, device), zb=k.Planes.empty(2 * TB, n, device),
            V=k.Planes.empty(n, n, device),
            Vt=[k.Planes.empty(TB, n, device) for _ in range(panels)],
            T=[k.Planes.empty(TB, TB, device) for _ in range(panels)],
            Tt=[k.Planes.empty(TB, TB, device) for _ in range(panels)],
            lam=torch.zeros(n, **f64),
            scratch64=torch.empty(3 * n * n, **f64),
            z=torch.empty((n, n), **f32),
            Z=k.Planes.empty(n, n, device),
            zt=k.Planes.empty(TB, n, device), w=k.Planes.empty(TB, n, device),
            partials=torch.empty(16 * 128 * n, **f32),
        )
        _WORKSPACES[key] = ws
    return ws


def release_workspaces() -> None:
    _WORKSPACES.clear()


def tridiagonalise(A: Tensor, ws: dict) -> None:
    """Reduce the symmetric ``A`` (both triangles, overwritten) to ``ws['d'], ws['e']``; reflectors into ``ws``."""
    n = A.shape[0]
    device = A.device
    status = k.status_word(device).data_ptr()
    lda = A.stride(1) if n > 1 else 1
    V = ws["V"]
    for p, j0 in enumerate(range(0, n - 1, TB)):
        nb = min(TB, n - 1 - j0)
        # V of this panel: rows j0 .. n - 1 (row j0 holds zeros) at element (j0, j0) of the n x n store
        v_hi = V.hi[j0:, j0:]
        v_lo = V.lo[j0:, j0:]
        vt, T, Tt = ws["Vt"][p], ws["T"][p], ws["Tt"][p]
        last = int(j0 + nb >= n - 1)
        _C.sytrd_panel(A.data_ptr(), lda, n, j0, nb, ws["vw"].data_ptr(), ws["x"].data_ptr(), ws["y"].data_ptr(),
                       ws["partial"].data_ptr(), ws["d"].data_ptr(), ws["e"].data_ptr(), ws["tau"].data_ptr(),
                       ws["za"].hi.data_ptr(), ws["za"].lo.data_ptr(), ws["zb"].hi.data_ptr(), ws["zb"].lo.data_ptr(),
                       v_hi.data_ptr(), v_lo.data_ptr(), V.ld, vt.hi.data_ptr(), vt.lo.data_ptr(), vt.ld,
                       T.hi.data_ptr(), T.lo.data_ptr(), Tt.hi.data_ptr(), Tt.lo.data_ptr(), T.ld,
                       ws["barrier"].data_ptr(), status, last, k._stream())
        k._count("sytrd_panel_kernel")
        rest = n - (j0 + nb)
        if rest > 0 and not last:
            za, zb = ws["za"].sub(0, 0, 2 * TB, rest), ws["zb"].sub(0, 0, 2 * TB, rest)
            k.gemm(za, zb, out=A[j0 + nb:, j0 + nb:], alpha=-1.0, beta=1.0, symmetric=True)    # A -= V W^T + W V^T


def symmetric_eigenbasis(P: Tensor, Q: Tensor, work: Tensor, values: Tensor) -> Tensor:
    n = P.shape[0]
    device = P.device
    if n < MIN_SIZE:
        return jacobi.symmetric_eigenbasis(P, Q, work, values)
    ws = _workspace(n, device)
    A = work[:n, :n]
    k.gather2d(P, A, None, None)
    tridiagonalise(A, ws)
    d, e, lam = ws["d"], ws["e"], ws["lam"]
    # Gershgorin interval and the smallest pivot the recurrences accept (host scalars: initialisation path)
    off = torch.zeros(n + 1, dtype=torch.float64, device=device)
    off[1:n] = e[: n - 1].abs()
    radius = off[:-1] + off[1:]
    low, high = float((d - radius).min()), float((d + radius).max())
    norm = max(abs(low), abs(high), 1e-300)
    margin = 1e-12 * norm + 1e-300
    pivmin = max(1e-290, 2.2e-16 * 2.2e-16 * norm)
    stream = k._stream()
    _C.tridiagonal_bisect(d.data_ptr(), e.data_ptr(), n, low - margin, high + margin, pivmin, lam.data_ptr(), stream)
    k._count("bisect_kernel")
    smallest_gap = float((lam[1:] - lam[:-1]).min()) if n > 1 else norm
    if not smallest_gap > 4.0 * 2.2e-16 * norm:
        # eigenvalues that float64 cannot separate: the twisted factorisation would repeat vectors
        symmetric_eigenbasis.fallbacks = getattr(symmetric_eigenbasis, "fallbacks", 0) + 1
        return jacobi.symmetric_eigenbasis(P, Q, work, values)
    scratch = ws["scratch64"]
    nn = n * n
    _C.tridiagonal_vectors(d.data_ptr(), e.data_ptr(), n, lam.data_ptr(), pivmin, scratch.data_ptr(),
                           scratch[nn:].data_ptr(), scratch[2 * nn:].data_ptr(), ws["z"].data_ptr(), stream)
    k._count("twisted_kernel")
    Z = ws["Z"]
    k.split_planes(ws["z"], out=Z)                    # z is row-major n x n: element (i, k) = entry i of vector k
    back_transform(Z, ws, n)
    X = work[:n, :n]                                   # the reduced matrix is no longer needed
    _C.planes_sum(Z.hi.data_ptr(), Z.lo.data_ptr(), Z.ld, ws["z"].data_ptr(), n, n, n, stream)     # z[c][i] = X[i, c]
    k._count("planes_sum_kernel")
    k.gather2d(ws["z"].T, X, None, None)
    if not bool(torch.isfinite(X).all()):
        symmetric_eigenbasis.fallbacks = getattr(symmetric_eigenbasis, "fallbacks", 0) + 1
        return jacobi.symmetric_eigenbasis(P, Q, work, values)
    jacobi._polish(X, Q)
    product = torch.empty((n, n), dtype=torch.float32, device=device).T
    k.gemm(k.split_planes(P), k.split_planes(Q), out=product)
    k.column_dot(Q, product, n, n, out=values)
    k.mark_written(Q, values)
    return Q


def back_transform(Z: k.Planes, ws: dict, n: int) -> None:
    """``Z <- H_0 H_1 ... H_{n-2} Z``, panel by panel from the last one (each panel's product is ``I - V T V^T``)."""
    V = ws["V"]
    scratch = {"partials": ws["partials"]}
    starts = list(range(0, n - 1, TB))
    for p in reversed(range(len(starts))):
        j0 = starts[p]
        nb = min(TB, n - 1 - j0)
        r0, r = j0, n - j0       # from row j0 (a zero row of V), so that the planes start on a 16-byte boundary
        vt, T = ws["Vt"][p], ws["T"][p]
        t_op = k.Planes(T.hi, T.lo, nb, nb, T.ld)
        zt = ws["zt"].sub(0, 0, nb, r)
        k.gemm(t_op, vt.sub(0, 0, nb, r), mode=k.EPI_SPLIT, out_planes=zt, force_narrow=True)      # T^T V^T
        v = V.sub(r0, j0, r, nb)
        block = Z.sub(r0, 0, r, n)
        w = ws["w"].sub(0, 0, nb, n)
        qr_driver._skinny_product(scratch, v, block, w)                                          # W = V^T Z
        k.gemm(zt, w, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0)                   # Z -= V T (V^T Z)

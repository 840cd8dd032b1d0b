"""Two-sided block-Jacobi eigensolver for symmetric matrices on one GPU.

``symmetric_eigenbasis(P, Q, work, values)`` fills ``Q`` with orthonormal eigenvectors of the
symmetric matrix ``P`` and ``values`` with its eigenvalues, both in DESCENDING eigenvalue order --
the contract of the reference's basis initialisation, which calls ELPA in fp64
(``src/soap_tp/csrc/elpa_bindings.cpp:61-196``) or ``torch.linalg.eigh`` on rank 0
(``src/soap_tp/ops/factorizations.py:421-470``).

Method: drive ``M = V^T P V`` to diagonal form (``M = P``, ``V = I`` at the start) by rotating pairs of
64-wide index blocks.  One round treats ``n / 128`` disjoint pairs at once:

    solve    the 128 x 128 diagonal block of every pair, M_pp = U_p diag U_p^T     jacobi_small_kernel
    columns  [M; V][:, pair p] <- [M; V][:, pair p] U_p                            batched 3xTF32 tcgen05 GEMM
    rows     M[pair p, :] <- U_p^T M[pair p, :]                                    the same GEMM on the transpose

Both GEMMs are the pair-update launch of ``csrc/gemm_tf32x3.cu``: its epilogue writes the result as
operand planes in both orientations and moves every 64-wide half pair to its seat of the next
round (round-robin tournament), so pairs are always 128 adjacent indices, the transposed output of
the column update is directly the input of the row update, and no permutation or transpose pass
exists.  A sweep is ``n / 64 - 1`` rounds; sweeps repeat until the largest off-diagonal entry met
during a sweep is below ``tolerance`` times the largest diagonal entry.  The accumulated ``V`` is
polished with one Newton-Schulz step (two GEMMs) so that ``Q^T Q = I`` to fp32 rounding.

Sizes that are not multiples of 128 are embedded in the next multiple with distinct negative values
on the padded diagonal: the padding never couples to the true block and sorts to the end.
"""
from __future__ import annotations

from typing import Dict

import torch
from torch import Tensor

from . import kernels as k

_C = k._C
PAIR = 128
HALF = 64
_WORKSPACES: Dict[tuple, dict] = {}


def _seat_map(blocks: int) -> torch.Tensor:
    """Round-robin rotation of the 64-column blocks: seat ``s`` of this round -> seat of the next round.

    Pair ``i`` sits in seats ``(2i, 2i + 1)`` (top, bottom).  Seat 0 keeps its block; the others
    move one place around the circle top_1 -> top_2 -> ... -> top_last -> bottom_last -> ... ->
    bottom_0 -> top_1, which meets every pair of blocks once in ``blocks - 1`` rounds.
    """
    pairs = blocks // 2
    nxt = list(range(blocks))
    if pairs == 1:
        return torch.tensor(nxt, dtype=torch.int32)
    for i in range(1, pairs - 1):
        nxt[2 * i] = 2 * (i + 1)              # top_i -> top_{i+1}
    nxt[2 * (pairs - 1)] = 2 * (pairs - 1) + 1  # top_last -> bottom_last
    for i in range(1, pairs):
        nxt[2 * i + 1] = 2 * (i - 1) + 1      # bottom_i -> bottom_{i-1}
    nxt[1] = 2                                # bottom_0 -> top_1
    return torch.tensor(nxt, dtype=torch.int32)


def _workspace(size: int, device) -> dict:
    key = (size, str(device))
    ws = _WORKSPACES.get(key)
    if ws is None:
        pairs = size // PAIR
        ws = dict(
            S=[k.Planes.empty(size, 2 * size, device) for _ in range(2)],   # [M; V]: operand rows = matrix rows, K = column
            R=k.Planes.empty(size, size, device),                            # (M J)^T between the two GEMMs of a round
            U=k.Planes.empty(PAIR, PAIR * pairs, device),
            offdiag=torch.zeros(1, dtype=torch.float32, device=device),
            remap=_seat_map(size // HALF).to(device),
        )
        _WORKSPACES[key] = ws
    return ws


def release_workspaces() -> None:
    _WORKSPACES.clear()


def symmetric_eigenbasis(P: Tensor, Q: Tensor, work: Tensor, values: Tensor, *, tolerance: float = 4e-6,
                         max_sweeps: int = 24) -> Tensor:
    n = P.shape[0]
    device = P.device
    size = -(-n // PAIR) * PAIR
    pairs, blocks = size // PAIR, size // HALF
    ws = _workspace(size, device)
    S, R, U = ws["S"], ws["R"], ws["U"]

    padded = P
    if size != n:
        padded = torch.zeros((size, size), dtype=torch.float32, device=device).T
        padded[:n, :n] = P
        shift = 1.0 + 2.0 * float(torch.linalg.matrix_norm(P.float()))
        padded.diagonal()[n:] = -shift * (1.0 + torch.arange(size - n, device=device, dtype=torch.float32) / size)
    scale = float(padded.diagonal().abs().max())
    if scale == 0.0:
        scale = float(padded.abs().max()) or 1.0
    m_part = S[0].sub(0, 0, size, size)
    k.split_planes(padded, transpose=True, out=m_part)        # planes element (K = column, row) = M[row, column]
    v_part = S[0].sub(0, size, size, size)
    _C.identity_planes(v_part.hi.data_ptr(), v_part.lo.data_ptr(), v_part.ld, size, size, k._stream())
    k._count("identity_planes_kernel")

    remap = ws["remap"]
    columns = dict(count=pairs, M=2 * size, N=PAIR, K=PAIR, a_k_step=PAIR, b_row_step=PAIR, remap=remap,
                   out2_planes=R, m_limit=size, o1_row_start=size)
    rows = dict(count=pairs, M=size, N=PAIR, K=PAIR, a_k_step=PAIR, b_row_step=PAIR, remap=remap)
    current = 0
    sweeps_done = 0
    last_offdiag = 1.0
    for sweep in range(max_sweeps):
        ws["offdiag"].zero_()
        # While the matrix is far from diagonal the diagonal blocks need not be diagonalised to working
        # precision: a few inner sweeps give the same outer convergence at a fraction of the cost
        # (a fully dense 128 x 128 block costs 0.4 ms per inner sweep, a converged one 0.2 ms in total).
        inner_sweeps = 2 if (blocks > 2 and last_offdiag > 1e-3) else 10
        for _ in range(max(1, blocks - 1)):
            nxt = current ^ 1
            _C.jacobi_small(S[current].hi.data_ptr(), S[current].lo.data_ptr(), S[current].ld, pairs, U.hi.data_ptr(),
                            U.lo.data_ptr(), U.ld, ws["offdiag"].data_ptr(), scale, inner_sweeps, 1e-7, k._stream())
            k._count("jacobi_small_kernel")
            # [M; V] J: the V part goes to the next arrangement, (M J)^T lands in R
            k.gemm(S[current], U, mode=k.EPI_PAIR_UPDATE, out_planes=S[nxt], force_narrow=True, batch=columns)
            # (J^T M) J from R = (M J)^T: the rotated, re-seated symmetric matrix
            k.gemm(R, U, mode=k.EPI_PAIR_UPDATE, out_planes=S[nxt], force_narrow=True, batch=rows)
            current = nxt
        sweeps_done = sweep + 1
        last_offdiag = float(ws["offdiag"].item())
        if last_offdiag <= tolerance:
            break
    final = S[current].dense()                       # (K = column j) x (rows: M rows then V rows)
    eigen = final[:, :size].diagonal().clone()
    v_cols = final[:, size:]                         # row j = column j of V
    order = torch.argsort(eigen, descending=True, stable=True)[:n]
    selected = torch.empty((n, n), dtype=torch.float32, device=device).T
    k.gather2d(v_cols.T, selected, None, order)      # selected[:, j] = V[:n, order[j]]
    _polish(selected, Q)
    # Eigenvalues as Rayleigh quotients q_j^T P q_j of the polished vectors: the diagonal of the rotated
    # matrix carries the rounding of thousands of similarity updates, the quotient only that of one product.
    product = torch.empty((n, n), dtype=torch.float32, device=device).T
    k.gemm(k.split_planes(P), k.split_planes(Q), out=product)          # P^T Q = P Q
    k.column_dot(Q, product, n, n, out=values)
    k.mark_written(Q, values)
    symmetric_eigenbasis.last_sweeps = sweeps_done
    return Q


def _polish(V: Tensor, Q: Tensor) -> None:
    """One Newton-Schulz step, ``Q = V (1.5 I - 0.5 V^T V)``: removes the 1e-5-level drift from
    orthogonality that thousands of fp32 rotations leave behind (the correction is second order for
    the eigen-residual)."""
    n = V.shape[0]
    planes = k.split_planes(V)
    gram = torch.empty((n, n), dtype=torch.float32, device=V.device).T
    k.gemm(planes, planes, out=gram, alpha=-0.5, symmetric=True)
    gram.diagonal().add_(1.5)
    k.gemm(k.split_planes(V, transpose=True), k.split_planes(gram), out=Q)

"""Single-process dense SOAP for one 2-D parameter: the trajectory oracle.

This is an independent restatement of the SOAP recipe (Adam run in the eigenbasis of Shampoo's
``L = EMA(G G^T)`` and ``R = EMA(G^T G)``) in the formulation of the original optimizer, which
the reference vendors as its oracle (``tests/reference/soap.py``): the first call only seeds
``L``, ``R`` and their eigenbases and returns a zero update (``tests/reference/soap.py:185-215``);
the first moment is kept in PARAMETER space and projected every step
(``tests/reference/soap.py:261-292``) whereas the tensor-parallel implementation keeps it in
rotated space and transports it at refresh time -- equal in exact arithmetic, so agreement
between the two is a real test; the refresh is one power iteration followed by QR with the
second moment permuted by the estimated eigenvalue order (``tests/reference/soap.py:505-562``).

``dtype=torch.float64`` gives a high-precision trajectory for noise-floor studies.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
from torch import Tensor


class DenseSOAP:
    def __init__(
        self,
        shape: Tuple[int, int],
        *,
        beta1: float = 0.95,
        beta2: float = 0.95,
        preconditioner_beta: float = 0.95,
        eps: float = 1e-8,
        basis_refresh_interval: int = 10,
        dtype: torch.dtype = torch.float32,
        device: str | torch.device = "cpu",
    ) -> None:
        self.shape = tuple(shape)
        self.beta1, self.beta2 = beta1, beta2
        self.preconditioner_beta = preconditioner_beta
        self.eps = eps
        self.interval = basis_refresh_interval
        self.dtype, self.device = dtype, torch.device(device)
        rows, columns = self.shape
        zeros = lambda *s: torch.zeros(*s, dtype=dtype, device=self.device)
        self.L, self.R = zeros(rows, rows), zeros(columns, columns)
        self.QL: Optional[Tensor] = None
        self.QR: Optional[Tensor] = None
        self.exp_avg = zeros(rows, columns)       # parameter space
        self.exp_avg_sq = zeros(rows, columns)    # rotated space
        self.step_count = 0
        self.profile = False   # emit SOAP_PROFILE taps with impl "reference" (needs SOAP_PROFILE=1)
        self.qr_calls = 0
        self.last_orders: Optional[Tuple[Tensor, Tensor]] = None

    @staticmethod
    def eigenbasis_descending(P: Tensor) -> Tuple[Tensor, Tensor]:
        values, vectors = torch.linalg.eigh(P)
        return values.flip(0), vectors.flip(1)

    def _update_grams(self, G: Tensor) -> None:
        self.L.lerp_(G @ G.T, 1.0 - self.preconditioner_beta)
        self.R.lerp_(G.T @ G, 1.0 - self.preconditioner_beta)

    def _refresh(self) -> None:
        orders = []
        for axis, (P, name) in enumerate(((self.L, "QL"), (self.R, "QR"))):
            Q = getattr(self, name)
            estimates = torch.einsum("ij,ij->j", Q, P @ Q)
            order = torch.argsort(estimates, descending=True, stable=True)
            self.exp_avg_sq = self.exp_avg_sq.index_select(axis, order)
            new_Q, _ = torch.linalg.qr(P @ Q[:, order])
            setattr(self, name, new_Q)
            self.qr_calls += 1
            orders.append(order)
        self.last_orders = (orders[0], orders[1])

    @torch.no_grad()
    def step(self, gradient: Tensor) -> Tensor:
        """Consume one full gradient; return the normalised update (before learning rate)."""
        G = gradient.to(dtype=self.dtype, device=self.device)
        tap = self._tap
        if self.QL is None:
            tap("gradient", 0, G)
            self._update_grams(G)
            tap("left_preconditioner", 0, self.L)
            tap("right_preconditioner", 0, self.R)
            _, self.QL = self.eigenbasis_descending(self.L)
            _, self.QR = self.eigenbasis_descending(self.R)
            tap("left_basis", 0, self.QL)
            tap("right_basis", 0, self.QR)
            tap("returned_update", 0, torch.zeros_like(G))
            return torch.zeros_like(G)
        self.step_count += 1
        t = self.step_count
        tap("gradient", t, G)
        for name, value in (("left_preconditioner", self.L), ("right_preconditioner", self.R),
                            ("left_basis", self.QL), ("right_basis", self.QR)):
            tap(name, t, value)
        rotated = self.QL.T @ G @ self.QR
        tap("projected_gradient", t, rotated)
        self.exp_avg.mul_(self.beta1).add_(G, alpha=1.0 - self.beta1)
        self.exp_avg_sq.mul_(self.beta2).addcmul_(rotated, rotated, value=1.0 - self.beta2)
        denominator = self.exp_avg_sq.sqrt().add_(self.eps)
        rotated_momentum = self.QL.T @ self.exp_avg @ self.QR
        scale = math.sqrt(1.0 - self.beta2**t) / (1.0 - self.beta1**t)
        coordinate_update = rotated_momentum / denominator * scale
        update = self.QL @ coordinate_update @ self.QR.T
        tap("momentum_after_adam", t, rotated_momentum)
        tap("variance_after_adam", t, self.exp_avg_sq)
        tap("coordinate_update", t, coordinate_update)
        tap("returned_update", t, update)
        self._update_grams(G)
        tap("left_preconditioner_after_step", t, self.L)
        tap("right_preconditioner_after_step", t, self.R)
        if t % self.interval == 0:
            self._refresh()
        tap("left_basis_after_step", t, self.QL)
        tap("right_basis_after_step", t, self.QR)
        tap("momentum_after_step", t, self.QL.T @ self.exp_avg @ self.QR)
        tap("variance_after_step", t, self.exp_avg_sq)
        return update

    def _tap(self, stage: str, step: int, tensor: Tensor) -> None:
        if not self.profile:
            return
        from ..profiling import emit_profile_tensor, profile_enabled

        if profile_enabled(step):
            emit_profile_tensor(stage, step, tensor.to(torch.float32), impl="reference")


def relative_l2(actual: Tensor, expected: Tensor) -> float:
    """``||actual - expected|| / ||expected||`` (absolute norm if the expectation is zero)."""
    actual = actual.detach().double().cpu()
    expected = expected.detach().double().cpu()
    denominator = float(expected.norm())
    error = float((actual - expected).norm())
    return error / denominator if denominator > 0 else error


def align_column_signs(Q: Tensor, reference: Tensor) -> Tensor:
    """Flip columns of ``Q`` so that each has a non-negative inner product with ``reference``'s
    (eigenvectors and Householder ``Q`` columns are defined up to sign; the reference's tests
    and its profile diff tool align signs the same way, ``scripts/compare_soap_profiles.py:298-411``)."""
    signs = torch.sign((Q * reference).sum(dim=0))
    signs[signs == 0] = 1
    return Q * signs


__all__ = ["DenseSOAP", "align_column_signs", "relative_l2"]

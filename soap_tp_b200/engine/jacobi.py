"""Symmetric eigensolver of a local column-major matrix (bring-up version: library solver)."""
from __future__ import annotations

import torch
from torch import Tensor


def symmetric_eigenbasis(P: Tensor, Q: Tensor, work: Tensor, values: Tensor) -> Tensor:
    eigenvalues, vectors = torch.linalg.eigh(P)
    values.copy_(eigenvalues.flip(0))
    Q.copy_(vectors.flip(1))
    return Q

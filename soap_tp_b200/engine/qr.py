"""Householder QR of a local column-major matrix (bring-up version: library factorisation)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor


def householder_qr(matrix: Tensor, Q: Tensor, column_order: Optional[Tensor] = None) -> Tensor:
    source = matrix if column_order is None else matrix[:, column_order]
    factor, _ = torch.linalg.qr(source)
    Q.copy_(factor)
    return Q

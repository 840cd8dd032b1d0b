"""Fused Adam update in the rotated (eigenbasis) coordinates.

Same contract as the reference's ``adam_update`` (``src/soap_tp/ops/optimizer.py:12-44``):
``momentum`` and ``variance`` are updated in place and the returned tensor is
``(m / bc1) / (sqrt(v) / sqrt(bc2) + eps)``; it has the strides of ``variance`` so a
column-major packed buffer stays column-major for the rotation that follows.  The
reference issues ten elementwise launches; on CUDA this is one kernel
(``csrc/elementwise.cu``) that streams g, m, v once.
"""
from __future__ import annotations

import math

import torch
from torch import Tensor


def _validate(gradient: Tensor, momentum: Tensor, variance: Tensor, step: int, beta1: float, beta2: float, eps: float) -> None:
    if step < 1:
        raise ValueError(f"step must be positive, got {step}.")
    if not 0.0 <= beta1 < 1.0:
        raise ValueError(f"beta1 must be in [0, 1), got {beta1}.")
    if not 0.0 <= beta2 < 1.0:
        raise ValueError(f"beta2 must be in [0, 1), got {beta2}.")
    if eps <= 0.0:
        raise ValueError(f"eps must be positive, got {eps}.")
    if gradient.shape != momentum.shape or gradient.shape != variance.shape:
        raise ValueError("gradient, momentum, and variance must have identical shapes.")


@torch.no_grad()
def adam_update(
    gradient: Tensor,
    momentum: Tensor,
    variance: Tensor,
    step: int,
    beta1: float = 0.9,
    beta2: float = 0.999,
    eps: float = 1e-8,
) -> Tensor:
    """Update local Adam moments in place and return the bias-corrected update."""
    _validate(gradient, momentum, variance, step, beta1, beta2, eps)
    bias_correction1 = 1.0 - beta1**step
    bias_correction2 = 1.0 - beta2**step
    if momentum.is_cuda:
        from ..engine import kernels

        return kernels.adam_update(
            gradient, momentum, variance, beta1, beta2, eps, bias_correction1, bias_correction2
        )
    momentum.mul_(beta1).add_(gradient, alpha=1.0 - beta1)
    variance.mul_(beta2).addcmul_(gradient, gradient, value=1.0 - beta2)
    denominator = variance.sqrt().div_(math.sqrt(bias_correction2)).add_(eps)
    return denominator.reciprocal_().mul_(momentum).div_(bias_correction1)


__all__ = ["adam_update"]

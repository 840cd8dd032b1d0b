"""One-sided SOAP for a matrix whose tensor-parallel (sharded) dimension is too long to precondition.

Original SOAP skips the preconditioner of a dimension above ``max_precond_dim`` and keeps the identity as that
side's basis (the dense oracle the reference tests against does so: ``tests/reference/soap.py:363-367``); the
reference's ``soap_step`` itself is two-sided only.  For vocabulary-sized weights of a tensor-parallel model
(``[vocab / W, hidden]`` row shards) the long side is the sharded one, which makes the one-sided update local:

    R   <- beta R + (1 - beta) sum_ranks G_r^T G_r       hidden x hidden, replicated (one all-reduce)
    Y_r  = G_r Q_R,  Adam(Y_r) -> U_r,  update_r = U_r Q_R^T         rows of a shard never mix

so every rank runs the single-GPU kernels on its shard and the ranks only meet in the all-reduce of the Gram
matrix; the replicated basis is refreshed redundantly (power iteration + Householder QR) from identical inputs.
Products are carried in transposed form (``Y^T = Q^T G^T``) so that each result is already the K-contiguous
operand of the next one.  CUDA only; ``SoapTP`` uses AdamW for such matrices on CPU.
"""
from __future__ import annotations

import math
from typing import Any, MutableMapping

import torch
import torch.distributed as dist
from torch import Tensor

from . import factor
from . import kernels as k
from . import local


_PLANES: dict = {}       # operand planes of each replicated basis, by the basis buffer's address


def step(gradient: Tensor, state: MutableMapping[str, Any], *, beta: float, beta1: float, beta2: float, eps: float,
         interval: int, implementation: str) -> Tensor:
    """One update for the row shard ``gradient`` (``rows_local x h``); returns the fp32 update of that shape."""
    rows, h = gradient.shape
    device = gradient.device
    g32 = gradient.detach()
    if g32.dtype != torch.float32:
        g32 = g32.float()
    world = dist.get_world_size() if dist.is_initialized() else 1
    gp = k.split_planes(g32, out=local.workspace_planes("os_G", rows, h, device))              # operand G   (K = rows)
    gtp = k.split_planes(g32, transpose=True, out=local.workspace_planes("os_GT", h, rows, device))  # operand G^T (K = h)

    def gram_update() -> None:
        fresh = local.workspace_matrix("os_gram", h, h, device)
        k.gemm(gp, gp, out=fresh, symmetric=True)                      # G_r^T G_r
        if world > 1:
            dist.all_reduce(fresh.T)               # the contiguous view of the column-major buffer (same layout on every rank)
        state["right_preconditioner"].mul_(beta).add_(fresh, alpha=1.0 - beta)

    if "right_basis" not in state:
        state["right_preconditioner"] = torch.zeros((h, h), dtype=torch.float32, device=device).T
        state["right_basis"] = torch.zeros((h, h), dtype=torch.float32, device=device).T
        state["right_work"] = torch.zeros((h, h), dtype=torch.float32, device=device).T
        state["momentum"] = torch.zeros((rows, h), dtype=torch.float32, device=device).T       # stored transposed: h x rows
        state["variance"] = torch.zeros((rows, h), dtype=torch.float32, device=device).T
        gram_update()
        factor.symmetric_eigenbasis(state["right_preconditioner"], state["right_basis"], state["right_work"],
                                    torch.empty(h, dtype=torch.float32, device=device), implementation)
        state["step"] = 0
        return torch.zeros((rows, h), dtype=torch.float32, device=device)

    count = int(state["step"]) + 1
    basis = _PLANES.get(state["right_basis"].data_ptr())
    if basis is None:
        basis = _PLANES[state["right_basis"].data_ptr()] = local.BasisPlanes()
    basis.refresh(state["right_basis"], h)
    bias2 = 1.0 - beta2**count
    adam = dict(beta1=beta1, beta2=beta2, eps=eps / math.sqrt(bias2), bias_correction1=1.0 - beta1**count,
                bias_correction2=bias2)
    ut = local.workspace_planes("os_UT", h, rows, device)
    # Y^T = Q^T G^T with Adam in the epilogue: momentum, variance and U^T are h x rows_local, column-major
    k.gemm(basis.plain, gtp, mode=k.EPI_ADAM, out_planes=ut, momentum=state["momentum"], variance=state["variance"], adam=adam)
    update = torch.empty((rows, h), dtype=torch.float32, device=device)
    k.gemm(basis.transposed, ut, out=update.T)                          # (U Q^T)^T = Q U^T, i.e. the row-major update
    gram_update()
    if count % interval == 0:
        # momentum leaves the old basis, M' = (M Q_old^T) Q_new, in the transposed storage: M'^T = Q_new^T Q_old M^T
        mt = k.split_planes(state["momentum"], out=local.workspace_planes("os_MT", h, rows, device))
        middle = local.workspace_planes("os_mid", h, rows, device)
        k.gemm(basis.transposed, mt, mode=k.EPI_SPLIT, out_planes=middle)                       # Q_old M^T
        order = local.power_iteration_qr(state["right_preconditioner"], state["right_basis"], state["right_work"], h)
        scratch = local.workspace_matrix("os_perm", h, rows, device)
        k.gather2d(state["variance"], scratch, order, None)             # the rotated coordinates are the rows here
        k.gather2d(scratch, state["variance"], None, None)
        basis.refresh(state["right_basis"], h)
        k.gemm(basis.plain, middle, out=state["momentum"])                                     # Q_new^T (Q_old M^T)
    state["step"] = count
    k.poll_status(device)
    return update

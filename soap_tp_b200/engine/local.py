"""Single-GPU (grid (1, 1)) device pipeline.

With one rank the packed block-cyclic buffers ARE the dense column-major matrices, so the whole
step is a chain of this package's kernels on one stream:

    split G (both orientations)                                   split_planes_kernel x2
    T   = X^T Q_L                (planes)                          gemm_tf32x3 / split epilogue
    Y   = T^T Q_R, Adam(Y) -> U  (planes), m, v updated in place   gemm_tf32x3 / Adam epilogue
    T2  = U^T Q_L^T              (planes)                          gemm_tf32x3 / split epilogue
    out = T2^T Q_R^T             (row-major shard)                 gemm_tf32x3 / row-major epilogue
    L   = b L + (1-b) G G^T,  R = b R + (1-b) G^T G                gemm_tf32x3 / EMA epilogue, lower tiles + mirror

Every product is brought to the kernel's single form ``acc = Za^T Zb`` with K-contiguous operands
by keeping each basis in both orientations as hi/lo planes; the planes are rebuilt only when the
basis tensor changes (refresh, initialisation, or a user writing into ``state``).
"""
from __future__ import annotations

import math
import os
import weakref
from collections import OrderedDict
from typing import Any, Dict, MutableMapping, Optional, Tuple

import torch
from torch import Tensor

from ..profiling import GLOBAL_STAGE_TIMER as TIMER
from . import kernels as k
from . import factor


class BasisPlanes:
    """Both orientations of one orthogonal basis as operand planes, tied to a tensor version."""

    def __init__(self) -> None:
        self.key: Optional[tuple] = None
        self.owner = None                           # weak reference to the tensor object the planes were made from
        self.plain: Optional[k.Planes] = None       # operand Q   (depth = rows of Q)
        self.transposed: Optional[k.Planes] = None  # operand Q^T (depth = cols of Q)

    def refresh(self, Q: Tensor, size: int) -> None:
        key = (Q.data_ptr(), Q._version, size)
        # the planes belong to one tensor OBJECT: a new tensor at a recycled address with the same version count
        # (a freshly loaded checkpoint, a test's next case) must not be taken for the old one
        if key == self.key and self.owner is not None and self.owner() is Q:
            return
        view = Q[:size, :size]
        if self.plain is not None and (self.plain.depth != size or self.plain.hi.device != Q.device):
            self.plain = self.transposed = None   # the address was recycled by a tensor of another size
        self.plain = k.split_planes(view, out=self.plain, mixed=k.MIXED_CORRECTIONS)
        self.transposed = k.split_planes(view, transpose=True, out=self.transposed, mixed=k.MIXED_CORRECTIONS)
        self.key = (Q.data_ptr(), Q._version, size)
        self.owner = weakref.ref(Q)


class ParameterContext:
    """Per-parameter device-side caches (basis planes)."""

    def __init__(self) -> None:
        self.left = BasisPlanes()
        self.right = BasisPlanes()
        self.bytes = 0


_CONTEXTS: "OrderedDict[tuple, ParameterContext]" = OrderedDict()
_WORKSPACES: Dict[tuple, Any] = {}


# Operand planes of the eigenbases kept between steps (SOAP_TP_BASIS_CACHE_GB, default 40): 12 bytes per basis element
# (two orientations, value plane + low plane), three times the bases themselves.  Beyond the limit the least recently
# used parameters' planes are dropped and split again on use (most recently used first, see ``context_for``).
BASIS_CACHE_BYTES = int(float(os.environ.get("SOAP_TP_BASIS_CACHE_GB", "40")) * 2**30)


def context_for(state: MutableMapping[str, Any]) -> ParameterContext:
    key = (state["left_basis"].data_ptr(), state["right_basis"].data_ptr(),
           tuple(state["momentum"].shape))
    ctx = _CONTEXTS.get(key)
    if ctx is None:
        ctx = ParameterContext()
        rows, cols = state["momentum"].shape
        ctx.bytes = 12 * (rows * rows + cols * cols)
        _CONTEXTS[key] = ctx
    else:
        _CONTEXTS.move_to_end(key)
    total = sum(c.bytes for c in _CONTEXTS.values())
    if total > BASIS_CACHE_BYTES or len(_CONTEXTS) > 4096:
        # contexts of tensors that no longer exist go first; then the MOST recently used ones: an optimizer walks
        # its parameters in the same order every step, so the oldest contexts are the next to be used
        dead = [other for other, c in _CONTEXTS.items()
                if other != key and c.left.owner is not None and c.left.owner() is None]
        for other in dead + [other for other in reversed(_CONTEXTS) if other != key and other not in dead]:
            if total <= BASIS_CACHE_BYTES and len(_CONTEXTS) <= 4096:
                break
            total -= _CONTEXTS.pop(other).bytes
    return ctx


CLASSIC_TAGS = {"P", "Qtmp"}      # operands of the power iteration, which feeds the QR: always 3xTF32


def workspace_planes(tag: str, depth: int, cols: int, device) -> k.Planes:
    """Scratch operand planes shared by every parameter of the same shape on ``device``.  The operands of the
    optimizer-step products are mixed planes (``kernels.Planes``) unless that is switched off."""
    mixed = k.MIXED_CORRECTIONS and tag not in CLASSIC_TAGS
    key = (tag, depth, cols, str(device), mixed)
    planes = _WORKSPACES.get(key)
    if planes is None:
        planes = k.Planes.empty(depth, cols, device, mixed=mixed)
        _WORKSPACES[key] = planes
    return planes


def workspace_matrix(tag: str, rows: int, cols: int, device) -> Tensor:
    key = ("m", tag, rows, cols, str(device))
    matrix = _WORKSPACES.get(key)
    if matrix is None:
        matrix = torch.empty((max(1, cols), max(1, rows)), dtype=torch.float32, device=device).T
        _WORKSPACES[key] = matrix
    return matrix


def release_workspaces() -> None:
    _WORKSPACES.clear()
    _CONTEXTS.clear()


def _gradient_planes(gradient: Tensor, rows: int, cols: int) -> Tuple[k.Planes, k.Planes]:
    """Planes of G (depth = rows) and of G^T (depth = cols) from the row-major gradient."""
    g32 = gradient.detach()
    if g32.dtype != torch.float32:
        g32 = g32.float()
    device = g32.device
    xp = k.split_planes(g32, out=workspace_planes("X", rows, cols, device))
    gtp = k.split_planes(g32, transpose=True, out=workspace_planes("GT", cols, rows, device))
    return xp, gtp


def rotate_planes(source: k.Planes, first: k.Planes, second: k.Planes, rows: int, cols: int, device, *, tag: str,
                  **final) -> None:
    """``final epilogue( (source^T first)^T second )`` -- two chained GEMMs through scratch planes."""
    middle = workspace_planes(tag, source.cols, first.cols, device)
    k.gemm(source, first, mode=k.EPI_SPLIT, out_planes=middle)
    k.gemm(middle, second, **final)


def gram_updates(xp: k.Planes, gtp: k.Planes, state, beta: float, rows: int, cols: int) -> None:
    k.gemm(gtp, gtp, out=state["left_preconditioner"][:rows, :rows], alpha=1.0 - beta, beta=beta, symmetric=True)
    k.gemm(xp, xp, out=state["right_preconditioner"][:cols, :cols], alpha=1.0 - beta, beta=beta, symmetric=True)


def soap_step(
    gradient: Tensor,
    state: MutableMapping[str, Any],
    *,
    global_shape,
    beta: float,
    beta1: float,
    beta2: float,
    eps: float,
    interval: int,
    implementation: str,
    initializing: bool,
) -> Tensor:
    rows, cols = global_shape
    device = gradient.device
    with TIMER.stage("split_gradient", device):
        xp, gtp = _gradient_planes(gradient.reshape(rows, cols), rows, cols)
    if initializing:
        gram_updates(xp, gtp, state, beta, rows, cols)
        for side, size in (("left", rows), ("right", cols)):
            values = torch.empty(size, dtype=torch.float32, device=device)
            factor.symmetric_eigenbasis(
                state[f"{side}_preconditioner"][:size, :size], state[f"{side}_basis"][:size, :size],
                state[f"{side}_work"][:size, :size], values, implementation,
            )
        prepare_refresh(rows, cols, device)
        state["step"] = 0
        return torch.zeros((rows, cols), dtype=torch.float32, device=device)

    step = int(state["step"]) + 1
    ctx = context_for(state)
    ctx.left.refresh(state["left_basis"], rows)
    ctx.right.refresh(state["right_basis"], cols)
    bias2 = 1.0 - beta2**step
    adam = dict(beta1=beta1, beta2=beta2, eps=eps / math.sqrt(bias2),
                bias_correction1=1.0 - beta1**step, bias_correction2=bias2)
    up = workspace_planes("U", rows, cols, device)
    with TIMER.stage("rotate_forward+adam", device):
        rotate_planes(xp, ctx.left.plain, ctx.right.plain, rows, cols, device, tag="T",
                      mode=k.EPI_ADAM, out_planes=up, momentum=state["momentum"][:rows, :cols],
                      variance=state["variance"][:rows, :cols], adam=adam)
    update = torch.empty((rows, cols), dtype=torch.float32, device=device)
    with TIMER.stage("rotate_backward", device):
        rotate_planes(up, ctx.left.transposed, ctx.right.transposed, rows, cols, device, tag="T",
                      mode=k.EPI_ROW_MAJOR, out=update)
    with TIMER.stage("gram", device):
        gram_updates(xp, gtp, state, beta, rows, cols)
    if step % interval == 0:
        with TIMER.stage("refresh", device):
            refresh(state, global_shape)
    state["step"] = step
    return update


_WARMED: Dict[Any, bool] = {}


def warm_refresh_kernels(device, sizes=()) -> None:
    """Launch every kernel variant a refresh uses once, on a tiny problem.

    CUDA loads a kernel's code the first time it is launched; without this the first refresh of a
    training run pays tens of milliseconds of module loading in the middle of a step.  The eigenvalue-order sort
    sizes its shared memory by length, so it is warmed at the real ``sizes``.
    """
    for size in sizes:
        if not _WARMED.get((str(torch.device(device)), "sort", size)):
            _WARMED[(str(torch.device(device)), "sort", size)] = True
            k.order_by_estimate(torch.rand((size, 2), device=device).T)
    key = str(torch.device(device))
    if _WARMED.get(key):
        return
    _WARMED[key] = True
    n = 384
    generator = torch.Generator(device=device).manual_seed(0)
    matrix = torch.randn(n, n, generator=generator, device=device).T
    out = torch.empty(n, n, device=device).T
    order = torch.randperm(n, generator=generator, device=device)
    factor_jobs = [(matrix.clone(), out, order), (matrix.clone(), torch.empty(n, n, device=device).T, None)]
    from . import qr as qr_driver

    qr_driver.householder_qr_pair(factor_jobs)
    qr_driver.householder_qr(matrix.clone(), out)      # a lone factorisation takes the forward-accumulation path
    estimated_order(matrix, out, torch.empty(n, n, device=device).T, n)
    k.gather2d(matrix, out, order, order)
    qr_driver.release_workspaces_for(n, device)


def prepare_refresh(rows: int, cols: int, device) -> None:
    """Allocate what a refresh needs at initialisation time, so that the first refresh in the middle of
    training launches kernels only."""
    from . import qr as qr_driver

    for size in {rows, cols}:
        workspace_planes("P", size, size, device)
        workspace_planes("Qtmp", size, size, device)
        qr_driver._workspace(size, device, 0)
    if rows == cols:
        qr_driver._workspace(cols, device, 1)     # the second of two concurrent factorisations
    else:
        qr_driver._workspace(rows, device, 0), qr_driver._workspace(cols, device, 1)
    workspace_matrix("perm", rows, cols, device)
    for tag, depth, width in (("X", rows, cols), ("U", rows, cols), ("T", cols, rows)):
        workspace_planes(tag, depth, width, device)
    warm_refresh_kernels(device, sizes={rows, cols})


def rotate(matrix: Tensor, Q_left: Tensor, Q_right: Tensor, global_shape, direction: str) -> Tensor:
    rows, cols = global_shape
    device = matrix.device
    left, right = BasisPlanes(), BasisPlanes()
    left.refresh(Q_left, rows)
    right.refresh(Q_right, cols)
    view = matrix[:rows, :cols]
    source = k.split_planes(view, out=workspace_planes("X", rows, cols, device))
    if direction == "forward":
        rotate_planes(source, left.plain, right.plain, rows, cols, device, tag="T", mode=k.EPI_STORE, out=view)
    else:
        rotate_planes(source, left.transposed, right.transposed, rows, cols, device, tag="T", mode=k.EPI_STORE, out=view)
    return matrix


def estimated_order(P: Tensor, Q: Tensor, work: Tensor, size: int) -> Tensor:
    """``work <- P Q`` (P symmetric, so ``P^T Q``), estimates ``colsum(Q * work)``, stable descending order."""
    device = P.device
    pp = k.split_planes(P[:size, :size], out=workspace_planes("P", size, size, device))
    qp = k.split_planes(Q[:size, :size], out=workspace_planes("Qtmp", size, size, device))
    k.gemm(pp, qp, out=work[:size, :size])
    estimates = k.column_dot(Q, work, size, size)
    return k.order_by_estimate(estimates.view(1, size))


def power_iteration_qr(P: Tensor, Q: Tensor, work: Tensor, size: int) -> Tensor:
    order = estimated_order(P, Q, work, size)
    factor.householder_qr(work[:size, :size], Q[:size, :size], column_order=order)
    return order


def permute(matrix: Tensor, global_shape, row_order: Tensor, column_order: Tensor) -> Tensor:
    rows, cols = global_shape
    scratch = workspace_matrix("perm", rows, cols, matrix.device)
    view = matrix[:rows, :cols]
    k.gather2d(view, scratch, row_order, column_order)
    k.gather2d(scratch, view, None, None)
    return matrix


def refresh(state: MutableMapping[str, Any], global_shape) -> Tuple[Tensor, Tensor]:
    """Power iteration + QR on both sides with momentum transport and variance permutation."""
    rows, cols = global_shape
    momentum, variance = state["momentum"], state["variance"]
    device = momentum.device
    ctx = context_for(state)
    ctx.left.refresh(state["left_basis"], rows)
    ctx.right.refresh(state["right_basis"], cols)
    # momentum out of the old bases: Q_L M Q_R^T, kept as planes for the way back
    with TIMER.stage("refresh.momentum_out", device):
        mp = k.split_planes(momentum[:rows, :cols], out=workspace_planes("X", rows, cols, device))
        parameter_space = workspace_planes("U", rows, cols, device)
        rotate_planes(mp, ctx.left.transposed, ctx.right.transposed, rows, cols, device, tag="T",
                      mode=k.EPI_SPLIT, out_planes=parameter_space)
    with TIMER.stage("refresh.power_iteration", device):
        left_order = estimated_order(state["left_preconditioner"], state["left_basis"], state["left_work"], rows)
        right_order = estimated_order(state["right_preconditioner"], state["right_basis"], state["right_work"], cols)
    with TIMER.stage("refresh.qr", device):
        # the two factorisations are independent: issued on two streams they fill each other's gaps
        if os.environ.get("SOAP_TP_SERIAL_QR", "0") == "1":
            factor.householder_qr(state["left_work"][:rows, :rows], state["left_basis"][:rows, :rows], column_order=left_order)
            factor.householder_qr(state["right_work"][:cols, :cols], state["right_basis"][:cols, :cols], column_order=right_order)
        else:
            factor.householder_qr_pair([
                (state["left_work"][:rows, :rows], state["left_basis"][:rows, :rows], left_order),
                (state["right_work"][:cols, :cols], state["right_basis"][:cols, :cols], right_order)])
    with TIMER.stage("refresh.permute_variance", device):
        permute(variance, global_shape, left_order, right_order)
    with TIMER.stage("refresh.momentum_in", device):
        ctx.left.refresh(state["left_basis"], rows)
        ctx.right.refresh(state["right_basis"], cols)
        rotate_planes(parameter_space, ctx.left.plain, ctx.right.plain, rows, cols, device, tag="T",
                      mode=k.EPI_STORE, out=momentum[:rows, :cols])
    return left_order, right_order

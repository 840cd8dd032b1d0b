"""Python wrappers of the native kernels (module ``soap_tp_b200._C``).

Everything here launches this package's own sm_100a kernels on the current CUDA stream; there is
no eager-PyTorch fallback.  If the extension is missing it is built in place
(``soap_tp_b200.build_ext``); if that fails the import error propagates -- a CUDA tensor never
silently takes another path.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, Optional

import torch
from torch import Tensor

try:
    from .. import _C  # type: ignore[attr-defined]
except ImportError:  # pragma: no cover - build on first use
    from .. import build_ext

    build_ext.build()
    from .. import _C  # type: ignore[attr-defined]

EPI_STORE, EPI_SPLIT, EPI_ADAM, EPI_ROW_MAJOR, EPI_PAIR_UPDATE, EPI_PUSH = 0, 1, 2, 3, 4, 5

STATUS_MESSAGES = {
    1: "GEMM consumer timed out waiting for a TMA stage",
    2: "GEMM producer timed out waiting for a free stage",
    3: "GEMM epilogue timed out waiting for the accumulator",
    4: "cross-rank barrier timed out",
    5: "bad kernel argument",
    6: "QR panel exchange between thread blocks timed out",
    7: "wait for a peer's data-ready flag timed out",
    8: "tridiagonalisation grid barrier timed out",
}

LAUNCH_COUNTS: Dict[str, int] = {}


def _count(name: str) -> None:
    LAUNCH_COUNTS[name] = LAUNCH_COUNTS.get(name, 0) + 1


def total_launches() -> int:
    """Number of kernels of this library launched by this process so far."""
    return sum(LAUNCH_COUNTS.values())


class SoapKernelError(RuntimeError):
    """A kernel of this library reported a bounded-wait timeout or a bad argument."""


class SoapCommTimeout(SoapKernelError):
    """A bounded device-side wait on a peer (barrier flag, data-ready flag) ran out."""


_STATUS: Dict[int, Tensor] = {}


def status_word(device: torch.device) -> Tensor:
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS.get(index)
    if word is None:
        word = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", index))
        _STATUS[index] = word
    return word


def _raise_for(index: int, code: int) -> None:
    kind = SoapCommTimeout if code in (4, 7) else SoapKernelError
    raise kind(f"cuda:{index}: {STATUS_MESSAGES.get(code, f'status {code}')}")


def check_status(device: Optional[torch.device] = None) -> None:
    """Synchronise and raise :class:`SoapKernelError` if any kernel gave up on a wait."""
    words = _STATUS.items() if device is None else [(device.index or 0, status_word(device))]
    for index, word in list(words):
        code = int(word[0].item())
        if code != 0:
            word.zero_()
            _MONITORS.pop(index, None)
            _raise_for(index, code)


class _StatusMonitor:
    """Deferred read-back of one device's status word: a 4-byte copy into pinned memory per step, looked at
    one step later, so that a timed-out wait surfaces as an exception without a device synchronisation."""

    waited_seconds = 0.0      # host time spent waiting for the previous step's copy (all devices of the process)

    def __init__(self, index: int, on_device: bool = True) -> None:
        self.index = index
        self.host = torch.zeros(2, dtype=torch.int32)
        # `on_device=False` serves the host-side tests, which hand in a CPU tensor as the status word
        self.events = [torch.cuda.Event(), torch.cuda.Event()] if on_device else None
        if on_device:
            self.host = self.host.pin_memory()
        self.pending = [False, False]
        self.turn = 0

    def poll(self, word: Tensor) -> None:
        previous = 1 - self.turn
        if self.pending[previous]:
            if self.events is not None:
                # recorded a whole step ago: complete unless the host runs a full step ahead of the device
                begin = time.perf_counter()
                self.events[previous].synchronize()
                _StatusMonitor.waited_seconds += time.perf_counter() - begin
            self.pending[previous] = False
            code = int(self.host[previous])
            if code != 0:
                word.zero_()
                self.pending = [False, False]
                _raise_for(self.index, code)
        self.host[self.turn:self.turn + 1].copy_(word[:1], non_blocking=True)
        if self.events is not None:
            self.events[self.turn].record()
        self.pending[self.turn] = True
        self.turn = previous


_MONITORS: Dict[int, _StatusMonitor] = {}


def poll_status(device: torch.device) -> None:
    """Called once per optimizer step on the step's stream.  Raises :class:`SoapKernelError` if the status
    word copied at the end of the PREVIOUS step was non-zero, then enqueues this step's copy.  A failure is
    therefore reported at most one step late and costs no synchronisation when nothing failed."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    monitor = _MONITORS.get(index)
    if monitor is None:
        monitor = _MONITORS[index] = _StatusMonitor(index)
    monitor.poll(status_word(torch.device("cuda", index)))


def mark_written(*tensors: Optional[Tensor]) -> None:
    """Bump the version counter of tensors a kernel wrote through a raw pointer, so that caches
    keyed on ``tensor._version`` (basis planes) notice the change."""
    for tensor in tensors:
        if tensor is not None:
            torch.autograd.graph.increment_version(tensor)


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


# SOAP_TP_MIXED_CORRECTIONS=0 keeps every product on three tf32 MMAs per k-step.  By default the products of the
# optimizer step (rotations, Gram EMAs, momentum transport) take their two correction terms as bf16 MMAs, see
# ``Planes``; the factorisations (QR, eigensolvers, power iteration) always use the full 3xTF32 form.
MIXED_CORRECTIONS = os.environ.get("SOAP_TP_MIXED_CORRECTIONS", "1") != "0"


def use_cta_pairs(on: bool) -> None:
    """Large plain products (at least 148 tiles of 128 x 256, no batching, no split-K) run on CTA pairs
    (``cta_group::2``: 256 x 256 tiles, each CTA staging half of the B tile) unless switched off here or with
    ``SOAP_TP_GEMM_CTA_PAIRS=0``."""
    _C.gemm_use_cta_pairs(bool(on))


if os.environ.get("SOAP_TP_GEMM_CTA_PAIRS", "1") == "0":
    use_cta_pairs(False)


@dataclass
class Planes:
    """Operand planes of a K x cols column-major matrix ``x``.

    Classic form: ``hi = rn_tf32(x)`` and ``lo = x - hi`` in fp32; a product is three tf32 MMAs per k-step
    (``lo*hi + hi*lo + hi*hi``).  Mixed form (``hl`` present, ``lo`` absent): ``hi`` as before plus one bf16 plane
    that holds, for every 32 elements of K, the 32 values ``hb = bf16(x)`` followed by the 32 values
    ``lb = bf16(x - hi)`` (one 128-byte row per TMA box and k-block; elements past K are zero).  The two correction
    products then run as bf16 MMAs at twice the tf32 rate (their terms are 2^-11 of the main term, so bf16's 2^-9
    leaves about 2^-20), with the same bytes per element.  Both operands of a product must be of the same form.
    """

    hi: Tensor
    lo: Optional[Tensor]
    depth: int   # K: the contiguous, contracted extent
    cols: int
    ld: int
    hl: Optional[Tensor] = None
    ld16: int = 0
    # windows handed out by `sub` (a launch-heavy driver asks for the same few thousand windows at every refresh, and
    # slicing tensors is what its launching thread would otherwise spend its time on)
    _windows: Dict[tuple, "Planes"] = field(default_factory=dict, repr=False, compare=False)

    @property
    def mixed(self) -> bool:
        return self.hl is not None

    @staticmethod
    def empty(depth: int, cols: int, device, mixed: bool = False) -> "Planes":
        ld = max(4, round_up(depth, 4))
        if not mixed:
            storage = torch.empty((2, max(1, cols), ld), dtype=torch.float32, device=device)
            return Planes(storage[0], storage[1], depth, cols, ld)
        ld16 = 2 * round_up(max(1, depth), 32)
        hi = torch.empty((max(1, cols), ld), dtype=torch.float32, device=device)
        hl = torch.zeros((max(1, cols), ld16), dtype=torch.bfloat16, device=device)     # zeros: the tail past K stays zero
        return Planes(hi, None, depth, cols, ld, hl, ld16)

    def sub(self, k0: int, c0: int, depth: int, cols: int) -> "Planes":
        """Operand planes of the sub-matrix starting at row ``k0`` (a multiple of 4; of 32 for mixed planes, whose
        depth may only be shortened to a multiple of 32), column ``c0``.  Windows are cached: treat them as
        read-only descriptions of the parent's memory."""
        key = (k0, c0, depth, cols)
        window = self._windows.get(key)
        if window is not None:
            return window
        assert k0 + depth <= self.ld and c0 + cols <= self.hi.shape[0]
        if self.mixed:
            assert k0 % 32 == 0 and (k0 + depth == self.depth or depth % 32 == 0)
            window = Planes(self.hi[c0:, k0:], None, depth, cols, self.ld, self.hl[c0:, 2 * k0:], self.ld16)
        else:
            assert k0 % 4 == 0
            window = Planes(self.hi[c0:, k0:], self.lo[c0:, k0:], depth, cols, self.ld)
        if len(self._windows) < 65536:
            self._windows[key] = window
        return window

    def low_pointers(self) -> dict:
        """Pointer arguments of the low part for the native calls."""
        if self.mixed:
            return dict(lo=0, hl=self.hl.data_ptr(), ld16=self.ld16)
        return dict(lo=self.lo.data_ptr(), hl=0, ld16=0)

    def halves(self):
        """(hb, lb) of mixed planes as ``cols x depth`` fp32 tensors (tests)."""
        groups = self.hl[: max(1, self.cols)].view(max(1, self.cols), -1, 2, 32).float()
        hb = groups[:, :, 0, :].reshape(max(1, self.cols), -1)[: self.cols, : self.depth]
        lb = groups[:, :, 1, :].reshape(max(1, self.cols), -1)[: self.cols, : self.depth]
        return hb, lb

    def dense(self) -> Tensor:
        """The represented K x cols matrix (for tests; to bf16 accuracy of the low part for mixed planes)."""
        low = self.halves()[1] if self.mixed else self.lo[: self.cols, : self.depth]
        return (self.hi[: self.cols, : self.depth] + low).T


SPLIT_ROUND_NEAREST = os.environ.get("SOAP_TP_SPLIT_NEAREST", "1") == "1"


def split_planes(source: Tensor, *, transpose: bool = False, out: Optional[Planes] = None, scale: float = 1.0,
                 nearest: Optional[bool] = None, mixed: bool = False) -> Planes:
    """Split a 2-D fp32 tensor (any strides) into operand planes (of the form of ``out``, else of ``mixed``).

    The operand is ``source`` itself (``depth = rows``) or, with ``transpose=True``, its transpose.
    """
    if source.dtype != torch.float32:
        source = source.float()
    rows, cols = source.shape
    s_i, s_j = source.stride()
    if transpose:
        rows, cols, s_i, s_j = cols, rows, s_j, s_i
    if out is None:
        out = Planes.empty(rows, cols, source.device, mixed=mixed)
    assert out.depth == rows and out.cols == cols
    low = out.low_pointers()
    _C.split_planes(source.data_ptr(), s_i, s_j, out.hi.data_ptr(), low["lo"], out.ld, rows, cols,
                    float(scale), int(SPLIT_ROUND_NEAREST if nearest is None else nearest), _stream(),
                    hl=low["hl"], ld16=low["ld16"])
    _count("split_planes_kernel")
    return out


def gemm(
    a: Planes,
    b: Planes,
    *,
    mode: int = EPI_STORE,
    out: Optional[Tensor] = None,
    out_ld: Optional[int] = None,
    out_planes: Optional[Planes] = None,
    alpha: float = 1.0,
    beta: float = 0.0,
    symmetric: bool = False,
    momentum: Optional[Tensor] = None,
    variance: Optional[Tensor] = None,
    adam: Optional[dict] = None,
    force_narrow: bool = False,
    k_splits: int = 1,
    split_stride: int = 0,
    batch: Optional[dict] = None,
    lower_of_grid: Optional[tuple] = None,
    push: Optional[dict] = None,
) -> None:
    """``acc[m, n] = sum_k a[k, m] * b[k, n]`` then the fused epilogue (see ``csrc/gemm.h``).

    ``out`` is a column-major ``M x N`` view for ``EPI_STORE`` (and the optional plain copy of
    ``EPI_SPLIT``/``EPI_ADAM``) or a row-major ``M x N`` tensor for ``EPI_ROW_MAJOR``.  ``EPI_PUSH`` writes no
    local output: ``push`` = ``dict(table, ld, ld16, nb, Pr, Pc, pr, pc, mixed)`` names the operand planes of the
    consuming ranks (``csrc/gemm.h``, ``kEpiPush``), which the epilogue fills through peer pointers.
    """
    if batch is None:
        assert a.depth == b.depth, (a.depth, b.depth)
        M, N, K = a.cols, b.cols, a.depth
    else:
        M, N, K = batch["M"], batch["N"], batch["K"]   # per batch item; a and b describe the whole buffers
    if M == 0 or N == 0:
        return
    c_ptr, ldc = 0, 0
    if out is not None:
        c_ptr = out.data_ptr()
        if mode == EPI_ROW_MAJOR:
            assert out.stride(1) == 1 or out.shape[1] == 1
            ldc = out.stride(0) if out.shape[0] > 1 else max(1, out.shape[1])
        else:
            assert out.stride(0) == 1 or out.shape[0] == 1
            ldc = out_ld if out_ld is not None else (out.stride(1) if out.shape[1] > 1 else max(1, out.shape[0]))
    if a.mixed != b.mixed:
        raise ValueError("both operands of a product must be classic planes or both mixed planes.")
    chi = clo = ldp = 0
    mixed_arguments = {}
    if a.mixed:
        mixed_arguments.update(a_hl=a.hl.data_ptr(), lda16=a.ld16, b_hl=b.hl.data_ptr(), ldb16=b.ld16)
    if out_planes is not None:
        assert batch is not None or (out_planes.depth == M and out_planes.cols == N)
        low = out_planes.low_pointers()
        chi, clo, ldp = out_planes.hi.data_ptr(), low["lo"], out_planes.ld
        if out_planes.mixed:
            assert beta == 0.0, "mixed output planes cannot be read-modify-written"
            mixed_arguments.update(Chl=low["hl"], ldp16=low["ld16"])
    mom = var = ldm = ldv = 0
    b1 = b2 = eps = ibc1 = isbc2 = 0.0
    if mode == EPI_ADAM:
        assert momentum is not None and variance is not None and adam is not None
        mom, var = momentum.data_ptr(), variance.data_ptr()
        ldm = momentum.stride(1) if momentum.shape[1] > 1 else max(1, momentum.shape[0])
        ldv = variance.stride(1) if variance.shape[1] > 1 else max(1, variance.shape[0])
        b1, b2, eps = adam["beta1"], adam["beta2"], adam["eps"]
        ibc1, isbc2 = 1.0 / adam["bias_correction1"], 1.0 / math.sqrt(adam["bias_correction2"])
    push_arguments = {}
    if mode == EPI_PUSH:
        assert push is not None and batch is None and k_splits == 1 and not symmetric
        push_arguments = dict(push_table=push["table"].data_ptr(), push_ld=int(push["ld"]), push_ld16=int(push["ld16"]),
                              push_nb=int(push["nb"]), push_Pr=int(push["Pr"]), push_Pc=int(push["Pc"]),
                              push_pr=int(push["pr"]), push_pc=int(push["pc"]), push_mixed=int(bool(push["mixed"])))
    status = status_word(a.hi.device)
    _C.gemm_tf32x3(a.hi.data_ptr(), a.low_pointers()["lo"], a.ld, b.hi.data_ptr(), b.low_pointers()["lo"], b.ld, M, N, K,
                   mode, 2 if lower_of_grid is not None else int(symmetric), int(force_narrow), float(alpha), float(beta), c_ptr, ldc, chi, clo, ldp,
                   mom, var, ldm, ldv, b1, b2, eps, ibc1, isbc2, int(k_splits), int(split_stride), status.data_ptr(),
                   _stream(), **_batch_arguments(a, b, batch), **_triangle_arguments(lower_of_grid), **mixed_arguments,
                   **push_arguments)
    mark_written(out, momentum, variance)
    _count("gemm_tf32x3_kernel")


def _triangle_arguments(lower_of_grid: Optional[tuple]) -> dict:
    """``(block_size, pr, Pr, pc, Pc[, m0, n0])``: produce only the entries of this rank's packed block that
    lie on or below the global diagonal of a symmetric result; ``m0, n0`` is the local index of the output's
    first element when the output is a window of the packed block."""
    if lower_of_grid is None:
        return {}
    nb, pr, Pr, pc, Pc = lower_of_grid[:5]
    m0, n0 = (lower_of_grid[5], lower_of_grid[6]) if len(lower_of_grid) > 5 else (0, 0)
    return dict(tri_nb=int(nb), tri_pr=int(pr), tri_Pr=int(Pr), tri_pc=int(pc), tri_Pc=int(Pc), tri_m0=int(m0),
                tri_n0=int(n0))


def _batch_arguments(a: "Planes", b: "Planes", batch: Optional[dict]) -> dict:
    """Keyword arguments of the batched launch (see ``csrc/gemm.h``): ``a`` and ``b`` are the whole operand
    buffers, the per-item sub-blocks start at multiples of the ``*_step`` values."""
    if batch is None:
        return {}
    second = batch.get("out2_planes")
    remap = batch.get("remap")
    return dict(
        batches=int(batch["count"]), a_k_step=int(batch.get("a_k_step", 0)), a_row_step=int(batch.get("a_row_step", 0)),
        b_k_step=int(batch.get("b_k_step", 0)), b_row_step=int(batch.get("b_row_step", 0)),
        c_batch_stride=int(batch.get("c_batch_stride", 0)), a_k_total=a.depth, a_rows_total=a.cols, b_k_total=b.depth,
        b_rows_total=b.cols, remap=remap.data_ptr() if remap is not None else 0,
        C2hi=second.hi.data_ptr() if second is not None else 0, C2lo=second.lo.data_ptr() if second is not None else 0,
        ld2=second.ld if second is not None else 0, m_limit=int(batch.get("m_limit", 0)),
        o1_row_start=int(batch.get("o1_row_start", 0)))


def gemm_simt(a: Tensor, b: Tensor, out: Tensor, *, alpha: float = 1.0, beta: float = 0.0) -> Tensor:
    """``out[m, n] = alpha * sum_k a[k, m] * b[k, n] + beta * out`` in fp32 FMA (any strides)."""
    K, M = a.shape
    K2, N = b.shape
    assert K == K2 and out.shape == (M, N)
    _C.gemm_simt(a.data_ptr(), a.stride(0), a.stride(1), b.data_ptr(), b.stride(0), b.stride(1), out.data_ptr(),
                 out.stride(0), out.stride(1), M, N, K, float(alpha), float(beta), _stream())
    _count("gemm_simt_kernel")
    return out


def _ld(t: Tensor) -> int:
    return t.stride(1) if t.shape[1] > 1 else max(1, t.shape[0])


def adam_update(gradient: Tensor, momentum: Tensor, variance: Tensor, beta1: float, beta2: float, eps: float,
                bias_correction1: float, bias_correction2: float) -> Tensor:
    """Fused Adam on 2-D tensors; the result has the strides of ``variance``."""
    for t in (gradient, momentum, variance):
        if t.dtype != torch.float32 or t.ndim != 2:
            raise ValueError("adam_update on CUDA needs 2-D float32 tensors.")
    update = torch.empty_strided(variance.shape, variance.stride(), dtype=torch.float32, device=variance.device)
    rows, cols = variance.shape
    views = [gradient, momentum, variance, update]
    if not all(v.stride(0) == 1 or v.shape[0] == 1 for v in views):
        if all(v.stride(1) == 1 or v.shape[1] == 1 for v in views):
            views = [v.T for v in views]
            rows, cols = cols, rows
        else:
            raise ValueError("adam_update needs all operands column-major or all row-major.")
    g, m, v, u = views
    _C.adam_update(g.data_ptr(), _ld(g), m.data_ptr(), _ld(m), v.data_ptr(), _ld(v), u.data_ptr(), _ld(u), rows, cols,
                   beta1, beta2, eps, 1.0 / bias_correction1, 1.0 / math.sqrt(bias_correction2), _stream())
    _count("adam_kernel")
    return update


def column_dot(a: Tensor, b: Tensor, rows: int, cols: int, out: Optional[Tensor] = None) -> Tensor:
    if out is None:
        out = torch.empty(cols, dtype=torch.float32, device=a.device)
    _C.column_dot(a.data_ptr(), _ld(a), b.data_ptr(), _ld(b), out.data_ptr(), rows, cols, _stream())
    _count("column_dot_kernel")
    return out


def order_by_estimate(table: Tensor) -> Tensor:
    """Stable descending order of the column sums of ``table`` (``parts x n``, any strides with unit row stride or a
    single row): the eigenvalue order of a refresh.  One launch of this library's sort kernel for ``n`` up to
    ``ORDER_MAX_LENGTH``; longer vectors use the framework's sort."""
    parts, n = table.shape
    if n > _C.ORDER_MAX_LENGTH or (parts > 1 and table.stride(0) != 1):
        return torch.argsort(table.sum(dim=0), descending=True, stable=True)
    order = torch.empty(n, dtype=torch.int64, device=table.device)
    ld = table.stride(1) if n > 1 else parts
    _C.order_by_estimate(table.data_ptr(), ld, parts, n, order.data_ptr(), _stream())
    _count("order_by_estimate_kernel")
    return order


def gather2d(src: Tensor, dst: Tensor, row_map: Optional[Tensor], col_map: Optional[Tensor]) -> Tensor:
    """``dst[i, j] = src[row_map[i], col_map[j]]`` (``None`` = identity); ``dst`` must not alias ``src``."""
    rows, cols = dst.shape
    _C.gather2d(src.data_ptr(), src.stride(0), src.stride(1), dst.data_ptr(), dst.stride(0), dst.stride(1),
                row_map.data_ptr() if row_map is not None else 0, col_map.data_ptr() if col_map is not None else 0,
                rows, cols, _stream())
    _count("gather2d_kernel")
    return dst

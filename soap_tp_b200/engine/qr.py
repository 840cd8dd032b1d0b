"""Blocked Householder QR on one GPU with tensor-core trailing updates.

``householder_qr(A, Q, order)`` overwrites ``Q`` with the explicit orthogonal factor of
``A[:, order]``, the contract of the reference's ``slate_qr_float`` (``geqrf`` + ``unmqr`` on an
identity, ``src/soap_tp/csrc/slate_bindings.cpp:125-189``).  Per 128-column panel:

    panel kernel (cooperative, panel resident in registers)      -> V, V^T, T, T^T planes, tau
    Z = T V^T                      (3xTF32 tcgen05 GEMM, K = 128)
    W = V^T C_trailing             (split-K GEMM, partials summed in fixed order -> deterministic)
    C_trailing -= Z^T W            (GEMM whose epilogue read-modify-writes the operand planes)

and the same three GEMMs build the explicit ``Q``: in reverse panel order from the identity when two
factorisations run together (fewest flops), or forwards, panel by panel on a stream of its own under
the panel chain, when a factorisation runs alone (nothing left to do after the last panel).  The
trailing matrix and ``Q`` live as hi/lo operand planes throughout, so no separate split pass is
needed between panels.  Look-ahead: panel ``p + 1`` is factored on a high-priority stream as soon as
the reflector of panel ``p`` has reached its columns, while the rest of the update proceeds.  All
arithmetic is fp32-class (3xTF32 products, fp32 panel).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch
from torch import Tensor

from . import kernels as k

_C = k._C
PANEL = _C.QR_PANEL_WIDTH
# Two Householder columns per exchange step of the panel kernel where that is numerically safe
# (SOAP_TP_QR_PAIR_STEPS=0: the one-column kernel).
PAIR_STEPS = os.environ.get("SOAP_TP_QR_PAIR_STEPS", "1") != "0"
# The reflectors of two consecutive panels reach the far columns (and the forward-accumulated Q^T) as ONE rank-256
# update: half the passes over those matrices, which are what the updates cost (SOAP_TP_QR_AGGREGATE=0: one rank-128
# update per panel).
AGGREGATE = os.environ.get("SOAP_TP_QR_AGGREGATE", "1") != "0"
_WORKSPACES: Dict[tuple, dict] = {}


def _workspace(n: int, device, slot: int = 0) -> dict:
    key = (n, str(device), slot)
    ws = _WORKSPACES.get(key)
    if ws is None:
        panels = -(-n // PANEL)
        ws = {
            "C": k.Planes.empty(n, n, device),
            "Q": k.Planes.empty(n, n, device),
            "V": k.Planes.empty(n, n, device),
            "Vt": [k.Planes.empty(min(PANEL, n - p * PANEL), n, device) for p in range(panels)],
            "T": [k.Planes.empty(min(PANEL, n - p * PANEL), PANEL, device) for p in range(panels)],
            "Tt": [k.Planes.empty(min(PANEL, n - p * PANEL), PANEL, device) for p in range(panels)],
            "Z": k.Planes.empty(PANEL, n, device),
            "W": k.Planes.empty(PANEL, n, device),
            "tau": torch.zeros(n + PANEL, dtype=torch.float32, device=device),
            "S": torch.zeros(PANEL * PANEL, dtype=torch.float32, device=device),
            "exchange": torch.zeros(8 * 160 * PANEL + 8 * PANEL, dtype=torch.float32, device=device),
            "partials": torch.empty(16 * PANEL * n, dtype=torch.float32, device=device),
            # scratch of the forward accumulation of Q, which runs on a stream of its own
            "partials_q": torch.empty(16 * PANEL * n, dtype=torch.float32, device=device),
            "Zq": k.Planes.empty(PANEL, n, device), "Wq": k.Planes.empty(PANEL, n, device),
            "staging": torch.empty((n, n), dtype=torch.float32, device=device).T,
            # reflectors of two consecutive panels applied as one rank-256 update (see `_pair_reflector`); the set
            # with the suffix "q" serves the forward accumulation of Q on its own stream
            "zero_block": torch.zeros((PANEL, PANEL), dtype=torch.float32, device=device),
        }
        for suffix in ("", "q"):
            ws["Z2" + suffix] = k.Planes.empty(2 * PANEL, n, device)
            ws["W2" + suffix] = k.Planes.empty(2 * PANEL, n, device)
            ws["partials2" + suffix] = torch.empty(16 * 2 * PANEL * n, dtype=torch.float32, device=device)
            for name in ("S2", "Y2", "A2"):
                ws[name + suffix] = k.Planes.empty(PANEL, PANEL, device)
        _WORKSPACES[key] = ws
    return ws


def release_workspaces() -> None:
    _WORKSPACES.clear()


def release_workspaces_for(n: int, device) -> None:
    for key in [key for key in _WORKSPACES if key[0] == n and key[1] == str(device)]:
        del _WORKSPACES[key]


def _splits(tiles: int, k_blocks: int) -> int:
    wanted = max(1, -(-296 // max(1, tiles)))
    return max(1, min(wanted, 16, max(1, k_blocks // 4)))


def _skinny_product(ws: dict, a: k.Planes, b: k.Planes, out: k.Planes, scratch: str = "partials") -> None:
    """``out <- a^T b`` for a narrow ``a`` (at most 128 columns): split-K partials + ordered sum."""
    M, N, K = a.cols, b.cols, a.depth
    splits = _splits(-(-N // 128), -(-K // 32))
    ld = M
    partials = ws[scratch]
    view = partials[: ld * N].view(N, ld).T
    k.gemm(a, b, mode=k.EPI_STORE, out=view, out_ld=ld, force_narrow=True, k_splits=splits, split_stride=ld * N)
    _C.sum_partials_to_planes(partials.data_ptr(), splits, ld * N, ld, out.hi.data_ptr(), out.lo.data_ptr(), out.ld,
                              M, N, k._stream())
    k._count("sum_partials_kernel")


def householder_qr(matrix: Tensor, Q: Tensor, column_order: Optional[Tensor] = None) -> Tensor:
    """``Q <- explicit orthogonal factor of matrix[:, column_order]`` on the current stream.

    A lone factorisation is bound by its chain of panel kernels, so ``Q`` is accumulated forwards
    (``Q^T <- H_p^T Q^T`` as soon as panel ``p`` exists) on a third stream under that chain: 50 % more
    arithmetic than the backward accumulation, none of it on the critical path.
    """
    forward = os.environ.get("SOAP_TP_QR_FORWARD_Q", "1") != "0"
    for _ in _factorisation_steps(matrix, Q, column_order, 0, forward_q=forward):
        pass
    return Q


_SIDE_STREAMS: Dict[tuple, "torch.cuda.Stream"] = {}
_PANEL_STREAMS: Dict[tuple, "torch.cuda.Stream"] = {}


def _panel_stream(device, slot: int) -> "torch.cuda.Stream":
    key = (str(device), slot)
    if key not in _PANEL_STREAMS:
        _PANEL_STREAMS[key] = torch.cuda.Stream(device=device, priority=-1)
    return _PANEL_STREAMS[key]


def householder_qr_pair(jobs) -> None:
    """Factor several independent matrices at the same time.

    ``jobs`` is a list of ``(matrix, Q, column_order)``.  Each factorisation is issued panel by panel on
    its own stream, alternating between the jobs, so that the latency-bound panel kernel of one
    factorisation (a few dozen thread blocks) runs while the tensor-core updates of the other keep the
    remaining SMs busy.  The calling stream waits for all of them.
    """
    if len(jobs) == 1:
        householder_qr(*jobs[0])
        return
    device = jobs[0][0].device
    main = torch.cuda.current_stream(device)
    ready = torch.cuda.Event()
    ready.record(main)
    streams, steps = [], []
    for slot, (matrix, Q, order) in enumerate(jobs):
        key = (str(device), slot)
        if key not in _SIDE_STREAMS:
            _SIDE_STREAMS[key] = torch.cuda.Stream(device=device)
        stream = _SIDE_STREAMS[key]
        stream.wait_event(ready)
        streams.append(stream)
        steps.append(_factorisation_steps(matrix, Q, order, slot))
    alive = list(range(len(jobs)))
    while alive:
        for slot in list(alive):
            with torch.cuda.stream(streams[slot]):
                try:
                    next(steps[slot])
                except StopIteration:
                    alive.remove(slot)
    for stream in streams:
        done = torch.cuda.Event()
        done.record(stream)
        main.wait_event(done)


def _q_stream(device, slot: int) -> "torch.cuda.Stream":
    key = (str(device), slot, "q")
    if key not in _PANEL_STREAMS:
        _PANEL_STREAMS[key] = torch.cuda.Stream(device=device)
    return _PANEL_STREAMS[key]


def _pair_reflector(ws: dict, V: k.Planes, a: int, n: int, suffix: str = "", backward: bool = False) -> tuple:
    """``(V2, Z2)`` for the reflectors of two full-width panels ``a``, ``b = a + 1`` taken together:
    ``H_a H_b = I - V2 T2 V2^T`` with ``V2 = [V_a, V_b]`` (the window of the reflector planes that starts at panel
    ``a``; the caller has zeroed the 128 rows of ``V_b``'s columns above its own first row) and
    ``T2 = [[T_a, T_ab], [0, T_b]]``, ``T_ab = -T_a (V_a^T V_b) T_b``.

    Forward (trailing matrix, forward accumulation of ``Q^T``): ``Z2 = T2 V2^T = [[Z_a + T_ab V_b^T], [0, Z_b]]`` and
    ``C -= Z2^T (V2^T C)`` applies ``(H_a H_b)^T`` in one pass over ``C``.  ``backward`` (explicit ``Q`` from the
    identity, last panel first): ``Z2 = T2^T V2^T = [[T_a^T V_a^T], [T_ab^T V_a^T + [0, T_b^T V_b^T]]]`` and
    ``Q -= Z2^T (V2^T Q)`` applies ``H_a H_b``.  Seven small products either way; ``suffix`` selects the scratch set
    (the forward accumulation of ``Q`` runs on its own stream).
    """
    ja = a * PANEL
    jb, ra = ja + PANEL, n - ja
    rb = ra - PANEL
    b = a + 1
    planes_of = lambda t: k.Planes(t.hi, t.lo, PANEL, PANEL, t.ld)
    T_a, Tt_a, T_b, Tt_b = (planes_of(ws[name][i]) for name, i in (("T", a), ("Tt", a), ("T", b), ("Tt", b)))
    vt_a, vt_b = ws["Vt"][a].sub(0, 0, PANEL, ra), ws["Vt"][b].sub(0, 0, PANEL, rb)
    S, Y, A, Z2 = ws["S2" + suffix], ws["Y2" + suffix], ws["A2" + suffix], ws["Z2" + suffix]
    va_low, vb = V.sub(jb, ja, rb, PANEL), V.sub(jb, jb, rb, PANEL)
    small = dict(mode=k.EPI_SPLIT, force_narrow=True)
    if backward:
        _skinny_product(ws, vb, va_low, S, scratch="partials2" + suffix)                # S^T = V_b^T V_a
        k.gemm(S, T_b, out_planes=Y, **small)                                            # S T_b
        k.gemm(Tt_a, Y, out_planes=A, alpha=-1.0, **small)                               # T_ab = -T_a (S T_b)
        k.gemm(T_a, vt_a, out_planes=Z2.sub(0, 0, PANEL, ra), **small)                   # T_a^T V_a^T
        k.gemm(A, vt_a, out_planes=Z2.sub(PANEL, 0, PANEL, ra), **small)                 # T_ab^T V_a^T
        k.gemm(T_b, vt_b, out_planes=Z2.sub(PANEL, PANEL, PANEL, rb), beta=1.0, **small)   # + T_b^T V_b^T
    else:
        _skinny_product(ws, va_low, vb, S, scratch="partials2" + suffix)                # S = V_a^T V_b
        k.gemm(S, Tt_a, out_planes=Y, **small)                                           # S^T T_a^T
        k.gemm(T_b, Y, out_planes=A, alpha=-1.0, **small)                                # T_ab^T = -T_b^T S^T T_a^T
        k.gemm(Tt_a, vt_a, out_planes=Z2.sub(0, 0, PANEL, ra), **small)                  # Z_a
        k.gemm(A, vt_b, out_planes=Z2.sub(0, PANEL, PANEL, rb), beta=1.0, **small)       # + T_ab V_b^T
        k.split_planes(ws["zero_block"], out=Z2.sub(PANEL, 0, PANEL, PANEL))
        k.gemm(Tt_b, vt_b, out_planes=Z2.sub(PANEL, PANEL, PANEL, rb), **small)          # Z_b
    return V.sub(ja, ja, ra, 2 * PANEL), Z2.sub(0, 0, 2 * PANEL, ra)


def _factorisation_steps(matrix: Optional[Tensor], Q: Optional[Tensor], column_order: Optional[Tensor], slot: int,
                         forward_q: bool = False, publisher=None, size: Optional[int] = None, device=None):
    """The blocked factorisation as a generator: yields after the launches of every panel.

    With a ``publisher`` (``engine/dist_qr.py``) this rank only runs the panel chain and the trailing updates:
    the reflectors ``V`` and the products ``Z_p = T_p V_p^T`` are written into the publisher's buffers, which
    other ranks can read, ``publisher.announce(p)`` is called on the main stream once panel ``p``'s are complete,
    and the explicit ``Q`` is accumulated elsewhere.  ``matrix=None``: the workspace planes ``C`` already hold
    the (column-permuted) input.
    """
    n = matrix.shape[0] if matrix is not None else int(size)
    device = matrix.device if matrix is not None else device
    ws = _workspace(n, device, slot)
    C, Qp = ws["C"], ws["Q"]
    V = publisher.V if publisher is not None else ws["V"]
    if matrix is not None:
        assert matrix.shape == (n, n)
        source = matrix
        if column_order is not None:
            source = ws["staging"]
            k.gather2d(matrix, source, None, column_order)
        k.split_planes(source, out=C)
    stream = k._stream
    panels = list(range(0, n, PANEL))
    main = torch.cuda.current_stream(device)
    side = _panel_stream(device, slot) if os.environ.get("SOAP_TP_QR_LOOKAHEAD", "1") != "0" else main
    status_pointer = k.status_word(device).data_ptr()

    def launch_panel(p: int, after: "torch.cuda.Event") -> "torch.cuda.Event":
        """Panel ``p`` on the panel stream, once ``after`` has happened; returns its completion event."""
        j0 = panels[p]
        bw, r = min(PANEL, n - j0), n - j0
        panel, v, vt = C.sub(j0, j0, r, bw), V.sub(j0, j0, r, bw), ws["Vt"][p]
        tau = ws["tau"][j0:]
        T, Tt = ws["T"][p], ws["Tt"][p]
        side.wait_event(after)
        # launched on the panel stream by its handle (entering a stream context costs the launching thread more
        # than the launch itself)
        arguments = (panel.hi.data_ptr(), panel.lo.data_ptr(), panel.ld, r, bw, v.hi.data_ptr(), v.lo.data_ptr(),
                     v.ld, vt.hi.data_ptr(), vt.lo.data_ptr(), vt.ld, tau.data_ptr(), T.hi.data_ptr(),
                     T.lo.data_ptr(), Tt.hi.data_ptr(), Tt.lo.data_ptr(), T.ld, ws["exchange"].data_ptr(),
                     status_pointer, side.cuda_stream)
        if PAIR_STEPS:
            # 256-row CTAs: measured faster than (2048 rows and up) or within 2 % of (1024 rows) 128-row CTAs
            _C.qr_panel_pairs(*arguments, 256)
        else:
            _C.qr_panel(*arguments)
        k._count("qr_panel_kernel")
        done = torch.cuda.Event()
        done.record(side)
        return done

    def z_of(p: int) -> k.Planes:
        bw, r = min(PANEL, n - panels[p]), n - panels[p]
        if publisher is not None:
            return publisher.z(p).sub(0, 0, bw, r)
        return ws["Z"].sub(0, 0, bw, r)      # only full-width panels have columns to their right

    def update(p: int, first_col: int, count: int) -> None:
        """Apply the block reflector of panel ``p`` to ``count`` columns starting at ``first_col``."""
        j0 = panels[p]
        bw, r = min(PANEL, n - j0), n - j0
        v = V.sub(j0, j0, r, bw)
        z = z_of(p)
        w = ws["W"].sub(0, 0, bw, count)
        block = C.sub(j0, first_col, r, count)
        _skinny_product(ws, v, block, w)                                                    # W = V^T C
        k.gemm(z, w, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0)               # C -= Z^T W

    # Look-ahead: as soon as the reflector of panel p has been applied to the columns of panel p + 1,
    # that panel is factored on a second (high-priority) stream while this stream applies the reflector
    # to the remaining columns.  The latency-bound panel kernel occupies a few dozen SMs; the
    # tensor-core updates use the others.
    start = torch.cuda.Event()
    start.record(main)
    done = launch_panel(0, start)

    q_stream = None
    forward_q = forward_q and publisher is None
    if forward_q:
        # Q^T lives in the planes `Qp`; every panel's reflector is applied to its rows j0.. from the left,
        # exactly like the trailing matrix, on a stream of its own with its own scratch.
        q_stream = _q_stream(device, slot)
        q_stream.wait_event(start)
        with torch.cuda.stream(q_stream):
            _C.identity_planes(Qp.hi.data_ptr(), Qp.lo.data_ptr(), Qp.ld, n, n, stream())
            k._count("identity_planes_kernel")

    def accumulate_q(p: int, after: "torch.cuda.Event") -> None:
        j0 = panels[p]
        bw, r = min(PANEL, n - j0), n - j0
        q_stream.wait_event(after)
        with torch.cuda.stream(q_stream):
            v, vt, Tt = V.sub(j0, j0, r, bw), ws["Vt"][p], ws["Tt"][p]
            t_op = k.Planes(Tt.hi, Tt.lo, bw, bw, Tt.ld)
            z = ws["Zq"].sub(0, 0, bw, r) if bw == PANEL else k.Planes.empty(bw, r, device)
            k.gemm(t_op, vt.sub(0, 0, bw, r), mode=k.EPI_SPLIT, out_planes=z, force_narrow=True)   # Z = T V^T
            block = Qp.sub(j0, 0, r, n)
            w = ws["Wq"].sub(0, 0, bw, n) if bw == PANEL else k.Planes.empty(bw, n, device)
            _skinny_product(ws, v, block, w, scratch="partials_q")                                # W = V^T Q^T
            k.gemm(z, w, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0)                 # Q^T -= Z^T W
    # A leader that publishes its reflectors to worker ranks keeps one update per panel: its factorisation is bound by
    # the chain of panels (and, with eight processes on one host, by its launching thread), so the pair update's
    # dozen extra small launches per pair buy nothing there (8192 on 4 GPUs: refresh.qr 3.29 against 3.26-3.35 ms/step).
    aggregate = AGGREGATE and publisher is None

    def paired(p: int) -> bool:
        """Panel ``p`` (even) hands its far updates over to a rank-256 update together with panel ``p + 1``."""
        return aggregate and p % 2 == 0 and p + 1 < len(panels) and n - panels[p + 1] >= PANEL

    def far_update(p: int, first_col: int, count: int) -> None:
        """The reflector of panel ``p`` for the columns beyond the next panel."""
        if p % 2 == 1 and paired(p - 1):
            # both panels' reflectors in one pass over these columns (they have seen neither)
            ja = panels[p - 1]
            v2, z2 = _pair_reflector(ws, V, p - 1, n)
            w2 = ws["W2"].sub(0, 0, 2 * PANEL, count)
            block = C.sub(ja, first_col, n - ja, count)
            _skinny_product(ws, v2, block, w2, scratch="partials2")
            k.gemm(z2, w2, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0)
        elif paired(p):
            update(p, first_col, min(PANEL, count))    # only the panel after next, which is factored before the pair update
        else:
            update(p, first_col, count)

    def accumulate_q_pair(p: int, after: "torch.cuda.Event") -> None:
        """``Q^T <- (H_{p-1} H_p)^T Q^T`` in one pass (forward accumulation, own stream and scratch)."""
        ja = panels[p - 1]
        q_stream.wait_event(after)
        with torch.cuda.stream(q_stream):
            v2, z2 = _pair_reflector(ws, V, p - 1, n, suffix="q")
            block = Qp.sub(ja, 0, n - ja, n)
            w2 = ws["W2q"].sub(0, 0, 2 * PANEL, n)
            _skinny_product(ws, v2, block, w2, scratch="partials2q")
            k.gemm(z2, w2, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0)

    for p, j0 in enumerate(panels):
        bw, r = min(PANEL, n - j0), n - j0
        nc = n - j0 - bw
        main.wait_event(done)
        panel_done = done
        if paired(p):
            # rows of the next panel's reflector columns above its own first row: zero, so that the two panels'
            # reflectors can be used as one 256-column operand (nothing else ever writes there)
            k.split_planes(ws["zero_block"], out=V.sub(j0, j0 + PANEL, PANEL, PANEL))
        if nc > 0 or publisher is not None:
            vt, Tt = ws["Vt"][p], ws["Tt"][p]
            t_op = k.Planes(Tt.hi, Tt.lo, bw, bw, Tt.ld)
            vt_op = vt.sub(0, 0, bw, r)
            k.gemm(t_op, vt_op, mode=k.EPI_SPLIT, out_planes=z_of(p), force_narrow=True)      # Z = T V^T
            if publisher is not None:
                publisher.announce(p)
        if nc > 0:
            ahead = min(PANEL, nc)
            update(p, j0 + bw, ahead)
            ready = torch.cuda.Event()
            ready.record(main)
            done = launch_panel(p + 1, ready)
            if nc > ahead:
                far_update(p, j0 + bw + ahead, nc - ahead)
        if forward_q:
            if p % 2 == 1 and paired(p - 1):
                accumulate_q_pair(p, panel_done)
            elif not paired(p):
                accumulate_q(p, panel_done)
        yield
    if publisher is not None:
        return
    if forward_q:
        finished = torch.cuda.Event()
        finished.record(q_stream)
        main.wait_event(finished)
        # planes element [c, k] of Q^T is Q[c, k]: hi + lo, read row-major, is Q itself
        row_major = ws["staging"].T
        _C.planes_sum(Qp.hi.data_ptr(), Qp.lo.data_ptr(), Qp.ld, row_major.data_ptr(), n, n, n, stream())
        k._count("planes_sum_kernel")
        k.gather2d(row_major, Q, None, None)
        k.mark_written(Q)
        return
    # explicit Q = H_0 H_1 ... applied to the identity, last panel first
    _C.identity_planes(Qp.hi.data_ptr(), Qp.lo.data_ptr(), Qp.ld, n, n, stream())
    k._count("identity_planes_kernel")
    for p in reversed(range(len(panels))):
        j0 = panels[p]
        bw, r = min(PANEL, n - j0), n - j0
        if p % 2 == 1 and paired(p - 1):
            continue                                     # applied together with panel p - 1
        block = Qp.sub(j0, j0, r, r)
        if paired(p):
            v2, z2 = _pair_reflector(ws, V, p, n, backward=True)
            w2 = ws["W2"].sub(0, 0, 2 * PANEL, r)
            _skinny_product(ws, v2, block, w2, scratch="partials2")                         # W = [V_a V_b]^T Q
            k.gemm(z2, w2, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0,
                   out=Q if p == 0 else None)                                               # Q -= Z2^T W
            continue
        v, vt, T = V.sub(j0, j0, r, bw), ws["Vt"][p], ws["T"][p]
        t_op = k.Planes(T.hi, T.lo, bw, bw, T.ld)
        vt_op = vt.sub(0, 0, bw, r)
        z = ws["Z"].sub(0, 0, bw, r) if bw == PANEL else k.Planes.empty(bw, r, device)
        k.gemm(t_op, vt_op, mode=k.EPI_SPLIT, out_planes=z, force_narrow=True)                # Z = T^T V^T
        w = ws["W"].sub(0, 0, bw, r) if bw == PANEL else k.Planes.empty(bw, r, device)
        _skinny_product(ws, v, block, w)                                                    # W = V^T Q
        k.gemm(z, w, mode=k.EPI_SPLIT, out_planes=block, alpha=-1.0, beta=1.0,
               out=Q if p == 0 else None)                                                   # Q -= Z^T W
    k.mark_written(Q)

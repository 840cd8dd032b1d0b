"""Executable specification of the two-columns-per-exchange Householder panel (``csrc/qr_panel_pairs.cu``).

A NumPy restatement, in fp32, of the arithmetic the device kernel performs per step -- without the
CTA partitioning, since sums over CTAs are plain sums here.  It exists so that the algebra can be
checked on a CPU: every quantity the second reflector of a step needs is derived from the dot
products of the two RAW pivot columns with all columns (``D1``, ``D2``) and from the two pivot rows
(``p1``, ``p2``), because the first reflector is orthogonal.  ``threshold`` is the kernel's guard
against cancellation in ``|y'|^2 = D2[c+1] - y'[c]^2``: below it the step retires one column only.

Returns ``V`` (unit lower trapezoid), ``tau``, the compact-WY factor ``T`` with
``H_0 ... H_{b-1} = I - V T V^T``, and the numbers of one- and two-column steps taken.
"""
from __future__ import annotations

from typing import Tuple

import numpy as np


def _householder_scalars(alpha: np.float32, normsq: np.float32) -> Tuple[np.float32, np.float32]:
    f = np.float32
    tail = normsq - alpha * alpha
    if tail > 0 and normsq > 0:
        beta = -np.copysign(np.sqrt(normsq), alpha)
        return f((beta - alpha) / beta), f(f(1) / (alpha - beta))
    return f(0), f(0)


def factor_panel(A: np.ndarray, threshold: float = 0.5):
    f = np.float32
    P = np.array(A, dtype=f)                  # the register slab: finished columns keep their unscaled v
    m, b = P.shape
    tau = np.zeros(b, f)
    scale = np.ones(b, f)
    S = np.zeros((b, b), f)                   # S[j, c] = v_j . v_c for j < c
    steps = [0, 0]
    c = 0
    reflectors = min(m, b)
    while c < reflectors:
        can_pair = c + 1 < reflectors
        x = P[:, c].copy()
        x[:c] = 0
        y = P[:, c + 1].copy() if c + 1 < b else np.zeros(m, f)
        y[:c] = 0
        D1 = (x[:, None] * P).sum(0, dtype=f)
        D2 = (y[:, None] * P).sum(0, dtype=f)
        p1 = P[c, :].copy()
        p2 = P[c + 1, :].copy() if c + 1 < m else np.zeros(b, f)
        sj = np.where(np.arange(b) < c, scale, f(1))
        a1, n1, p2c = p1[c], D1[c], p2[c]
        t1, s1 = _householder_scalars(a1, n1)
        w1 = (p1 + s1 * (D1 - a1 * p1)) * sj                  # v_c . column_j
        tau[c], scale[c] = t1, s1
        S[:c, c] = w1[:c]
        pair = False
        if can_pair:
            k = t1 * w1[c + 1]                                  # y' = H_c y = y - k v_c
            yc = p1[c + 1] - k
            yc1 = p2[c + 1] - k * s1 * p2c
            n2 = D2[c + 1] - yc * yc
            pair = bool(n2 > f(threshold) * D2[c + 1])
        if pair:
            t2, s2 = _householder_scalars(yc1, n2)
            tau[c + 1], scale[c + 1] = t2, s2
            ajc = p1 - t1 * w1                                  # (H_c a_j)[c]
            ajc1 = p2 - t1 * w1 * s1 * p2c                      # (H_c a_j)[c + 1]
            w2 = ajc1 + s2 * (D2 - yc * ajc - yc1 * ajc1)       # v_{c+1} . (H_c a_j), columns right of the pair
            sum_y = D2 - p1[c + 1] * p1 - p2[c + 1] * p2
            sum_x = D1 - a1 * p1 - p2c * p2
            left = (p2 + s2 * (sum_y - k * s1 * sum_x)) * sj    # v_{c+1} . v_j, finished columns
            S[:c, c + 1] = left[:c]
            sxy = (D1[c + 1] - a1 * p1[c + 1] - p2c * p2[c + 1]) - k * s1 * (n1 - a1 * a1 - p2c * p2c)
            S[c, c + 1] = s1 * p2c + s1 * s2 * sxy              # v_c . v_{c+1}
        first_free = c + (2 if pair else 1)
        for j in range(c + 1, b):                               # sweep 2
            B = t2 * w2[j] * s2 if (pair and j > c + 1) else f(0)
            Acoef = t1 * w1[j] * s1 - (B * k * s1 if pair else f(0))
            P[:, j] = P[:, j] - Acoef * x - (B * y if pair else f(0))
            P[c, j] = 0                                         # retired pivot rows
            if pair:
                P[c + 1, j] = 0
        steps[1 if pair else 0] += 1
        c = first_free
    V = np.zeros((m, b), f)
    for j in range(reflectors):
        V[j + 1:, j] = P[j + 1:, j] * scale[j]
        V[j, j] = 1
    T = np.zeros((b, b), f)
    for j in range(reflectors):
        T[:j, j] = -tau[j] * (T[:j, :j] @ S[:j, j])
        T[j, j] = tau[j]
    return V, tau, T, tuple(steps)


__all__ = ["factor_panel"]

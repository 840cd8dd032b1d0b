"""The distributed op cases on CUDA devices.

World size 1 exercises the single-GPU pipeline.  Larger worlds start one process per rank; when
the box has fewer GPUs than ranks several ranks share a GPU (the kernels never wait on another
rank inside a launch -- cross-rank ordering is host-side on such a box -- so this is safe), and
the control plane is gloo.
"""
import pytest

import op_cases as cases
from distributed_helpers import run_distributed

pytestmark = pytest.mark.gpu

RECT = [(8, 8), (8, 12), (12, 8), (9, 13), (13, 9)]
TINY = (10, 2, (0.8, 0.9), 0.75, 1e-6, 1e-5)


def test_single_gpu_ops():
    g = (1, 1)
    specs = [("case_redistribute", ((9, 13), 4, g, 0)), ("case_redistribute", ((300, 200), 128, g, 1))]
    specs += [("case_gram", (shape, 2, g, sd, 0.0)) for shape in RECT for sd in (0, 1)]
    specs += [("case_gram", ((300, 520), 128, g, 1, 0.25))]
    specs += [("case_rotate", (shape, 2, g)) for shape in RECT] + [("case_rotate", ((260, 390), 128, g))]
    specs += [("case_permute", ((9, 13), 2, g)), ("case_permute", ((200, 300), 64, g))]
    specs += [("case_power_iteration_qr", (n, 2, g)) for n in (8, 9, 12, 13)]
    specs += [("case_power_iteration_qr", (200, 64, g)), ("case_estimated_order_and_qr", (12, 2, g))]
    specs += [("case_initialize_basis", (gs, side, 2, g, "eigh")) for gs, side in
              [((8, 8), "left"), ((8, 12), "right"), ((12, 8), "left"), ((9, 13), "left")]]
    specs += [("case_initialize_basis", ((150, 100), "left", 32, g, "jacobi"))]
    specs += [("case_refresh", (shape, 2, g)) for shape in [(8, 8), (8, 12), (13, 9)]]
    specs += [("case_refresh", ((200, 136), 64, g))]
    run_distributed(cases.case_batch, 1, "cuda", specs)


def test_single_gpu_trajectory():
    g = (1, 1)
    specs = [("case_soap_trajectory", (shape, 2, g, sd) + TINY)
             for shape in [(8, 8), (20, 20), (12, 12), (8, 12)] for sd in (0, 1)]
    run_distributed(cases.case_batch, 1, "cuda", specs)

"""End-to-end ``soap_step`` trajectories on CPU ranks against the dense oracle.

The tiny regime (block 2, betas (0.8, 0.9), preconditioner beta 0.75, eps 1e-6, refresh every
2 steps, 10 calls, relative L2 <= 1e-5 on update and parameter; first update exactly zero; QR
called 2*floor(step/interval) times) is the reference's end-to-end test
(``tests/unit/test_soap.py:34-54,791-817,844-854``).
"""
import op_cases as cases
from distributed_helpers import run_distributed

TINY = (10, 2, (0.8, 0.9), 0.75, 1e-6, 1e-5)


def test_reference_matches_distributed_soap():
    specs = [("case_soap_trajectory", (shape, 2, (2, 2), sd) + TINY)
             for shape in [(8, 8), (20, 20), (12, 12)] for sd in (0, 1)]
    specs += [("case_soap_trajectory", ((8, 12), 2, (2, 2), 1) + TINY),
              ("case_soap_trajectory", ((12, 8), 2, (2, 2), 0) + TINY)]
    run_distributed(cases.case_batch, 4, "cpu", specs)


def test_two_ranks_and_one_rank():
    run_distributed(cases.case_batch, 2, "cpu", [("case_soap_trajectory", ((12, 12), 2, (1, 2), 1) + TINY)])
    run_distributed(cases.case_batch, 1, "cpu", [("case_soap_trajectory", ((8, 8), 2, (1, 1), 0) + TINY)])

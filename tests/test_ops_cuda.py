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
# ..., noise-floor perturbation: 3e-6 relative is the measured backward error of the device eigensolver and
# of a chain of 3xTF32 products (residual ||P Q - Q diag|| / ||P|| = 1e-6 ... 2.5e-6 for n = 1024 ... 8192)
TINY = (10, 2, (0.8, 0.9), 0.75, 1e-6, 1e-5, "eigh", 2.0, 3e-6)


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


def test_shared_basis_trajectory():
    """The oracle's eigenbases injected after the warm-up call, so that the bound (1e-5, no noise floor) does not
    depend on the eigensolver under test: 1 GPU and a (2, 2) grid, ragged and multi-block shapes."""
    run_distributed(cases.case_batch, 1, "cuda", [
        ("case_soap_shared_basis", ((20, 20), 2, (1, 1), 1, 6, 1e-5)),
        ("case_soap_shared_basis", ((384, 260), 64, (1, 1), 0, 6, 1e-5))])
    run_distributed(cases.case_batch, 4, "cuda", [
        ("case_soap_shared_basis", ((12, 16), 3, (2, 2), 0, 6, 1e-5)),
        ("case_soap_shared_basis", ((384, 256), 64, (2, 2), 1, 6, 1e-5))])


GRID4 = (2, 2)


def test_four_ranks_ops():
    specs = [("case_redistribute", (shape, 2, GRID4, sd)) for shape, sd in
             [((8, 8), 0), ((20, 20), 1), ((12, 16), 0), ((9, 12), 1)]]
    specs += [("case_redistribute", ((20, 20), 3, GRID4, 1)), ("case_redistribute", ((8, 8), 16, GRID4, 0)),
              ("case_redistribute", ((300, 200), 64, GRID4, 1))]
    specs += [("case_gram", (shape, 2, GRID4, sd, 0.0)) for shape in RECT for sd in (0, 1)]
    specs += [("case_gram", ((9, 13), 2, GRID4, 1, 0.25)), ("case_gram", ((300, 520), 64, GRID4, 1, 0.25))]
    specs += [("case_gram_1d", ((8, 12), 0.0)), ("case_gram_1d", ((300, 520), 0.25))]
    specs += [("case_rotate", (shape, 2, GRID4)) for shape in RECT] + [("case_rotate", ((260, 390), 64, GRID4))]
    specs += [("case_permute", ((9, 13), 2, GRID4)), ("case_permute", ((200, 300), 64, GRID4))]
    specs += [("case_power_iteration_qr", (n, 2, GRID4)) for n in (8, 9, 13)]
    specs += [("case_power_iteration_qr", (200, 64, GRID4)), ("case_estimated_order_and_qr", (12, 2, GRID4))]
    specs += [("case_initialize_basis", ((8, 12), "right", 2, GRID4, "eigh")),
              ("case_initialize_basis", ((9, 13), "left", 2, GRID4, "jacobi"))]
    specs += [("case_refresh", (shape, 2, GRID4)) for shape in [(8, 12), (13, 9)]]
    specs += [("case_redistribute_permute_subgroups", ((12, 8), 2)), ("case_redistribute_permute_subgroups", ((260, 384), 64))]
    run_distributed(cases.case_batch, 4, "cuda", specs)


def test_qr_spread_over_the_ranks():
    """Factorisations with several panels on 4 and 8 ranks: the panel chain runs on a leader rank, the explicit
    Q is accumulated by the other ranks of the job's group and pulled into the packed layout."""
    specs = [("case_power_iteration_qr", (700, 128, GRID4)), ("case_refresh", ((520, 390), 128, GRID4)),
             ("case_qr_properties", (1100, 128, GRID4, "random")), ("case_qr_properties", (650, 64, GRID4, "rank_deficient")),
             ("case_qr_properties", (384, 128, GRID4, "graded"))]
    run_distributed(cases.case_batch, 4, "cuda", specs)
    run_distributed(cases.case_batch, 8, "cuda", [
        ("case_refresh", ((400, 300), 64, (2, 4))), ("case_qr_properties", (900, 128, (2, 4), "rank_deficient"))])


def test_four_ranks_trajectory():
    specs = [("case_soap_trajectory", (shape, 2, GRID4, sd) + TINY)
             for shape in [(8, 8), (20, 20), (12, 12)] for sd in (0, 1)]
    specs += [("case_soap_trajectory", ((8, 12), 2, GRID4, 1) + TINY)]
    run_distributed(cases.case_batch, 4, "cuda", specs)


def test_two_ranks_and_eight_ranks():
    run_distributed(cases.case_batch, 2, "cuda", [
        ("case_rotate", ((9, 13), 2, (1, 2))), ("case_gram", ((9, 13), 2, (2, 1), 0, 0.5)),
        ("case_soap_trajectory", ((12, 12), 2, (1, 2), 1) + TINY)])
    run_distributed(cases.case_batch, 8, "cuda", [
        ("case_rotate", ((40, 24), 4, (2, 4))), ("case_soap_trajectory", ((16, 16), 2, (2, 4), 1) + TINY)])


def test_chunked_gather_product_pipeline(monkeypatch):
    """Force the peer pulls to be split into chunks that overlap with their products (as they are at
    8192 on real grids) on shapes small enough for a shared test GPU; compare with the dense oracle."""
    monkeypatch.setenv("SOAP_TP_PIPELINE_GATHERS", "1")
    monkeypatch.setenv("SOAP_TP_PIPELINE_MIN_TILES", "1")
    big = (10, 3, (0.8, 0.9), 0.75, 1e-6, 1e-5, "eigh", 2.0, 3e-6)
    for world, grid in ((4, GRID4), (2, (1, 2))):
        run_distributed(cases.case_batch, world, "cuda", [
            ("case_gram", ((600, 520), 64, grid, 1, 0.25)), ("case_gram", ((520, 650), 128, grid, 0, 0.5)),
            ("case_rotate", ((520, 650), 64, grid)),
            ("case_soap_trajectory", ((384, 384), 64, grid, 1) + big)])


def test_push_products(monkeypatch):
    """The first product of every two-sided product pushes its result into the consumers' operand planes through
    peer pointers (GEMM -> all-gather in the epilogue) instead of being pulled: rotations, refresh (momentum
    transport) and whole trajectories on (2, 2), (1, 2) and (2, 4) grids against the same oracles."""
    monkeypatch.setenv("SOAP_TP_PUSH_PRODUCTS", "1")
    run_distributed(cases.case_batch, 4, "cuda", [
        ("case_rotate", ((9, 13), 2, GRID4)), ("case_rotate", ((260, 390), 64, GRID4)),
        ("case_refresh", ((200, 136), 64, GRID4)), ("case_soap_shared_basis", ((384, 256), 64, GRID4, 1, 6, 1e-5)),
        ("case_soap_trajectory", ((20, 20), 2, GRID4, 1) + TINY)])
    run_distributed(cases.case_batch, 2, "cuda", [("case_rotate", ((260, 390), 128, (1, 2))),
                                                   ("case_soap_trajectory", ((12, 12), 2, (1, 2), 1) + TINY)])
    run_distributed(cases.case_batch, 8, "cuda", [("case_rotate", ((520, 390), 64, (2, 4)))])


def test_grids_that_are_not_powers_of_two():
    """Three ranks as a (3, 1) grid and six ranks as a (2, 3) grid through the CUDA engine (the single-GPU QR's
    leader/worker split then has groups of one and three ranks), small and multi-block shapes."""
    def specs(grid):
        return [("case_redistribute", ((12, 18), 2, grid, 0)), ("case_gram", ((12, 18), 2, grid, 1, 0.25)),
                ("case_gram", ((384, 252), 64, grid, 0, 0.5)), ("case_rotate", ((12, 18), 2, grid)),
                ("case_rotate", ((390, 264), 64, grid)), ("case_permute", ((18, 12), 4, grid)),
                ("case_power_iteration_qr", (13, 2, grid)), ("case_power_iteration_qr", (700, 128, grid)),
                ("case_initialize_basis", ((12, 18), "right", 2, grid, "eigh")), ("case_refresh", ((12, 18), 2, grid)),
                ("case_refresh", ((390, 264), 64, grid)), ("case_soap_shared_basis", ((12, 18), 2, grid, 1, 5, 1e-5)),
                ("case_soap_shared_basis", ((384, 252), 64, grid, 0, 5, 1e-5))]

    run_distributed(cases.case_batch, 3, "cuda", specs((3, 1)))
    run_distributed(cases.case_batch, 6, "cuda", specs((2, 3)))


def test_basis_planes_rebuilt_after_eviction(monkeypatch):
    """With no room in the cache of basis planes every basis is split again on every use (the two bases of a
    parameter evict each other): same trajectories on one GPU and on a (2, 2) grid."""
    monkeypatch.setenv("SOAP_TP_BASIS_CACHE_GB", "0")
    run_distributed(cases.case_batch, 1, "cuda", [("case_soap_shared_basis", ((384, 260), 64, (1, 1), 0, 5, 1e-5)),
                                                   ("case_soap_trajectory", ((20, 20), 2, (1, 1), 1) + TINY)])
    run_distributed(cases.case_batch, 4, "cuda", [("case_soap_shared_basis", ((384, 256), 64, GRID4, 1, 5, 1e-5)),
                                                   ("case_soap_trajectory", ((20, 20), 2, GRID4, 1) + TINY)])

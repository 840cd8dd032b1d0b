"""Distributed op tests on CPU ranks (gloo; 4 processes on grid (2, 2), plus 1- and 2-rank grids).

Shapes and tolerances follow the reference's op-level tests: block size 2, shapes 8x8, 8x12,
12x8, 9x13, 13x9 with unequal ``tensor_split`` shards for the Gram updates
(``tests/unit/test_preconditioners.py:137-141,387-418``), rotations and refresh at 1e-5 / 2e-4
(``tests/unit/test_factorizations.py:345-373``), QR sizes 8, 9, 12, 13
(``tests/unit/test_slate_bindings.py:244-323``), eigenpairs of rank-deficient Gram matrices
(``tests/unit/test_elpa_bindings.py:478-501``).  Cases that share a world size run in one
process group because process start-up dominates at these sizes.
"""
import op_cases as cases
from distributed_helpers import run_distributed

GRID = (2, 2)
RECT = [(8, 8), (8, 12), (12, 8), (9, 13), (13, 9)]


def test_redistribution():
    specs = [("case_redistribute", (shape, 2, GRID, sd)) for shape, sd in
             [((8, 8), 0), ((8, 8), 1), ((20, 20), 1), ((12, 16), 0), ((16, 12), 1), ((9, 12), 1), ((12, 9), 0)]]
    specs.append(("case_redistribute", ((20, 20), 3, GRID, 1)))   # shard boundary cuts blocks
    specs.append(("case_redistribute", ((8, 8), 16, GRID, 0)))    # three ranks own nothing
    run_distributed(cases.case_batch, 4, "cpu", specs)


def test_gram_updates():
    specs = [("case_gram", (shape, 2, GRID, sd, 0.0)) for shape in RECT for sd in (0, 1)]
    specs.append(("case_gram", ((9, 13), 2, GRID, 1, 0.25)))      # beta and initial value
    specs += [("case_gram_1d", ((8, 12), 0.0)), ("case_gram_1d", ((12, 8), 0.25))]   # 1-D row-sharded results
    specs += [("case_gram_1d_subgroups", ((8, 12), 0.25))]
    run_distributed(cases.case_batch, 4, "cpu", specs)


def test_rotations_and_permutation():
    specs = [("case_rotate", (shape, 2, GRID)) for shape in RECT]
    specs += [("case_permute", (shape, 2, GRID)) for shape in [(8, 8), (9, 13)]]
    specs += [("case_redistribute_permute_subgroups", ((12, 8), 2))]
    run_distributed(cases.case_batch, 4, "cpu", specs)


def test_power_iteration_qr_and_basis():
    specs = [("case_power_iteration_qr", (n, 2, GRID)) for n in (8, 9, 12, 13)]
    specs.append(("case_estimated_order_and_qr", (12, 2, GRID)))
    specs += [("case_qr_properties", (24, 4, GRID, "rank_deficient")), ("case_qr_properties", (20, 4, GRID, "graded"))]
    specs += [("case_initialize_basis", (g, side, 2, GRID, "eigh")) for g, side in
              [((8, 8), "left"), ((8, 12), "right"), ((12, 8), "left"), ((9, 13), "left")]]
    specs += [("case_refresh", (shape, 2, GRID)) for shape in [(8, 8), (8, 12), (13, 9)]]
    run_distributed(cases.case_batch, 4, "cpu", specs)


def test_single_rank_grid():
    run_distributed(cases.case_batch, 1, "cpu", [
        ("case_rotate", ((9, 13), 4, (1, 1))), ("case_refresh", ((8, 12), 3, (1, 1))),
        ("case_gram", ((9, 13), 4, (1, 1), 1, 0.5)), ("case_redistribute", ((9, 13), 4, (1, 1), 0)),
        ("case_gram_1d", ((9, 13), 0.5)),
    ])


def test_two_rank_grids():
    run_distributed(cases.case_batch, 2, "cpu", [
        ("case_rotate", ((9, 13), 2, (1, 2))), ("case_gram", ((9, 13), 2, (2, 1), 0, 0.5)),
        ("case_refresh", ((8, 12), 2, (2, 1))), ("case_redistribute", ((12, 10), 3, (1, 2), 1)),
    ])


def test_shared_basis_trajectory():
    """The oracle's eigenbases injected after the warm-up call: every later step agrees to 1e-5 with no noise floor."""
    run_distributed(cases.case_batch, 4, "cpu", [
        ("case_soap_shared_basis", ((20, 20), 2, (2, 2), 1, 6, 1e-5)),
        ("case_soap_shared_basis", ((12, 16), 3, (2, 2), 0, 6, 1e-5)),
        ("case_soap_shared_basis", ((96, 64), 16, (2, 2), 1, 5, 1e-5))])


ODD_GRID_SPECS = lambda grid, world: [
    ("case_redistribute", ((12, 18), 2, grid, 0)), ("case_redistribute", ((18, 12), 4, grid, 1)),
    ("case_gram", ((12, 18), 2, grid, 1, 0.25)), ("case_gram", ((18, 12), 4, grid, 0, 0.0)),
    ("case_rotate", ((12, 18), 2, grid)), ("case_permute", ((18, 12), 4, grid)),
    ("case_power_iteration_qr", (13, 2, grid)), ("case_initialize_basis", ((12, 18), "right", 2, grid, "eigh")),
    ("case_refresh", ((12, 18), 2, grid)),
    ("case_soap_shared_basis", ((12, 18), 2, grid, 1, 5, 1e-5)),
]


def test_grids_that_are_not_powers_of_two():
    """Three ranks as a (3, 1) column of processes and six ranks as a (2, 3) grid: every rank class has a different
    number of blocks and some ranks own ragged or empty edges."""
    run_distributed(cases.case_batch, 3, "cpu", ODD_GRID_SPECS((3, 1), 3))
    run_distributed(cases.case_batch, 6, "cpu", ODD_GRID_SPECS((2, 3), 6))

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


def test_headline_cpu_configuration_1024():
    """The CPU configuration of record: four gloo ranks on grid (2, 2), one 1024 x 1024 fp32 parameter, column
    shards, block 128, N(0, 1) gradients, betas (0.95, 0.95), refresh every 10 steps, ``"eigh"``, 21 calls.
    At this size two correct fp32 implementations agree only down to the dense oracle's own sensitivity to
    rounding, so the bound per step is ``max(1e-5, 3 x distance of the oracle to itself under a 1e-6 relative
    perturbation of the gradients)`` (about 4e-4 after the initialisation and 6e-4 after the refresh)."""
    spec = ("case_soap_trajectory", ((1024, 1024), 128, (2, 2), 1, 21, 10, (0.95, 0.95), 0.95, 1e-8, 1e-5, "eigh", 1.0, 1e-6))
    run_distributed(cases.case_batch, 4, "cpu", [spec], timeout=900.0)


def _injected_bindings(rank, world):
    """The reference's own test pattern (``tests/unit/test_soap.py:402-412``): a proxy around the native binding
    counts QR calls while ``soap_step`` runs through it; the trajectory must equal the built-in path's."""
    import torch

    from soap_tp_b200 import bindings, soap_step

    class Counting:
        def __init__(self, inner):
            self._inner, self.calls = inner, {}

        def __getattr__(self, name):
            target = getattr(self._inner, name)
            if not callable(target):
                return target

            def counted(*args, **kwargs):
                self.calls[name] = self.calls.get(name, 0) + 1
                return target(*args, **kwargs)

            return counted

    slate, elpa = Counting(bindings.slate_bindings), Counting(bindings.elpa_bindings)
    shape, steps, interval = (12, 8), 7, 2
    plain, routed = {}, {}
    for it in range(steps):
        G = torch.randn(shape, generator=torch.Generator().manual_seed(200 + it))
        shard = G.chunk(world, dim=1)[rank].contiguous()
        common = dict(global_shape=shape, shard_dim=1, block_size=2, process_grid_shape=(2, 2),
                      basis_refresh_interval=interval, basis_implementation="elpa")
        expected = soap_step(shard, plain, **common)
        got = soap_step(shard, routed, slate_binding=slate, elpa_binding=elpa, **common)
        torch.testing.assert_close(got, expected, rtol=2e-4, atol=2e-5)
    refreshes = (steps - 1) // interval
    assert slate.calls["slate_qr_float"] == 2 * refreshes
    assert slate.calls["slate_symmetric_multiply_float"] == 2 * refreshes
    assert slate.calls["slate_forward_rotation_float"] == (steps - 1) + refreshes
    assert slate.calls["slate_backward_rotation_float"] == (steps - 1) + refreshes
    assert elpa.calls["elpa_eigenvectors_2d_block_cyclic_double"] == 2


def test_injected_native_bindings_are_called():
    run_distributed(_injected_bindings, 4)

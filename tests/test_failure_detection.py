"""Failure detection without a device fault: every failure is made on the host.

* ranks that disagree about a collective (shape, op order, permutation) get a clean error on EVERY rank;
* a rank that leaves between steps makes the others' next collective end with an error after a short
  process-group timeout instead of hanging;
* a checkpoint written on another grid is refused.

The reference's counterparts are the permutation check of ``src/soap_tp/ops/optimizer.py:439-452`` and the
rank-matching comment of ``src/soap_tp/ops/factorizations.py:85-101``; it has no checkpoint or liveness checks.
"""
import os

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


def _mismatched_shape(rank, world):
    from soap_tp_b200 import soap_step
    from soap_tp_b200.parallel.guard import SoapCollectiveMismatch

    os.environ["SOAP_TP_CHECK_COLLECTIVES"] = "1"
    shape = (8, 8) if rank != 1 else (8, 12)           # rank 1 believes in another parameter
    shard = torch.randn(shape[0], shape[1] // world)
    with pytest.raises(SoapCollectiveMismatch) as caught:
        soap_step(shard, {}, global_shape=shape, shard_dim=1, block_size=2, process_grid_shape=(2, 2),
                  basis_implementation="eigh")
    assert "rank 1: ('soap_step', (8, 12)" in str(caught.value) and "rank 0: ('soap_step', (8, 8)" in str(caught.value)
    dist.barrier()     # every rank raised and is still usable


def _mismatched_op_order(rank, world):
    from soap_tp_b200 import layout, ops
    from soap_tp_b200.parallel.guard import SoapCollectiveMismatch

    os.environ["SOAP_TP_CHECK_COLLECTIVES"] = "1"
    grid, nb, n = (2, 2), 2, 8
    buffer = lambda: layout.allocate_2d_block_cyclic((n, n), nb, grid)
    with pytest.raises(SoapCollectiveMismatch, match="ranks disagree"):
        if rank == 2:    # skips ahead to the next op of its program
            ops.qr_2d_block_cyclic_(buffer(), buffer(), n, nb, grid)
        else:
            ops.rotate_2d_block_cyclic_(buffer(), buffer(), buffer(), (n, n), nb, grid, direction="forward")
    dist.barrier()


def _mismatched_permutation(rank, world):
    from soap_tp_b200 import layout, ops

    grid, nb, shape = (2, 2), 2, (8, 8)
    matrix = layout.allocate_2d_block_cyclic(shape, nb, grid)
    order = list(range(8))
    mine = order if rank != 3 else order[::-1]
    with pytest.raises(ValueError, match="must match on every rank"):
        ops.permute_2d_block_cyclic_(matrix, shape, mine, order, nb, grid)
    dist.barrier()


def _rank_leaves_between_steps(rank, world):
    from soap_tp_b200 import soap_step

    shape = (8, 8)
    state: dict = {}
    step = lambda seed: soap_step(torch.randn(8, 8 // world, generator=torch.Generator().manual_seed(seed + rank)), state,
                                  global_shape=shape, shard_dim=1, block_size=2, process_grid_shape=(1, 2),
                                  basis_implementation="eigh")
    step(0)
    step(1)
    dist.barrier()
    if rank == 1:
        return           # leaves between steps, nothing of its own in flight
    with pytest.raises(Exception) as caught:      # gloo reports a timeout or a closed connection
        step(2)
    assert not isinstance(caught.value, AssertionError)


def test_mismatched_global_shape_raises_on_every_rank():
    run_distributed(_mismatched_shape, 4)


def test_mismatched_op_order_raises_on_every_rank():
    run_distributed(_mismatched_op_order, 4)


def test_mismatched_permutation_raises_on_every_rank():
    run_distributed(_mismatched_permutation, 4)


def test_rank_that_leaves_between_steps_ends_the_others_collective():
    run_distributed(_rank_leaves_between_steps, 2, pg_timeout=5.0, timeout=120.0)


def _stale_layout(rank, world):
    from soap_tp_b200.optim import SoapTP

    weight = torch.nn.Parameter(torch.zeros(8, 8 // world))
    weight.tp_shard_dim, weight.tp_global_shape = 1, (8, 8)
    make = lambda grid: SoapTP([weight], block_size=2, process_grid_shape=grid, basis_implementation="eigh",
                               precondition_frequency=2)
    written = make((1, 2))
    for seed in range(3):
        weight.grad = torch.randn(weight.shape, generator=torch.Generator().manual_seed(seed + rank))
        written.step()
    checkpoint = written.state_dict()
    make((1, 2)).load_state_dict(checkpoint)                 # same grid: accepted
    with pytest.raises(ValueError, match="does not match the current layout"):
        make((2, 1)).load_state_dict(checkpoint)             # another grid: refused on every rank
    dist.barrier()


def test_checkpoint_of_another_grid_is_refused():
    run_distributed(_stale_layout, 2)


def _long_leader_work_is_awaited_on_the_host(rank, world):
    """The device barrier's budget must not have to cover a leader's long factorisation: with
    ``after_long_work`` every rank first meets the others on the control plane.  Here the device barrier is
    replaced by a recorder, and rank 0 is late by more than the 'budget' the recorder would allow."""
    import time

    from soap_tp_b200.parallel import comm as comm_module

    class Recorder(comm_module.Communicator):
        def __init__(self):            # no device, no segments: only the ordering logic is under test
            self.world, self.rank, self.control = world, rank, dist.group.WORLD
            self.use_device_barrier, self.barrier_count = True, 0
            self._epochs, self._channel_stride = [0] * self.CHANNELS, 64
            self.device, self.barrier_timeout_s = torch.device("cpu"), 0.75
            self.arrivals = []

    recorder = Recorder()

    class FakeC:
        @staticmethod
        def device_barrier(*args):
            recorder.arrivals.append(time.monotonic())

    recorder._C = FakeC()
    recorder._pads = type("P", (), {"peer_table": torch.zeros(1, dtype=torch.int64)})()
    import soap_tp_b200.engine.kernels as kernels

    original_status, original_count = kernels.status_word, kernels._count
    original_sync = torch.cuda.current_stream
    kernels.status_word = lambda device: torch.zeros(4, dtype=torch.int32)
    torch.cuda.current_stream = lambda *a, **k: type("S", (), {"synchronize": lambda self: None, "cuda_stream": 0})()
    try:
        if rank == 0:
            time.sleep(2.0)        # the "leader" is still factoring
        recorder.barrier(after_long_work=True)
    finally:
        kernels.status_word, kernels._count, torch.cuda.current_stream = original_status, original_count, original_sync
    stamps = [None] * world
    dist.all_gather_object(stamps, recorder.arrivals[0])
    # every rank reached the device barrier within the spin budget of the others, although rank 0 was 2 s late
    assert max(stamps) - min(stamps) < recorder.barrier_timeout_s, stamps


def test_long_waits_are_taken_on_the_host_before_the_device_barrier():
    run_distributed(_long_leader_work_is_awaited_on_the_host, 2)


@pytest.mark.gpu
def test_device_barrier_gives_up_within_its_budget_and_reports():
    """A bounded device-side wait that nothing satisfies: the barrier kernel of "rank 0 of 2" spins on a flag
    that no peer ever writes, with a 2 ms budget.  The kernel must return by itself, leave code 4 in the
    status word and keep the context usable; the deferred monitor turns the code into SoapCommTimeout."""
    from soap_tp_b200.engine import kernels

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    kernels._MONITORS.pop(0, None)
    pads = [torch.zeros(64, dtype=torch.int32, device=device) for _ in range(2)]
    table = torch.tensor([p.data_ptr() for p in pads], dtype=torch.int64, device=device)
    status = kernels.status_word(device)
    status.zero_()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    kernels._C.device_barrier(table.data_ptr(), 0, 2, 1, status.data_ptr(), 0.002, torch.cuda.current_stream().cuda_stream)
    stop.record()
    torch.cuda.synchronize()
    assert start.elapsed_time(stop) < 500.0            # milliseconds: it gave up, it did not hang
    assert int(pads[1][0]) == 1                         # its own arrival was published to the "peer"
    assert int(status[0]) == 4
    kernels.poll_status(device)                         # takes the copy
    with pytest.raises(kernels.SoapCommTimeout, match="barrier timed out"):
        kernels.poll_status(device)                     # reads it one step later
    assert int(status[0]) == 0
    # the context is still usable
    assert float((torch.ones(8, device=device) * 2).sum()) == 16.0
    # a barrier whose peer HAS arrived passes and leaves the status word clean
    pads[0][1] = 2
    kernels._C.device_barrier(table.data_ptr(), 0, 2, 2, status.data_ptr(), 0.5, torch.cuda.current_stream().cuda_stream)
    kernels.check_status(device)

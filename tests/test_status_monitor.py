"""Host-side tests of the deferred status read-back (no GPU: the status word is a CPU tensor here).

Every bounded wait of the kernels reports through one int32 status word per device; ``poll_status`` is
what turns a non-zero word into an exception inside ``soap_step`` one step later.
"""
import pytest
import torch

from soap_tp_b200.engine import kernels


def test_monitor_raises_one_poll_after_the_word_was_set():
    word = torch.zeros(4, dtype=torch.int32)
    monitor = kernels._StatusMonitor(0, on_device=False)
    monitor.poll(word)          # step 1: clean
    monitor.poll(word)          # step 2: clean
    word[0] = 4                 # a barrier gave up during step 3
    monitor.poll(word)          # end of step 3: the copy is taken, nothing is raised yet
    with pytest.raises(kernels.SoapCommTimeout, match="barrier timed out"):
        monitor.poll(word)      # end of step 4: the copy of step 3 is read
    assert int(word[0]) == 0    # cleared, so that a caller who handles the error can go on
    monitor.poll(word)
    monitor.poll(word)


@pytest.mark.parametrize("code,kind", [(1, kernels.SoapKernelError), (6, kernels.SoapKernelError),
                                       (7, kernels.SoapCommTimeout)])
def test_monitor_maps_codes_to_exception_types(code, kind):
    word = torch.zeros(4, dtype=torch.int32)
    monitor = kernels._StatusMonitor(0, on_device=False)
    word[0] = code
    monitor.poll(word)
    with pytest.raises(kind) as caught:
        monitor.poll(word)
    assert kernels.STATUS_MESSAGES[code] in str(caught.value)
    assert issubclass(kernels.SoapCommTimeout, kernels.SoapKernelError)


def test_poll_status_uses_the_device_word(monkeypatch):
    word = torch.zeros(4, dtype=torch.int32)
    monkeypatch.setattr(kernels, "status_word", lambda device: word)
    monkeypatch.setitem(kernels._MONITORS, 0, kernels._StatusMonitor(0, on_device=False))
    device = torch.device("cuda", 0)
    kernels.poll_status(device)
    word[0] = 3
    kernels.poll_status(device)
    with pytest.raises(kernels.SoapKernelError, match="accumulator"):
        kernels.poll_status(device)


def test_basis_plane_cache_is_bounded(monkeypatch):
    """The per-parameter caches of basis planes evict entries beyond a byte limit (most recently used first, so that a cyclic
    walk over the parameters keeps a resident set); the entry in use always stays (host logic only: no planes are built here)."""
    import torch

    from soap_tp_b200.engine import local

    monkeypatch.setattr(local, "BASIS_CACHE_BYTES", 12 * (64 * 64 + 32 * 32) * 2)      # room for two parameters
    local._CONTEXTS.clear()
    states = [dict(left_basis=torch.zeros(64, 64), right_basis=torch.zeros(32, 32), momentum=torch.zeros(64, 32))
              for _ in range(4)]
    contexts = [local.context_for(state) for state in states]
    assert list(local._CONTEXTS.values()) == [contexts[0], contexts[3]]
    # an optimizer walks its parameters in the same order every step: with room for c of them, c - 1 accesses per
    # pass find their planes (dropping the least recently used one instead would make every access miss)
    for _ in range(3):
        hits = 0
        for state in states:
            resident = list(local._CONTEXTS.values())
            hits += any(local.context_for(state) is ctx for ctx in resident)
        assert hits >= 1 and len(local._CONTEXTS) == 2
    local._CONTEXTS.clear()


def test_grid_engine_evicts_dead_then_most_recent_basis_planes(monkeypatch):
    """Eviction in the multi-GPU engine depends only on the order of use and on rank-independent sizes, so every
    rank drops the same entries: entries of tensors that no longer exist first, then the most recently used."""
    import weakref
    from collections import OrderedDict

    import torch

    from soap_tp_b200.engine import distributed

    monkeypatch.setattr(distributed, "BASIS_CACHE_BYTES", 250)
    engine = object.__new__(distributed.GridEngine)
    engine._basis_cache = OrderedDict()
    alive = [torch.zeros(1) for _ in range(4)]
    gone = torch.zeros(1)
    engine._basis_cache[("gone", 1)] = dict(bytes=100, owner=weakref.ref(gone))
    del gone
    for index, tensor in enumerate(alive):
        engine._basis_cache[(index, 1)] = dict(bytes=100, owner=weakref.ref(tensor))
    engine._evict_basis_planes(keep=(3, 1))
    # 500 bytes -> the dead entry, then the most recently used ones other than the one in use, until 250 fit
    assert list(engine._basis_cache) == [(0, 1), (3, 1)]
    engine._evict_basis_planes(keep=(3, 1))
    assert list(engine._basis_cache) == [(0, 1), (3, 1)]


def test_windows_of_operand_planes_are_cached_views():
    import torch

    from soap_tp_b200.engine.kernels import Planes

    hi, lo = torch.arange(48.0).reshape(6, 8), torch.zeros(6, 8)
    planes = Planes(hi, lo, 8, 6, 8)
    window = planes.sub(4, 2, 4, 3)
    assert planes.sub(4, 2, 4, 3) is window and planes.sub(4, 2, 4, 2) is not window
    assert window.depth == 4 and window.cols == 3 and window.ld == 8
    assert window.hi.data_ptr() == hi[2:, 4:].data_ptr() and float(window.hi[0, 0]) == float(hi[2, 4])
    hi[2, 4] = -1.0                                   # a window is a view: it sees what is written to the parent
    assert float(window.hi[0, 0]) == -1.0
    assert window.dense().shape == (4, 3)

"""Host-side helpers of the device engines that need no GPU: chunk planning for the pull/product
pipeline, leader assignment of the dense factorisations, argument checks of the row-sharded Gram
updates."""
import importlib

import pytest
import torch


def _distributed(monkeypatch, **env):
    for key, value in env.items():
        monkeypatch.setenv(key, value)
    import soap_tp_b200.engine.distributed as module

    return importlib.reload(module)


def test_column_chunks_cover_the_range_once(monkeypatch):
    module = _distributed(monkeypatch, SOAP_TP_PIPELINE_GATHERS="1", SOAP_TP_PIPELINE_MIN_TILES="120")
    chunks = module.GridEngine._column_chunks
    for cols, tiles, granule in [(8192, 1024, 128), (4096, 256, 128), (4096, 512, 256), (520, 40, 128), (130, 600, 128)]:
        parts = chunks(cols, tiles, granule)
        assert parts[0][0] == 0 and parts[-1][1] == cols
        assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
        assert all(start % granule == 0 for start, _ in parts)
        assert 1 <= len(parts) <= 4
        assert len(parts) <= max(1, tiles // 120)
    assert len(chunks(8192, 1024, 128)) == 4 and len(chunks(4096, 256, 128)) == 2 and len(chunks(520, 40, 128)) == 1


def test_column_chunks_off_by_default(monkeypatch):
    monkeypatch.delenv("SOAP_TP_PIPELINE_GATHERS", raising=False)
    module = _distributed(monkeypatch)
    assert module.GridEngine._column_chunks(8192, 1024, 128) == [(0, 8192)]


def test_leaders_are_spread_over_the_ranks(monkeypatch):
    module = _distributed(monkeypatch)
    assert [module._leader_of(job, 2, 8) for job in range(2)] == [0, 4]
    assert [module._leader_of(job, 2, 2) for job in range(2)] == [0, 1]
    assert [module._leader_of(job, 2, 1) for job in range(2)] == [0, 0]
    assert [module._leader_of(job, 4, 8) for job in range(4)] == [0, 2, 4, 6]


def test_row_sharded_gram_updates_validate_their_arguments():
    from soap_tp_b200.ops import gram_1d

    with pytest.raises(ValueError):
        gram_1d.update_left_preconditioner_from_col_shards(torch.zeros(4, 2), None, 0.5)   # no process group

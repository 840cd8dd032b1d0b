"""Closed-form block-cyclic math against brute-force enumeration."""
import itertools

import pytest
import torch

from soap_tp_b200 import layout


def brute_indices(size, nb, p, P):
    return [g for g in range(size) if (g // nb) % P == p]


@pytest.mark.parametrize("size", [0, 1, 7, 8, 13, 20, 69])
@pytest.mark.parametrize("nb", [1, 2, 3, 5, 8, 16])
@pytest.mark.parametrize("P", [1, 2, 3, 4])
def test_owned_indices_and_numroc(size, nb, P):
    total = 0
    for p in range(P):
        expected = brute_indices(size, nb, p, P)
        assert layout.numroc(size, nb, p, P) == len(expected)
        assert layout.owned_indices(size, nb, p, P).tolist() == expected
        assert list(layout.block_cyclic_indices(size, nb, p, P)) == expected
        if expected:
            owner, local = layout.global_to_local(torch.tensor(expected), nb, P)
            assert owner.tolist() == [p] * len(expected)
            assert local.tolist() == list(range(len(expected)))
        total += len(expected)
    assert total == size


def test_local_shape_and_owner():
    grid = (2, 3)
    shape = (13, 20)
    counted = [[0, 0] for _ in range(6)]
    for rank in range(6):
        lr, lc = layout.local_2d_block_cyclic_shape(shape, 4, grid, rank)
        pr, pc = divmod(rank, 3)
        assert lr == len(brute_indices(13, 4, pr, 2))
        assert lc == len(brute_indices(20, 4, pc, 3))
    assert layout.block_cyclic_owner_rank(3, 4, grid) == (3 % 2) * 3 + 4 % 3


def test_tile_views_cover_owned_tiles():
    grid = (2, 2)
    shape = (9, 13)
    nb = 4
    full = torch.arange(9 * 13, dtype=torch.float32).reshape(shape)
    seen = set()
    for rank in range(4):
        pr, pc = divmod(rank, 2)
        ri = layout.owned_indices(9, nb, pr, 2)
        ci = layout.owned_indices(13, nb, pc, 2)
        local = layout.empty_2d_block_cyclic_like_shape(len(ri), len(ci))
        local[: len(ri), : len(ci)] = full[ri[:, None], ci]
        assert local.stride(0) == 1
        views = layout.block_cyclic_tile_views(local, shape, nb, grid, rank)
        for (bi, bj), view in views.items():
            assert layout.block_cyclic_owner_rank(bi, bj, grid) == rank
            r0, r1 = layout.block_bounds(bi, nb, 9)
            c0, c1 = layout.block_bounds(bj, nb, 13)
            assert torch.equal(view, full[r0:r1, c0:c1])
            seen.add((bi, bj))
        lower = layout.block_cyclic_tile_views(local, shape, nb, grid, rank, mode="lower")
        assert all(bi >= bj for bi, bj in lower)
    assert seen == set(itertools.product(range(3), range(4)))


def test_validation_errors():
    with pytest.raises(ValueError):
        layout.validate_process_grid((2, 2), 3)
    with pytest.raises(ValueError):
        layout.numroc(4, 0, 0, 1)
    with pytest.raises(ValueError):
        layout.validate_2d_block_cyclic_buffer("m", torch.zeros(4, 4), (4, 4), 2, (1, 1), 0)
    ok = torch.zeros(4, 4).T
    assert layout.validate_2d_block_cyclic_buffer("m", ok, (4, 4), 2, (1, 1), 0) == (4, 4)
    with pytest.raises(ValueError):
        layout.validate_2d_block_cyclic_buffer("m", torch.zeros(3, 3).T, (4, 4), 2, (1, 1), 0)
    assert layout.most_square_grid(8) == (2, 4)
    assert layout.most_square_grid(4) == (2, 2)
    assert layout.most_square_grid(1) == (1, 1)
    with pytest.raises(ValueError):
        layout.tp_shard_shape((10, 8), 0, 4)

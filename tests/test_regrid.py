"""Checkpoint conversion between process grids and block sizes (``soap_tp_b200.utils.regrid``)."""
import io

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


def test_pack_unpack_round_trip_between_grids():
    from soap_tp_b200.utils.regrid import pack_dense, unpack_dense

    dense = torch.arange(13 * 9, dtype=torch.float32).reshape(13, 9)
    for grid, nb in (((2, 2), 2), ((1, 4), 3), ((4, 2), 128), ((2, 4), 1)):
        parts = pack_dense(dense, nb, grid)
        assert all(part.stride(0) == 1 for part in parts)
        assert torch.equal(unpack_dense(parts, (13, 9), nb, grid), dense)
    with pytest.raises(ValueError):
        unpack_dense(pack_dense(dense, 2, (2, 2)), (13, 9), 3, (2, 2))


def _optimizers(rank, world, grid, block_size):
    from soap_tp_b200 import SoapTP

    torch.manual_seed(0)
    full = torch.randn(12, 8)
    shard = torch.nn.Parameter(full.chunk(world, dim=0)[rank].clone())
    shard.tp_shard_dim, shard.tp_global_shape = 0, (12, 8)
    vector = torch.nn.Parameter(torch.randn(8))
    opt = SoapTP([shard, vector], lr=0.1, betas=(0.8, 0.9), shampoo_beta=0.75, eps=1e-6, weight_decay=0.0,
                 precondition_frequency=3, block_size=block_size, basis_implementation="eigh", process_grid_shape=grid)
    return opt, shard, vector


def _step(opt, shard, vector, rank, world, seed):
    g = torch.Generator().manual_seed(seed)
    shard.grad = torch.randn(12, 8, generator=g).chunk(world, dim=0)[rank].clone()
    vector.grad = torch.randn(8, generator=g)
    opt.step()


def _regrid_case(rank, world):
    from soap_tp_b200.utils.regrid import regrid_state_dicts

    opt, shard, vector = _optimizers(rank, world, (2, 2), 2)
    for it in range(4):
        _step(opt, shard, vector, rank, world, 70 + it)
    buffer = io.BytesIO()
    torch.save(opt.state_dict(), buffer)
    gathered = [None] * world
    dist.all_gather_object(gathered, buffer.getvalue())
    state_dicts = [torch.load(io.BytesIO(blob), weights_only=False) for blob in gathered]
    converted = regrid_state_dicts(state_dicts, (4, 1), new_block_size=3)
    assert converted[rank]["soap_tp_layout"][0] == dict(global_shape=[12, 8], shard_dim=0, block_size=3, grid=[4, 1])
    opt2, shard2, vector2 = _optimizers(rank, world, (4, 1), 3)
    shard2.data.copy_(shard.data); vector2.data.copy_(vector.data)
    opt2.load_state_dict(converted[rank])
    assert opt2.state[shard2]["step"] == opt.state[shard]["step"]
    for it in range(4):                       # crosses a refresh (precondition_frequency 3)
        _step(opt, shard, vector, rank, world, 90 + it)
        _step(opt2, shard2, vector2, rank, world, 90 + it)
        assert float((shard.data - shard2.data).norm() / shard.data.norm()) < 2e-5, it
        assert torch.equal(vector.data, vector2.data)
    # a new world size: packed state converts, per-shard state (the vector's AdamW moments) has to be dropped explicitly
    with pytest.raises(ValueError):
        regrid_state_dicts(state_dicts, (1, 2))
    halved = regrid_state_dicts(state_dicts, (1, 2), drop_other_state=True)
    assert len(halved) == 2 and set(halved[0]["state"]) == {0}
    assert halved[1]["state"][0]["momentum"].shape == (12, 4)


def test_regrid_checkpoint_and_continue():
    run_distributed(_regrid_case, 4)

"""``SoapTP`` optimizer wrapper and the tensor-parallel Llama model on CPU ranks (gloo)."""
import io

import pytest
import torch
import torch.distributed as dist

from distributed_helpers import run_distributed


def _optimizer_case(rank, world):
    from soap_tp_b200 import SoapTP
    from soap_tp_b200.utils.dense_soap import DenseSOAP, relative_l2

    torch.manual_seed(0)
    full = torch.randn(12, 8)
    # a row-sharded (column-parallel-layer) weight, a replicated matrix, a vector
    shard = torch.nn.Parameter(full.chunk(world, dim=0)[rank].clone())
    shard.tp_shard_dim, shard.tp_global_shape = 0, (12, 8)
    replicated = torch.nn.Parameter(torch.randn(8, 8))
    vector = torch.nn.Parameter(torch.randn(8))
    opt = SoapTP([shard, replicated, vector], lr=0.1, betas=(0.8, 0.9), shampoo_beta=0.75, eps=1e-6,
                 weight_decay=0.0, precondition_frequency=2, block_size=2, basis_implementation="eigh")
    oracle = DenseSOAP((12, 8), beta1=0.8, beta2=0.9, preconditioner_beta=0.75, eps=1e-6, basis_refresh_interval=2)
    expected = full.clone().double()
    for it in range(6):
        g = torch.Generator().manual_seed(50 + it)
        G = torch.randn(12, 8, generator=g)
        shard.grad = G.chunk(world, dim=0)[rank].clone()
        replicated.grad = torch.randn(8, 8, generator=g)
        vector.grad = torch.randn(8, generator=g)
        opt.step()
        expected -= 0.1 * oracle.step(G).double()
        parts = [torch.empty_like(shard.data) for _ in range(world)]
        dist.all_gather(parts, shard.data.contiguous())
        assert relative_l2(torch.cat(parts, 0), expected) < 1e-5
    # replicated parameter stays identical on all ranks
    copies = [torch.empty_like(replicated.data) for _ in range(world)]
    dist.all_gather(copies, replicated.data.contiguous())
    assert all(torch.equal(copies[0], c) for c in copies)
    assert set(opt.state[shard]) >= {"left_basis", "momentum", "variance", "step"} and "exp_avg" in opt.state[vector]

    # checkpoint round trip: same next update from a fresh optimizer that loaded the state
    buffer = io.BytesIO()
    torch.save(opt.state_dict(), buffer)
    buffer.seek(0)
    shard2 = torch.nn.Parameter(shard.data.clone()); shard2.tp_shard_dim, shard2.tp_global_shape = 0, (12, 8)
    rep2, vec2 = torch.nn.Parameter(replicated.data.clone()), torch.nn.Parameter(vector.data.clone())
    opt2 = SoapTP([shard2, rep2, vec2], lr=0.1, betas=(0.8, 0.9), shampoo_beta=0.75, eps=1e-6, weight_decay=0.0,
                  precondition_frequency=2, block_size=2, basis_implementation="eigh")
    opt2.load_state_dict(torch.load(buffer, weights_only=False))
    assert opt2.state[shard2]["momentum"].stride(0) == 1 and opt2.state[shard2]["momentum"].dtype == torch.float32
    g = torch.Generator().manual_seed(99)
    G = torch.randn(12, 8, generator=g)
    for o, ps in ((opt, (shard, replicated, vector)), (opt2, (shard2, rep2, vec2))):
        ps[0].grad = G.chunk(world, dim=0)[rank].clone()
        ps[1].grad = torch.ones(8, 8)
        ps[2].grad = torch.ones(8)
        o.step()
    assert torch.equal(shard.data, shard2.data) and torch.equal(replicated.data, rep2.data)
    assert torch.equal(vector.data, vec2.data)
    bad = SoapTP([shard2, rep2, vec2], block_size=4, basis_implementation="eigh")
    try:
        buffer.seek(0)
        bad.load_state_dict(torch.load(buffer, weights_only=False))
    except ValueError:
        pass
    else:
        raise AssertionError("a checkpoint written for another block size was accepted")


def _model_case(rank, world):
    from soap_tp_b200.models.llama_tp import LlamaConfig, LlamaTP
    from soap_tp_b200.train import parse_args, train

    cfg = LlamaConfig.tiny()
    model = LlamaTP(cfg, dtype=torch.float32, device="cpu", seed=3)
    for p in model.parameters():
        if p.ndim == 2:
            assert p.tp_shard_dim in (0, 1) and len(p.tp_global_shape) == 2
    tokens = torch.randint(0, cfg.vocab_size, (2, 9), generator=torch.Generator().manual_seed(1))
    loss = model(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    # the loss is the full-vocabulary cross entropy: identical on every rank, near log(vocab) at init
    values = [torch.zeros(1) for _ in range(world)]
    dist.all_gather(values, loss.detach().reshape(1))
    assert all(torch.allclose(values[0], v) for v in values)
    assert abs(float(loss) - torch.log(torch.tensor(float(cfg.vocab_size)))) < 0.5
    # gather the sharded logits and compare the parallel cross entropy with the dense one
    with torch.no_grad():
        logits = model(tokens[:, :-1])
        parts = [torch.empty_like(logits) for _ in range(world)]
        dist.all_gather(parts, logits.contiguous())
        dense = torch.nn.functional.cross_entropy(torch.cat(parts, -1).flatten(0, 1), tokens[:, 1:].flatten())
    assert torch.allclose(dense, loss.detach(), atol=1e-5)
    summary = train(parse_args(["--preset", "tiny", "--device", "cpu", "--steps", "4", "--global-batch", "2",
                                "--block-size", "8", "--precondition-frequency", "2", "--basis-implementation", "eigh",
                                "--lr", "1e-2"]))
    assert all(l == l for l in summary["losses"]) and summary["losses"][-1] < summary["losses"][0] + 0.1


def test_soap_tp_optimizer_two_ranks():
    run_distributed(_optimizer_case, 2)


def test_llama_tp_two_ranks():
    run_distributed(_model_case, 2)


def _one_sided_case(rank, world):
    """A row-sharded matrix whose sharded side is above ``max_precond_dim``: ``SoapTP`` preconditions the other
    side only.  Float64 restatement of one-sided SOAP (identity basis on the long side) on every rank."""
    import torch.distributed as dist

    from soap_tp_b200.optim import SoapTP

    device = torch.device("cuda", rank % torch.cuda.device_count())
    rows_local, h, steps, interval = 24, 16, 6, 2
    beta, b1, b2, eps = 0.9, 0.8, 0.9, 1e-8
    weight = torch.nn.Parameter(torch.zeros(rows_local, h, device=device))
    weight.tp_shard_dim, weight.tp_global_shape = 0, (rows_local * world, h)
    optimizer = SoapTP([weight], lr=1.0, weight_decay=0.0, betas=(b1, b2), shampoo_beta=beta, eps=eps,
                       precondition_frequency=interval, max_precond_dim=20, basis_implementation="householder")
    assert optimizer._plan(weight, optimizer.param_groups[0]).get("one_sided")
    full = lambda t: torch.randn(rows_local * world, h, generator=torch.Generator().manual_seed(40 + t), dtype=torch.float64)
    R = Q = M = V = None
    expected = torch.zeros(rows_local * world, h, dtype=torch.float64)
    for t in range(steps):
        G = full(t)
        weight.grad = G[rank * rows_local:(rank + 1) * rows_local].float().to(device)
        optimizer.step()
        if t == 0:
            R = (1 - beta) * G.T @ G
            Q = torch.linalg.eigh(R)[1].flip(1)
            M, V = torch.zeros_like(G), torch.zeros_like(G)
            continue
        Y = G @ Q
        M = b1 * M + (1 - b1) * Y
        V = b2 * V + (1 - b2) * Y * Y
        U = (M / (1 - b1**t)) / ((V.sqrt() + eps) / (1 - b2**t) ** 0.5)
        expected -= U @ Q.T
        R = beta * R + (1 - beta) * G.T @ G
        if t % interval == 0:
            Mp = M @ Q.T
            order = torch.argsort(((Q * (R @ Q)).sum(0)), descending=True, stable=True)
            Qn = torch.linalg.qr((R @ Q)[:, order])[0]
            M, V, Q = Mp @ Qn, V[:, order], Qn
    got = weight.detach().double().cpu()
    want = expected[rank * rows_local:(rank + 1) * rows_local]
    error = float((got - want).norm() / want.norm())
    assert error < 2e-4, error
    # checkpoint round trip keeps the fp32 buffers bit for bit
    saved = optimizer.state_dict()
    fresh = SoapTP([weight], lr=1.0, weight_decay=0.0, max_precond_dim=20)
    fresh.load_state_dict(saved)
    for name in ("right_preconditioner", "right_basis", "momentum", "variance"):
        assert torch.equal(fresh.state[weight][name], optimizer.state[weight][name])
    dist.barrier()


@pytest.mark.gpu
def test_one_sided_soap_for_a_long_sharded_side():
    run_distributed(_one_sided_case, 1)
    run_distributed(_one_sided_case, 2)

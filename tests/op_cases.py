"""Rank-side bodies of the distributed op tests.

Each function runs on every rank of a real process group and checks a packed-layout op against
a dense single-process restatement computed from the same seeded inputs (the exact-input stage
oracle).  ``device_kind`` is ``"cpu"`` or ``"cuda"``; on CUDA several ranks may share one GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from soap_tp_b200 import layout, ops, soap_step
from soap_tp_b200.ops.basis import qr_call_count
from soap_tp_b200.utils.dense_soap import DenseSOAP, align_column_signs, relative_l2


def dev(device_kind: str, rank: int) -> torch.device:
    if device_kind == "cuda":
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


def pack(full: torch.Tensor, nb: int, grid, rank: int, device) -> torch.Tensor:
    pr, pc = divmod(rank, grid[1])
    ri = layout.owned_indices(full.shape[0], nb, pr, grid[0])
    ci = layout.owned_indices(full.shape[1], nb, pc, grid[1])
    local = layout.empty_2d_block_cyclic_like_shape(len(ri), len(ci), device=device)
    if len(ri) and len(ci):
        local[: len(ri), : len(ci)] = full[ri[:, None], ci].to(device)
    return local


def unpack(local: torch.Tensor, shape, nb: int, grid) -> torch.Tensor:
    """Dense copy on every rank (CPU)."""
    from soap_tp_b200.ops import _hostpath as host

    return host.gather_block_cyclic(local.detach().cpu(), tuple(shape), nb, grid)


def seeded(shape, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(shape, generator=g) * scale


def spd(n, seed):
    a = seeded((n, n), seed)
    return a @ a.T / n + torch.diag(torch.linspace(1.0, 3.0, n))


def orthogonal(n, seed):
    q, _ = torch.linalg.qr(seeded((n, n), seed).double())
    return q.float()


def case_redistribute(rank, world, device_kind, shape, nb, grid, shard_dim):
    device = dev(device_kind, rank)
    full = seeded(shape, 1)
    shard = full.chunk(world, dim=shard_dim)[rank].contiguous().to(device)
    packed = ops.redistribute_tp_shard_to_2d_block_cyclic(shard, shape, nb, grid, shard_dim=shard_dim)
    assert packed.stride(0) == 1
    expected = pack(full, nb, grid, rank, device)
    lr, lc = layout.local_2d_block_cyclic_shape(shape, nb, grid, rank)
    assert torch.equal(packed[:lr, :lc], expected[:lr, :lc])
    back = ops.redistribute_2d_block_cyclic_to_tp_shard(packed, shape, nb, grid, shard_dim=shard_dim)
    assert back.is_contiguous() and torch.equal(back, shard)


def case_gram(rank, world, device_kind, shape, nb, grid, shard_dim, beta):
    device = dev(device_kind, rank)
    full = seeded(shape, 2)
    shard = torch.tensor_split(full, world, dim=shard_dim)[rank].contiguous().to(device)
    rows, cols = shape
    L0, R0 = spd(rows, 3), spd(cols, 4)
    L = pack(L0, nb, grid, rank, device)
    R = pack(R0, nb, grid, rank, device)
    out = ops.update_left_preconditioner_2d_block_cyclic_(shard, L, beta, nb, grid, shard_dim=shard_dim)
    assert out is L
    ops.update_right_preconditioner_2d_block_cyclic_(shard, R, beta, nb, grid, shard_dim=shard_dim)
    fd = full.double()
    eL = beta * L0.double() + (1 - beta) * fd @ fd.T
    eR = beta * R0.double() + (1 - beta) * fd.T @ fd
    gL, gR = unpack(L, (rows, rows), nb, grid), unpack(R, (cols, cols), nb, grid)
    assert relative_l2(gL, eL) <= 1e-5, relative_l2(gL, eL)
    assert relative_l2(gR, eR) <= 1e-5, relative_l2(gR, eR)
    # elementwise bound of the reference's tests, scaled by the magnitude of the entries
    torch.testing.assert_close(gL.double(), eL, rtol=1e-5, atol=1e-5 * max(1.0, float(eL.abs().max())))
    torch.testing.assert_close(gR.double(), eR, rtol=1e-5, atol=1e-5 * max(1.0, float(eR.abs().max())))


def case_rotate(rank, world, device_kind, shape, nb, grid):
    device = dev(device_kind, rank)
    rows, cols = shape
    X0, QL0, QR0 = seeded(shape, 5), orthogonal(rows, 6), orthogonal(cols, 7)
    QL, QR = pack(QL0, nb, grid, rank, device), pack(QR0, nb, grid, rank, device)
    for direction in ("forward", "backward"):
        X = pack(X0, nb, grid, rank, device)
        out = ops.rotate_2d_block_cyclic_(X, QL, QR, shape, nb, grid, direction=direction)
        assert out is X
        if direction == "forward":
            expected = QL0.double().T @ X0.double() @ QR0.double()
        else:
            expected = QL0.double() @ X0.double() @ QR0.double().T
        got = unpack(X, shape, nb, grid)
        assert relative_l2(got, expected) <= 1e-5, (direction, relative_l2(got, expected))
        torch.testing.assert_close(got.double(), expected, rtol=2e-4, atol=2e-4)


def case_permute(rank, world, device_kind, shape, nb, grid):
    device = dev(device_kind, rank)
    rows, cols = shape
    X0 = seeded(shape, 8)
    g = torch.Generator().manual_seed(9)
    ro, co = torch.randperm(rows, generator=g), torch.randperm(cols, generator=g)
    X = pack(X0, nb, grid, rank, device)
    ops.permute_2d_block_cyclic_(X, shape, ro.tolist(), co.to(device), nb, grid)
    assert torch.equal(unpack(X, shape, nb, grid), X0[ro][:, co])
    try:
        ops.permute_2d_block_cyclic_(X, shape, [0] * rows, co, nb, grid)
    except ValueError:
        pass
    else:
        raise AssertionError("invalid permutation accepted")


def case_power_iteration_qr(rank, world, device_kind, n, nb, grid):
    device = dev(device_kind, rank)
    P0 = spd(n, 10)
    Q0 = orthogonal(n, 11)
    P, Q = pack(P0, nb, grid, rank, device), pack(Q0, nb, grid, rank, device)
    work = pack(torch.zeros(n, n), nb, grid, rank, device)
    before = qr_call_count()
    order = ops.power_iteration_qr_2d_block_cyclic_(P, Q, work, n, nb, grid)
    assert qr_call_count() == before + 1
    W = P0.double() @ Q0.double()
    estimates = (Q0.double() * W).sum(0)
    expected_order = torch.argsort(estimates, descending=True, stable=True)
    assert order.dtype == torch.int64 and torch.equal(order.cpu(), expected_order)
    eQ, _ = torch.linalg.qr(W[:, expected_order])
    got = unpack(Q, (n, n), nb, grid).double()
    got = align_column_signs(got, eQ)
    assert relative_l2(got, eQ) <= 1e-5, relative_l2(got, eQ)
    torch.testing.assert_close(got, eQ, rtol=3e-3, atol=3e-3)
    torch.testing.assert_close(got.T @ got, torch.eye(n, dtype=torch.float64), rtol=1e-4, atol=1e-4)


def case_estimated_order_and_qr(rank, world, device_kind, n, nb, grid):
    device = dev(device_kind, rank)
    P0, Q0 = spd(n, 12), orthogonal(n, 13)
    P, Q = pack(P0, nb, grid, rank, device), pack(Q0, nb, grid, rank, device)
    work = pack(torch.zeros(n, n), nb, grid, rank, device)
    order = ops.estimated_eigenvalue_order_2d_block_cyclic_(P, Q, work, n, nb, grid)
    W = P0.double() @ Q0.double()
    assert relative_l2(unpack(work, (n, n), nb, grid), W) <= 1e-5
    assert torch.equal(order.cpu(), torch.argsort((Q0.double() * W).sum(0), descending=True, stable=True))
    out = pack(torch.zeros(n, n), nb, grid, rank, device)
    ops.qr_2d_block_cyclic_(work, out, n, nb, grid)
    eQ, _ = torch.linalg.qr(W)
    got = align_column_signs(unpack(out, (n, n), nb, grid).double(), eQ)
    assert relative_l2(got, eQ) <= 1e-5, relative_l2(got, eQ)


def case_initialize_basis(rank, world, device_kind, gshape, side, nb, grid, implementation):
    """Eigenpairs of a (possibly rank-deficient) Gram matrix: eigenvalues, orthogonality,
    residual, sign-aligned vectors for the non-zero spectrum and projector for the null space
    (the recipe of the reference's ``tests/unit/test_elpa_bindings.py:262-501``)."""
    device = dev(device_kind, rank)
    G = seeded(gshape, 14).double()
    P0 = (G @ G.T if side == "left" else G.T @ G)
    n = P0.shape[0]
    P = pack(P0.float(), nb, grid, rank, device)
    Q = pack(torch.zeros(n, n), nb, grid, rank, device)
    work = pack(torch.zeros(n, n), nb, grid, rank, device)
    values = torch.empty(n, dtype=torch.float32, device=device)
    P_before = P.clone()
    out = ops.initialize_basis_2d_block_cyclic_(P, Q, work, values, n, nb, grid, implementation=implementation)
    assert out is Q and torch.equal(P, P_before)
    ev, evec = torch.linalg.eigh(P0)
    ev, evec = ev.flip(0), evec.flip(1)
    scale = float(ev.abs().max())
    got_values = values.cpu().double()
    if dist.get_world_size() > 1:
        reference = got_values.clone()
        dist.broadcast(reference, src=0)
        assert torch.equal(reference, got_values), "eigenvalues differ across ranks"
    Qf = unpack(Q, (n, n), nb, grid).double()
    tol = 2e-4
    assert float((got_values - ev).abs().max()) <= tol * scale
    assert float((Qf.T @ Qf - torch.eye(n, dtype=torch.float64)).abs().max()) <= tol
    assert float((P0 @ Qf - Qf * got_values).abs().max()) <= tol * scale
    nonzero = ev > 1e-6 * scale
    k = int(nonzero.sum())
    gaps_ok = k > 0 and float((ev[:k][:-1] - ev[:k][1:]).min() if k > 1 else 1.0) > 1e-3 * scale
    if gaps_ok:
        aligned = align_column_signs(Qf[:, :k], evec[:, :k])
        assert float((aligned - evec[:, :k]).abs().max()) <= 5e-3
    if k < n:
        proj_got = Qf[:, k:] @ Qf[:, k:].T
        proj_ref = evec[:, k:] @ evec[:, k:].T
        assert float((proj_got - proj_ref).abs().max()) <= 5e-3


def case_refresh(rank, world, device_kind, shape, nb, grid):
    device = dev(device_kind, rank)
    rows, cols = shape
    L0, R0 = spd(rows, 20), spd(cols, 21)
    QL0, QR0 = orthogonal(rows, 22), orthogonal(cols, 23)
    M0, V0 = seeded(shape, 24), seeded(shape, 25).abs()
    buf = lambda t: pack(t, nb, grid, rank, device)
    M, V, L, R, QL, QR = buf(M0), buf(V0), buf(L0), buf(R0), buf(QL0), buf(QR0)
    WL, WR = buf(torch.zeros(rows, rows)), buf(torch.zeros(cols, cols))
    lo, ro = ops.refresh_bases_and_transport_optimizer_state_(M, V, L, R, QL, QR, WL, WR, shape, nb, grid)
    d = lambda t: t.double()
    Mp = d(QL0) @ d(M0) @ d(QR0).T
    elo = torch.argsort((d(QL0) * (d(L0) @ d(QL0))).sum(0), descending=True, stable=True)
    ero = torch.argsort((d(QR0) * (d(R0) @ d(QR0))).sum(0), descending=True, stable=True)
    assert torch.equal(lo.cpu(), elo) and torch.equal(ro.cpu(), ero)
    nQL, _ = torch.linalg.qr((d(L0) @ d(QL0))[:, elo])
    nQR, _ = torch.linalg.qr((d(R0) @ d(QR0))[:, ero])
    gQL = unpack(QL, (rows, rows), nb, grid).double()
    gQR = unpack(QR, (cols, cols), nb, grid).double()
    sL = torch.sign((gQL * nQL).sum(0)); sL[sL == 0] = 1
    sR = torch.sign((gQR * nQR).sum(0)); sR[sR == 0] = 1
    assert relative_l2(gQL * sL, nQL) <= 1e-5
    assert relative_l2(gQR * sR, nQR) <= 1e-5
    torch.testing.assert_close(gQL.T @ gQL, torch.eye(rows, dtype=torch.float64), rtol=1e-4, atol=1e-4)
    eM = nQL.T @ Mp @ nQR
    gM = unpack(M, shape, nb, grid).double() * sL[:, None] * sR[None, :]
    assert relative_l2(gM, eM) <= 2e-5, relative_l2(gM, eM)
    assert torch.equal(unpack(V, shape, nb, grid), V0[elo][:, ero])


def case_soap_trajectory(rank, world, device_kind, shape, nb, grid, shard_dim, steps, interval,
                         betas, pbeta, eps, tolerance, implementation="eigh", grad_scale=2.0, noise=0.0):
    """``soap_step`` against the dense single-process SOAP (the end-to-end oracle).

    Eigenvectors of a Gram matrix of Gaussian gradients are ill-conditioned and Adam is not
    continuous at zero, so two correct fp32 implementations agree only down to the oracle's own
    sensitivity.  With ``noise > 0`` a second oracle consumes gradients perturbed by
    ``noise * N(0, 1)`` relative (the size of one GEMM's rounding error) and the bound becomes
    ``max(tolerance, 3 * ||oracle - perturbed oracle|| / ||oracle||)`` per step.
    """
    device = dev(device_kind, rank)
    make_oracle = lambda: DenseSOAP(shape, beta1=betas[0], beta2=betas[1], preconditioner_beta=pbeta, eps=eps,
                                    basis_refresh_interval=interval)
    oracle = make_oracle()
    shadow = make_oracle() if noise > 0 else None
    param_shadow = torch.zeros(shape, dtype=torch.float64)
    state = {}
    param_ref = torch.zeros(shape, dtype=torch.float64)
    param_tp = torch.zeros(shape, dtype=torch.float64)
    qr_before = qr_call_count()
    for it in range(steps):
        G = seeded(shape, 100 + it, grad_scale)
        shard = G.chunk(world, dim=shard_dim)[rank].contiguous().to(device)
        update = soap_step(
            shard, state, global_shape=shape, shard_dim=shard_dim, block_size=nb,
            process_grid_shape=grid, preconditioner_beta=pbeta, beta1=betas[0], beta2=betas[1],
            eps=eps, basis_refresh_interval=interval, basis_implementation=implementation,
        )
        assert update.dtype == torch.float32 and update.shape == shard.shape
        parts = [torch.empty_like(update.cpu()) for _ in range(world)]
        dist.all_gather(parts, update.cpu().contiguous())
        full = torch.cat(parts, dim=shard_dim)
        expected = oracle.step(G)
        bound_u = bound_p = tolerance
        if shadow is not None:
            perturbed = shadow.step(G * (1.0 + noise * seeded(shape, 900 + it)))
            if it > 0:
                param_shadow -= perturbed.double()
                bound_u = max(tolerance, 3.0 * relative_l2(perturbed, expected))
                bound_p = max(tolerance, 3.0 * relative_l2(param_shadow, param_ref - expected.double()))
        if it == 0:
            assert float(full.abs().max()) == 0.0 and state["step"] == 0
            continue
        assert state["step"] == it
        param_ref -= expected.double()
        param_tp -= full.double()
        err_u, err_p = relative_l2(full, expected), relative_l2(param_tp, param_ref)
        if rank == 0:
            print(f"{shape[0]}x{shape[1]} dim{shard_dim} basis={implementation} | step {it} | "
                  f"SOAP relL2={err_u:.2e} | PARAM relL2={err_p:.2e}", flush=True)
        assert err_u <= bound_u, (it, err_u, bound_u)
        assert err_p <= bound_p, (it, err_p, bound_p)
    assert qr_call_count() - qr_before == 2 * ((steps - 1) // interval)
    for name in ("left_preconditioner", "right_preconditioner", "left_basis", "right_basis",
                 "left_work", "right_work", "momentum", "variance"):
        assert state[name].dtype == torch.float32 and state[name].stride(0) == 1


def case_soap_shared_basis(rank, world, device_kind, shape, nb, grid, shard_dim, steps, tolerance):
    """``soap_step`` against the dense oracle with the ORACLE's eigenbases injected after the warm-up call.

    With both implementations rotating into the same bases, nothing ill-conditioned separates them until the first
    refresh: the bound is a plain ``tolerance`` that does not depend on the eigensolver under test or on a measured
    noise floor.  The reference compares whole trajectories the same way (``tests/unit/test_soap.py:186-290``) but
    has no mode that shares the bases."""
    device = dev(device_kind, rank)
    betas, pbeta, eps = (0.9, 0.95), 0.9, 1e-8
    # float64 oracle: in float32 its own rounding (momentum and gradient are rotated by separate products there)
    # already moves the update by 1e-5 through the entries whose rotated gradient nearly vanishes
    oracle = DenseSOAP(shape, beta1=betas[0], beta2=betas[1], preconditioner_beta=pbeta, eps=eps,
                       basis_refresh_interval=steps + 1, dtype=torch.float64)
    state = {}
    param_ref = torch.zeros(shape, dtype=torch.float64)
    param_tp = torch.zeros(shape, dtype=torch.float64)
    for it in range(steps):
        G = seeded(shape, 300 + it, 2.0)
        shard = G.chunk(world, dim=shard_dim)[rank].contiguous().to(device)
        update = soap_step(shard, state, global_shape=shape, shard_dim=shard_dim, block_size=nb,
                           process_grid_shape=grid, preconditioner_beta=pbeta, beta1=betas[0], beta2=betas[1],
                           eps=eps, basis_refresh_interval=steps + 1, basis_implementation="eigh")
        expected = oracle.step(G)
        if it == 0:
            assert float(update.abs().max()) == 0.0
            oracle.QL, oracle.QR = oracle.QL.float().double(), oracle.QR.float().double()   # the very same numbers
            state["left_basis"].copy_(pack(oracle.QL.float(), nb, grid, rank, device))
            state["right_basis"].copy_(pack(oracle.QR.float(), nb, grid, rank, device))
            continue
        parts = [torch.empty_like(update.cpu()) for _ in range(world)]
        dist.all_gather(parts, update.cpu().contiguous())
        full = torch.cat(parts, dim=shard_dim)
        param_ref -= expected.double()
        param_tp -= full.double()
        err_u, err_p = relative_l2(full.double(), expected), relative_l2(param_tp, param_ref)
        if rank == 0:
            print(f"{shape[0]}x{shape[1]} dim{shard_dim} shared bases | step {it} | SOAP relL2={err_u:.2e} | "
                  f"PARAM relL2={err_p:.2e}", flush=True)
        assert err_u <= tolerance, (it, err_u)
        assert err_p <= tolerance, (it, err_p)
    for side, (P, Q) in (("left", (oracle.L, oracle.QL)), ("right", (oracle.R, oracle.QR))):
        got = unpack(state[f"{side}_preconditioner"], P.shape, nb, grid)
        assert relative_l2(got.double(), P) <= tolerance, side
        assert torch.equal(unpack(state[f"{side}_basis"], Q.shape, nb, grid), Q.float())   # untouched without a refresh


def case_batch(rank, world, device_kind, specs):
    """Run several cases in one process group (process start-up dominates tiny cases).
    ``specs`` is a list of ``(function name, args)``; failures name the failing spec."""
    for name, args in specs:
        try:
            globals()[name](rank, world, device_kind, *args)
        except Exception as error:  # re-raise with the spec for a readable report
            raise AssertionError(f"{name}{args}: {type(error).__name__}: {error}") from error
        dist.barrier()


def case_gram_1d(rank, world, device_kind, shape, beta):
    """Row-sharded Gram updates for column-sharded gradients against the dense products."""
    from soap_tp_b200.ops.gram_1d import (update_left_preconditioner_from_col_shards,
                                          update_right_preconditioner_from_col_shards)

    device = dev(device_kind, rank)
    rows, cols = shape
    full = seeded(shape, 21)
    shard = full.chunk(world, dim=1)[rank].contiguous().to(device)
    L0, R0 = spd(rows, 22), spd(cols, 23)
    rows_here, cols_here = rows // world, cols // world
    L = L0[rank * rows_here:(rank + 1) * rows_here].clone().to(device)
    R = R0[rank * cols_here:(rank + 1) * cols_here].clone().to(device)
    out = update_left_preconditioner_from_col_shards(shard, L, beta)
    assert out is L
    update_right_preconditioner_from_col_shards(shard, R, beta)
    fd = full.double()
    eL = (beta * L0.double() + (1 - beta) * fd @ fd.T)[rank * rows_here:(rank + 1) * rows_here]
    eR = (beta * R0.double() + (1 - beta) * fd.T @ fd)[rank * cols_here:(rank + 1) * cols_here]
    assert relative_l2(L.cpu().double(), eL) < 1e-5
    assert relative_l2(R.cpu().double(), eR) < 1e-5
    fresh = update_left_preconditioner_from_col_shards(shard, None, 0.0)
    assert relative_l2(fresh.cpu().double(), (fd @ fd.T)[rank * rows_here:(rank + 1) * rows_here]) < 1e-5


def case_gram_1d_subgroups(rank, world, device_kind, shape, beta):
    """The 1-D Gram updates over a sub-group: two independent tensor-parallel groups of half the world."""
    from soap_tp_b200.ops.gram_1d import (update_left_preconditioner_from_col_shards,
                                          update_right_preconditioner_from_col_shards)

    assert world % 2 == 0
    half = world // 2
    groups = [dist.new_group(list(range(g * half, (g + 1) * half))) for g in range(2)]
    mine = rank // half
    group, local_rank = groups[mine], rank % half
    device = dev(device_kind, rank)
    rows, cols = shape
    full = seeded(shape, 31 + mine)                      # each group has its own gradient
    shard = full.chunk(half, dim=1)[local_rank].contiguous().to(device)
    rows_here, cols_here = rows // half, cols // half
    L = update_left_preconditioner_from_col_shards(shard, None, beta, TP_group=group)
    R = update_right_preconditioner_from_col_shards(shard, None, beta, TP_group=group)
    fd = full.double()
    eL = ((1 - beta) * fd @ fd.T)[local_rank * rows_here:(local_rank + 1) * rows_here]
    eR = ((1 - beta) * fd.T @ fd)[local_rank * cols_here:(local_rank + 1) * cols_here]
    assert L.shape == (rows_here, rows) and R.shape == (cols_here, cols)
    assert relative_l2(L.cpu().double(), eL) < 1e-5 and relative_l2(R.cpu().double(), eR) < 1e-5


def case_redistribute_permute_subgroups(rank, world, device_kind, shape, nb):
    """``group=`` of the redistributions and the permutation: two independent halves of the world, each a
    ``1 x half`` grid over its own process group with its own matrix
    (the reference plumbs ``group`` through exactly these ops, ``src/soap_tp/ops/optimizer.py:71,229,404``)."""
    assert world % 2 == 0
    half = world // 2
    groups = [dist.new_group(list(range(g * half, (g + 1) * half))) for g in range(2)]
    mine = rank // half
    group, local_rank = groups[mine], rank % half
    grid = (1, half)
    device = dev(device_kind, rank)
    rows, cols = shape
    full = seeded(shape, 41 + mine)
    for shard_dim in (0, 1):
        shard = full.chunk(half, dim=shard_dim)[local_rank].contiguous().to(device)
        packed = ops.redistribute_tp_shard_to_2d_block_cyclic(shard, shape, nb, grid, shard_dim=shard_dim, group=group)
        expected = pack(full, nb, grid, local_rank, device)
        lr, lc = layout.local_2d_block_cyclic_shape(shape, nb, grid, local_rank)
        assert torch.equal(packed[:lr, :lc], expected[:lr, :lc])
        back = ops.redistribute_2d_block_cyclic_to_tp_shard(packed, shape, nb, grid, shard_dim=shard_dim, group=group)
        assert torch.equal(back, shard)
    g = torch.Generator().manual_seed(50 + mine)
    ro, co = torch.randperm(rows, generator=g), torch.randperm(cols, generator=g)
    X = pack(full, nb, grid, local_rank, device)
    ops.permute_2d_block_cyclic_(X, shape, ro.to(device), co.to(device), nb, grid, group=group)
    lr, lc = layout.local_2d_block_cyclic_shape(shape, nb, grid, local_rank)
    want = pack(full[ro][:, co], nb, grid, local_rank, device)
    assert torch.equal(X[:lr, :lc], want[:lr, :lc])


def case_qr_properties(rank, world, device_kind, n, nb, grid, kind):
    """``qr_2d_block_cyclic_`` on inputs that stress the factorisation: several panels, ragged last panel,
    rank-deficient columns.  ``Q`` must be orthogonal and ``Q^T A`` upper triangular (the defining properties;
    the factor itself is not unique when ``A`` is singular)."""
    device = dev(device_kind, rank)
    A0 = seeded((n, n), 60)
    if kind == "rank_deficient":
        A0[:, n // 3] = A0[:, 1]                # a repeated column
        A0[:, n // 2] = 0.0                     # a zero column
        A0[:, -5:] = A0[:, :5] @ seeded((5, 5), 61)      # the last columns depend on the first
    elif kind == "graded":
        A0 = A0 * torch.logspace(0, -6, n)[None, :]
    A, Q = pack(A0, nb, grid, rank, device), pack(torch.zeros(n, n), nb, grid, rank, device)
    ops.qr_2d_block_cyclic_(A, Q, n, nb, grid)
    got = unpack(Q, (n, n), nb, grid).double()
    eye = torch.eye(n, dtype=torch.float64)
    assert float((got.T @ got - eye).abs().max()) <= 1e-4, float((got.T @ got - eye).abs().max())
    R = got.T @ A0.double()
    below = torch.tril(R, diagonal=-1)
    scale = float(A0.double().norm(dim=0).max())
    assert float(below.abs().max()) <= 2e-5 * scale * max(1.0, n ** 0.5 / 8), (float(below.abs().max()), scale)

"""``dist_gather`` (the kernel that carries every byte between ranks) against an index-level restatement.

The ranks' segments are emulated on ONE device: a peer table whose entries point at separate local buffers,
which is all the kernel sees of a peer.  Every configuration is run through the 16-byte kernels (where the
host-side conditions allow them) and through the element-wise kernel; both must reproduce
``out(i, j) = source(map_i(i), map_j(j))`` exactly (a gather moves bits; the hi/lo split is exact).
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _numroc(n, nb, p, P):
    full, rem = divmod(n, nb)
    count = (full // P) * nb
    extra = full % P
    return count + (nb if p < extra else rem if p == extra else 0)


def _make_source(dense, kind, nb, Pr, Pc, world, device):
    """Scatter ``dense`` into per-rank buffers; return (buffers, peer table)."""
    from soap_tp_b200.layout import owned_indices

    rows, cols = dense.shape
    buffers = []
    if kind == 0:
        for r in range(Pr * Pc):
            pr, pc = divmod(r, Pc)
            ri, ci = owned_indices(rows, nb, pr, Pr), owned_indices(cols, nb, pc, Pc)
            local = torch.zeros(max(1, len(ci)), max(1, len(ri)))
            if len(ri) and len(ci):
                local[: len(ci), : len(ri)] = dense[ri[:, None], ci].T
            buffers.append(local.contiguous().to(device))          # column-major, exact pitch
    elif kind == 1:
        buffers = [part.contiguous().to(device) for part in dense.chunk(world, dim=0)]
    else:
        buffers = [part.contiguous().to(device) for part in dense.chunk(world, dim=1)]
    table = torch.tensor([b.data_ptr() for b in buffers], dtype=torch.int64, device=device)
    return buffers, table


def _map(local_count, p, P, nb, offset, perm, local_offset):
    l = torch.arange(local_count) + local_offset
    g = ((l // nb) * P + p) * nb + l % nb if P > 1 else l.clone()
    g = g + offset
    return perm[g] if perm is not None else g


CASES = [
    # kind, shape, nb, (Pr, Pc), world, map_i (p, P, nb, offset, perm?, local_offset), map_j, transpose, planes
    (2, (512, 1024), 128, (2, 4), 8, (0, 1, 1, 0, False, 0), (1, 2, 128, 0, False, 0), False, True),   # gradient panel
    (2, (512, 1024), 128, (2, 4), 8, (0, 1, 1, 0, False, 0), (3, 4, 128, 0, False, 0), True, True),    # Gram, left
    (0, (640, 384), 64, (2, 2), 4, (0, 1, 1, 0, False, 0), (1, 2, 64, 0, False, 0), False, True),      # packed source
    (0, (640, 384), 64, (2, 2), 4, (0, 1, 1, 0, False, 0), (1, 2, 64, 0, False, 0), True, True),
    (0, (640, 384), 64, (2, 2), 4, (1, 2, 64, 0, False, 0), (0, 2, 64, 0, False, 0), False, False),    # packed -> packed
    (0, (300, 200), 64, (2, 2), 4, (0, 1, 1, 0, False, 0), (1, 2, 64, 0, False, 0), False, True),      # ragged sizes
    (0, (301, 203), 4, (2, 2), 4, (1, 2, 4, 0, False, 0), (1, 2, 4, 0, False, 0), True, True),         # odd local pitch
    (1, (512, 256), 128, (1, 1), 4, (0, 1, 1, 0, False, 0), (0, 1, 1, 0, False, 0), False, True),      # row shards
    (1, (512, 256), 128, (1, 1), 4, (0, 1, 1, 0, False, 0), (0, 1, 1, 0, False, 0), True, False),
    (0, (256, 256), 64, (2, 2), 4, (0, 1, 1, 0, True, 0), (1, 2, 64, 0, True, 0), False, True),        # permutations
    (0, (512, 512), 128, (2, 2), 4, (0, 1, 1, 0, False, 0), (1, 2, 128, 0, False, 128), False, True),  # a chunk
]


@pytest.mark.parametrize("case", CASES, ids=[f"case{i}" for i in range(len(CASES))])
def test_dist_gather_against_index_restatement(case):
    from soap_tp_b200.engine import kernels as k

    kind, shape, nb, (Pr, Pc), world, mi, mj, transpose, planes = case
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    g = torch.Generator().manual_seed(0)
    dense = torch.randn(shape, generator=g)
    buffers, table = _make_source(dense, kind, nb, Pr, Pc, world, device)
    src_rows, src_cols = shape
    first_extent = src_cols if transpose else src_rows      # map_i indexes source columns when transposed
    second_extent = src_rows if transpose else src_cols

    def build(spec, extent):
        p, P, mnb, offset, permuted, local_offset = spec
        perm = torch.randperm(extent, generator=g) if permuted else None
        count = (_numroc(extent, mnb, p, P) if P > 1 else extent) - local_offset
        return (p, P, mnb, offset, perm, local_offset), _map(count, p, P, mnb, offset, perm, local_offset), count

    spec_i, index_i, rows_out = build(mi, first_extent)
    spec_j, index_j, cols_out = build(mj, second_extent)
    expected = (dense.T if transpose else dense)[index_i[:, None], index_j]

    def run():
        perm_i = spec_i[4].to(device) if spec_i[4] is not None else None
        perm_j = spec_j[4].to(device) if spec_j[4] is not None else None
        if planes:
            out = k.Planes.empty(rows_out, cols_out, device)
            hi, lo, d_i, d_j = out.hi.data_ptr(), out.lo.data_ptr(), 1, out.ld
        else:
            out = torch.zeros(cols_out, rows_out, device=device).T
            hi, lo, d_i, d_j = out.data_ptr(), 0, 1, out.stride(1)
        k._C.dist_gather(table.data_ptr(), kind, src_rows, src_cols, nb, nb, Pr, Pc, world,
                         spec_i[0], spec_i[1], spec_i[2], spec_i[3], perm_i.data_ptr() if perm_i is not None else 0,
                         spec_j[0], spec_j[1], spec_j[2], spec_j[3], perm_j.data_ptr() if perm_j is not None else 0,
                         int(transpose), 0, spec_i[5], spec_j[5], hi, lo, d_i, d_j, rows_out, cols_out,
                         torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return (out.dense() if planes else out).cpu()

    fast = run()
    k._C.force_scalar_gather(True)
    try:
        slow = run()
    finally:
        k._C.force_scalar_gather(False)
    assert torch.equal(slow, expected)
    assert torch.equal(fast, expected)
    # a row-major output (tensor-parallel shard) takes the same kernels with the roles of i and j swapped
    if not planes:
        out = torch.zeros(rows_out, cols_out, device=device)
        k._C.dist_gather(table.data_ptr(), kind, src_rows, src_cols, nb, nb, Pr, Pc, world,
                         spec_i[0], spec_i[1], spec_i[2], spec_i[3], 0, spec_j[0], spec_j[1], spec_j[2], spec_j[3], 0,
                         int(transpose), 0, spec_i[5], spec_j[5], out.data_ptr(), 0, out.stride(0), 1, rows_out, cols_out,
                         torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert torch.equal(out.cpu(), expected)


@pytest.mark.parametrize("transpose", [False, True])
def test_dist_gather_into_mixed_planes(transpose):
    """The same pull with mixed operand planes as the output (hi in fp32, hb | lb interleaved in bf16): the 16-byte
    kernels and the element-wise kernel must write identical planes, and the planes must represent the source."""
    from soap_tp_b200.engine import kernels as k

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    shape, nb, Pr, Pc, world = (384, 512), 64, 2, 2, 4
    dense = torch.randn(shape, generator=torch.Generator().manual_seed(3))
    kind = 2 if not transpose else 0
    buffers, table = _make_source(dense, kind, nb, Pr, Pc, world, device)
    rows_out = shape[1] if transpose else shape[0]
    extent_j = shape[0] if transpose else shape[1]
    cols_out = _numroc(extent_j, nb, 1, 2)
    index_j = _map(cols_out, 1, 2, nb, 0, None, 0)
    expected = (dense.T if transpose else dense)[:, index_j]

    def run():
        out = k.Planes.empty(rows_out, cols_out, device, mixed=True)
        low = out.low_pointers()
        k._C.dist_gather_mixed(table.data_ptr(), kind, shape[0], shape[1], nb, nb, Pr, Pc, world, 0, 1, 1, 0, 0,
                               1, 2, nb, 0, 0, int(transpose), 0, 0, 0, out.hi.data_ptr(), 0, 1, out.ld, rows_out, cols_out,
                               torch.cuda.current_stream().cuda_stream, low["hl"], low["ld16"])
        torch.cuda.synchronize()
        return out

    fast = run()
    k._C.force_scalar_gather(True)
    try:
        slow = run()
    finally:
        k._C.force_scalar_gather(False)
    assert torch.equal(fast.hi, slow.hi) and torch.equal(fast.hl, slow.hl)
    hb, lb = fast.halves()
    hi = fast.hi[:cols_out, :rows_out]
    want = expected.T.to(device)
    assert float((hi + lb - want).abs().max()) <= 2.0 ** -18 * float(want.abs().max())
    assert float((hb - want).abs().max()) <= 2.0 ** -8 * float(want.abs().max())


@pytest.mark.parametrize("transpose", [False, True])
def test_dist_gather_triangle_mask(transpose):
    """``upper_only`` (the pull of the mirrored half of a symmetric packed matrix): only entries whose mapped row
    index is below their mapped column index are written, everything else keeps its value; the 16-byte kernels and
    the element-wise kernel must agree bit for bit."""
    from soap_tp_b200.engine import kernels as k

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    n, nb, Pr, Pc = 640, 64, 2, 2
    dense = torch.randn(n, n, generator=torch.Generator().manual_seed(5))
    buffers, table = _make_source(dense, 0, nb, Pr, Pc, 4, device)
    pr, pc = 1, 0
    lr, lc = _numroc(n, nb, pr, Pr), _numroc(n, nb, pc, Pc)
    gi, gj = _map(lr, pr, Pr, nb, 0, None, 0), _map(lc, pc, Pc, nb, 0, None, 0)
    source = dense.T if transpose else dense
    expected = torch.full((lr, lc), -7.0)
    mask = gi[:, None] < gj[None, :]
    expected[mask] = source[gi[:, None], gj[None, :]][mask]

    def run():
        out = torch.full((lc, lr), -7.0, device=device).T
        k._C.dist_gather(table.data_ptr(), 0, n, n, nb, nb, Pr, Pc, 4, pr, Pr, nb, 0, 0, pc, Pc, nb, 0, 0, int(transpose), 1,
                         0, 0, out.data_ptr(), 0, 1, out.stride(1), lr, lc, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        return out.cpu()

    fast = run()
    k._C.force_scalar_gather(True)
    try:
        slow = run()
    finally:
        k._C.force_scalar_gather(False)
    assert torch.equal(slow, expected)
    assert torch.equal(fast, expected)

"""Multi-GPU device pipeline on a ``Pr x Pc`` grid.

Every distributed product is a stationary-C GEMM: a rank computes exactly the tiles of the result
it owns in the packed block-cyclic layout.  For ``C = Za^T Zb`` it needs all K rows of the columns
of ``Za`` that map to its local rows and of the columns of ``Zb`` that map to its local columns.
Those two panels are PULLED from the peers' symmetric segments by ``dist_gather_kernel``
(``csrc/comm.cu``): one kernel that reads the peers' memory over NVLink, reorders it into local
column order and writes the hi/lo operand planes of the 3xTF32 GEMM -- the all-gather, the layout
change (including the tensor-parallel shard -> block-cyclic redistribution of the gradient and the
column permutation of the power iterate) and the operand split are one pass.  The GEMM then runs
entirely on local memory and its epilogue writes either the packed state buffer (EMA, Adam) or the
symmetric segment the next stage pulls from.  Panels of the bases are cached until the basis
changes, so a steady step moves only gradient-sized panels.

Ordering between ranks is one barrier per producer/consumer edge (see ``parallel/comm.py``).
"""
from __future__ import annotations

import math
import os
import weakref
from collections import OrderedDict
from dataclasses import dataclass
from typing import Any, Dict, MutableMapping, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor

from ..layout import grid_coords, numroc, owned_indices
from ..parallel.comm import Communicator, SymmetricSegment, get_communicator, group_key
from ..profiling import GLOBAL_STAGE_TIMER as TIMER
from . import factor
from . import kernels as k

KIND_BLOCK_CYCLIC, KIND_ROW_SHARDS, KIND_COL_SHARDS = 0, 1, 2
# SOAP_TP_PIPELINE_GATHERS=1 overlaps peer pulls with the products that consume them, chunk by chunk.  Off by
# default: at 8192 on 2 B200s it measured 23.8-24.0 ms/step against 23.2-23.5 with one pull and one product --
# under the 1 kW power cap the product slows down by what the overlap hides, and chunking adds partial waves.
PIPELINE_GATHERS = os.environ.get("SOAP_TP_PIPELINE_GATHERS", "0") == "1"
# SOAP_TP_DISTRIBUTED_QR=0: every factorisation runs on one leader rank even when its group has more ranks
DISTRIBUTED_QR = os.environ.get("SOAP_TP_DISTRIBUTED_QR", "1") != "0"
# SOAP_TP_OVERLAP_GRAM=0: the Gram EMAs run after the rotations on the same stream instead of beside them
OVERLAP_GRAM = os.environ.get("SOAP_TP_OVERLAP_GRAM", "1") != "0"
# SOAP_TP_PUSH_PRODUCTS=1: the first product of every two-sided product stores its result, split into operand
# planes, straight into the gathered operand of the ranks that run the second product (peer stores from the GEMM
# epilogue: GEMM -> all-gather in one kernel, no pull kernel in between).  Off by default: at 8192 on 4 B200s the steady
# step measured 6.57 ms against 6.27 ms with the pull (the epilogue then stores 16 bytes per element, half of them
# over NVLink, in the part of a tile that no other work of its CTA overlaps; the pull kernel streams the same bytes
# at 600-700 GB/s), and 11.35 against 11.34 ms on 2 GPUs.
PUSH_PRODUCTS = os.environ.get("SOAP_TP_PUSH_PRODUCTS", "0") == "1"
# Operand planes of the eigenbases kept per engine between steps (SOAP_TP_BASIS_CACHE_GB, default 40): beyond that the
# least recently used ones are dropped and rebuilt on use, trading about a millisecond per step and basis for memory.
BASIS_CACHE_BYTES = int(float(os.environ.get("SOAP_TP_BASIS_CACHE_GB", "40")) * 2**30)
# output tiles a chunk must keep (about one wave of the 148 SMs); tests lower it to chunk small problems
PIPELINE_MIN_TILES = max(1, int(os.environ.get("SOAP_TP_PIPELINE_MIN_TILES", "120")))


@dataclass
class Source:
    """A matrix spread over the ranks, addressable by every rank through a symmetric segment."""

    segment: SymmetricSegment
    kind: int
    rows: int
    cols: int
    nb_r: int = 1
    nb_c: int = 1
    Pr: int = 1
    Pc: int = 1
    world: int = 1


@dataclass
class IndexMap:
    p: int = 0
    P: int = 1
    nb: int = 1
    offset: int = 0
    perm: Optional[Tensor] = None
    local_offset: int = 0   # added to the local index before anything else (a chunk of the local range)


IDENTITY = IndexMap()


def dist_gather(src: Source, map_i: IndexMap, map_j: IndexMap, rows_out: int, cols_out: int, *, transpose: bool = False,
                planes: Optional[k.Planes] = None, out: Optional[Tensor] = None, upper_only: bool = False) -> None:
    """``out(i, j) = src(map_i(i), map_j(j))`` (``src(map_j(j), map_i(i))`` if ``transpose``)."""
    if rows_out <= 0 or cols_out <= 0:
        return
    extra = ()
    if planes is not None:
        low = planes.low_pointers()
        hi, lo, d_i, d_j = planes.hi.data_ptr(), low["lo"], 1, planes.ld
        if planes.mixed:
            extra = (low["hl"], low["ld16"])
    else:
        assert out is not None
        hi, lo = out.data_ptr(), 0
        d_i = out.stride(0) if out.shape[0] > 1 else 1
        d_j = out.stride(1) if out.shape[1] > 1 else max(1, out.shape[0])
    launch = k._C.dist_gather_mixed if extra else k._C.dist_gather
    launch(
        src.segment.peer_table.data_ptr(), src.kind, src.rows, src.cols, src.nb_r, src.nb_c, src.Pr, src.Pc, src.world,
        map_i.p, map_i.P, map_i.nb, map_i.offset, map_i.perm.data_ptr() if map_i.perm is not None else 0,
        map_j.p, map_j.P, map_j.nb, map_j.offset, map_j.perm.data_ptr() if map_j.perm is not None else 0,
        int(transpose), int(upper_only), map_i.local_offset, map_j.local_offset, hi, lo, d_i, d_j, rows_out, cols_out,
        k._stream(), *extra)
    k._count("dist_gather_kernel")
    if out is not None:
        k.mark_written(out)


def _packed_view(segment: SymmetricSegment, local_rows: int, local_cols: int) -> Tensor:
    """Column-major ``local_rows x local_cols`` view (exact pitch) at the start of a segment."""
    lr, lc = max(1, local_rows), max(1, local_cols)
    return segment.local[: lr * lc].view(lc, lr).T


class GridEngine:
    """Distributed kernels' driver for one ``(device, grid, block_size)``."""

    def __init__(self, device: torch.device, grid: Tuple[int, int], block_size: int, group=None) -> None:
        self.comm: Communicator = get_communicator(device, group)
        self.device = torch.device(device)
        self.grid = grid
        self.nb = block_size
        self.Pr, self.Pc = grid
        self.rank = self.comm.rank
        self.world = self.comm.world
        self.pr, self.pc = grid_coords(self.rank, grid)
        self._planes: Dict[tuple, k.Planes] = {}
        self._basis_cache: "OrderedDict[tuple, dict]" = OrderedDict()
        self._leader_tables: Dict[tuple, Tensor] = {}

    # ---- small helpers -----------------------------------------------------------------------
    def rows_of(self, n: int) -> int:
        return numroc(n, self.nb, self.pr, self.Pr)

    def cols_of(self, n: int) -> int:
        return numroc(n, self.nb, self.pc, self.Pc)

    def row_map(self, perm: Optional[Tensor] = None) -> IndexMap:
        return IndexMap(self.pr, self.Pr, self.nb, 0, perm)

    def col_map(self, perm: Optional[Tensor] = None) -> IndexMap:
        return IndexMap(self.pc, self.Pc, self.nb, 0, perm)

    def planes(self, tag: str, depth: int, cols: int, classic: bool = False) -> k.Planes:
        """Cached operand planes.  The operands of the optimizer-step products are mixed planes (``kernels.Planes``);
        ``classic`` asks for fp32 hi/lo planes (operands of the power iteration, which feeds the QR)."""
        mixed = k.MIXED_CORRECTIONS and not classic
        key = (tag, depth, cols, mixed)
        found = self._planes.get(key)
        if found is None:
            found = k.Planes.empty(depth, cols, self.device, mixed=mixed)
            self._planes[key] = found
        return found

    def leader_table(self, segment: SymmetricSegment, leader: int) -> Tensor:
        """One-entry peer table that points at ``leader``'s copy of ``segment``."""
        key = (segment.name, leader)
        table = self._leader_tables.get(key)
        if table is None:
            table = torch.tensor([segment.peer_ptrs[leader]], dtype=torch.int64, device=self.device)
            self._leader_tables[key] = table
        return table

    def packed_segment(self, tag: str, shape) -> Tuple[SymmetricSegment, Tensor, Source]:
        """Symmetric staging buffer holding a packed block-cyclic matrix of global ``shape``."""
        rows, cols = shape
        most_rows = numroc(rows, self.nb, 0, self.Pr)
        most_cols = numroc(cols, self.nb, 0, self.Pc)
        segment = self.comm.segment(f"{tag}:{rows}x{cols}:{self.nb}:{self.Pr}x{self.Pc}", max(1, most_rows) * max(1, most_cols))
        view = _packed_view(segment, self.rows_of(rows), self.cols_of(cols))
        return segment, view, Source(segment, KIND_BLOCK_CYCLIC, rows, cols, self.nb, self.nb, self.Pr, self.Pc, self.world)

    def stage_packed(self, tag: str, matrix: Tensor, shape) -> Source:
        """Copy this rank's packed buffer into the symmetric staging segment ``tag``."""
        _, view, source = self.packed_segment(tag, shape)
        lr, lc = self.rows_of(shape[0]), self.cols_of(shape[1])
        if lr and lc:
            k.gather2d(matrix[:lr, :lc], view[:lr, :lc], None, None)
        return source

    def stage_shard(self, shard: Tensor, global_shape, shard_dim: int) -> Source:
        rows, cols = global_shape
        segment = self.comm.segment(f"shard:{rows}x{cols}:{shard_dim}", max(1, shard.numel()))
        flat = segment.local[: shard.numel()].view(shard.shape)
        source = shard.detach()
        if source.dtype != torch.float32 or not source.is_contiguous():
            flat.copy_(source)
        else:
            k.gather2d(source, flat, None, None)
        kind = KIND_ROW_SHARDS if shard_dim == 0 else KIND_COL_SHARDS
        return Source(segment, kind, rows, cols, world=self.world)

    # ---- cached panels of a basis -------------------------------------------------------------
    def basis_panels(self, Q: Tensor, size: int, tag: str) -> Tuple[k.Planes, k.Planes]:
        """Planes of ``Q[:, my column class]`` (depth = size) and of ``Q^T[:, my column class]``,
        i.e. rows of ``Q`` in my column class.  Collective; cached on the tensor version."""
        cache_key = (Q.data_ptr(), size)
        entry = self._basis_cache.get(cache_key)
        if entry is None:
            entry = self._basis_cache[cache_key] = {}
        else:
            self._basis_cache.move_to_end(cache_key)
        # Ranks run the same program on the same step, so staleness is decided locally: a basis
        # changes on all ranks (refresh, initialisation, checkpoint load) or on none.  The entry belongs to one
        # tensor OBJECT: a new tensor that the allocator happens to place at the address of a freed one (with
        # the same version count) must miss on every rank, or the ranks would disagree about the barriers below.
        owner = entry.get("owner")
        if owner is not None and owner() is Q and entry.get("key") == (Q._version, size):
            return entry["plain"], entry["transposed"]
        source = self.stage_packed("basis", Q, (size, size))
        self.comm.barrier()
        cols = self.cols_of(size)
        plain = entry.get("plain") or k.Planes.empty(size, cols, self.device, mixed=k.MIXED_CORRECTIONS)
        transposed = entry.get("transposed") or k.Planes.empty(size, cols, self.device, mixed=k.MIXED_CORRECTIONS)
        dist_gather(source, IDENTITY, self.col_map(), size, cols, planes=plain)
        dist_gather(source, IDENTITY, self.col_map(), size, cols, transpose=True, planes=transposed)
        self.comm.barrier()
        # 12 bytes per element of this rank's share of the basis (two orientations, value plane + low plane), counted
        # with the widest rank's share so that every rank evicts the same entries
        entry.update(key=(Q._version, size), plain=plain, transposed=transposed, owner=weakref.ref(Q),
                     bytes=12 * size * numroc(size, self.nb, 0, self.Pc))
        self._evict_basis_planes(keep=cache_key)
        return plain, transposed

    def _evict_basis_planes(self, keep: tuple) -> None:
        """Operand planes of the bases are three times the size of the bases themselves.  With many parameters (a
        32-layer decoder) they are kept only up to ``BASIS_CACHE_BYTES`` per engine; an evicted basis is split again
        on its next use (one staging copy and two pulls per step).  Entries of tensors that no longer exist go
        first; then the MOST recently used ones, because an optimizer walks its parameters in the same order every
        step: the oldest entries are the next to be used, and dropping them would make every access miss."""
        total = sum(entry.get("bytes", 0) for entry in self._basis_cache.values())
        if total <= BASIS_CACHE_BYTES:
            return
        dead = [key for key, entry in self._basis_cache.items()
                if key != keep and (entry.get("owner") is None or entry["owner"]() is None)]
        for key in dead + [key for key in reversed(self._basis_cache) if key != keep and key not in dead]:
            if total <= BASIS_CACHE_BYTES:
                break
            total -= self._basis_cache.pop(key).get("bytes", 0)

    def side_stream(self) -> "torch.cuda.Stream":
        """The stream on which work that is independent of the rotations (the Gram EMAs) runs beside them."""
        if not hasattr(self, "_side_stream"):
            self._side_stream = torch.cuda.Stream(device=self.device)
        return self._side_stream

    # ---- gather / product pipelining ------------------------------------------------------------
    def _pipeline_streams(self):
        if not hasattr(self, "_gather_stream"):
            self._gather_stream = torch.cuda.Stream(device=self.device)
            self._product_stream = torch.cuda.Stream(device=self.device)
        return self._gather_stream, self._product_stream

    @staticmethod
    def _column_chunks(cols: int, tiles: int, granule: int):
        """Split ``cols`` operand columns into up to four chunks (boundaries on multiples of ``granule``) such
        that each chunk still launches about a wave of the ``tiles`` output tiles of the whole product."""
        slabs = -(-cols // granule)
        count = max(1, min(4, tiles // PIPELINE_MIN_TILES, slabs))
        if not PIPELINE_GATHERS or count == 1:
            return [(0, cols)]
        bounds = [granule * ((slabs * i) // count) for i in range(count)] + [cols]
        return [(bounds[i], bounds[i + 1]) for i in range(count) if bounds[i + 1] > bounds[i]]

    def gather_then_multiply(self, source: Source, column_map: IndexMap, depth: int, cols: int, planes: k.Planes,
                             multiply, *, transpose: bool = False, other_cols: int = 256, as_columns: bool = False) -> None:
        """Pull the operand ``planes`` (``depth x cols``; local column ``j`` is source column ``column_map(j)``)
        from the peers chunk by chunk and call ``multiply(c0, c1)`` for every chunk once it has landed.

        The pulls run on a stream of their own and the products alternate between the calling stream and a
        second one, so the NVLink transfer of chunk ``i + 1`` overlaps the tensor-core product of chunk
        ``i`` and consecutive products fill each other's tails.  ``multiply(c0, c1)`` must touch only rows
        ``[c0, c1)`` of its outputs (columns, with ``as_columns``: the operand is the product's second one);
        ``other_cols`` is the extent of the product's other output dimension.
        """
        if as_columns:
            tiles, granule = -(-other_cols // 128) * -(-cols // 256), 256
        else:
            tiles, granule = -(-cols // 128) * -(-other_cols // 256), 128
        chunks = self._column_chunks(cols, tiles, granule)
        if len(chunks) == 1:
            dist_gather(source, IDENTITY, column_map, depth, cols, transpose=transpose, planes=planes)
            multiply(0, cols)
            return
        main = torch.cuda.current_stream(self.device)
        pulls, second = self._pipeline_streams()
        start = torch.cuda.Event()
        start.record(main)
        pulls.wait_event(start)
        second.wait_event(start)
        for index, (c0, c1) in enumerate(chunks):
            with torch.cuda.stream(pulls):
                chunk_map = IndexMap(column_map.p, column_map.P, column_map.nb, column_map.offset, column_map.perm,
                                     column_map.local_offset + c0)
                dist_gather(source, IDENTITY, chunk_map, depth, c1 - c0, transpose=transpose,
                            planes=planes.sub(0, c0, depth, c1 - c0))
                landed = torch.cuda.Event()
                landed.record(pulls)
            target = main if index % 2 == 0 else second
            target.wait_event(landed)
            with torch.cuda.stream(target):
                multiply(c0, c1)
        joined = torch.cuda.Event()
        joined.record(second)
        main.wait_event(joined)

    def two_sided(self, source: Source, shape, first: k.Planes, second: k.Planes, *, panel: Optional[k.Planes] = None,
                  gathered: bool = False, **final) -> k.Planes:
        """``final( (X^T F)^T S )`` for the ``rows x cols`` matrix ``X`` behind ``source``.

        ``first`` holds ``F[:, my column class]`` (depth rows), ``second`` holds ``S[:, my column
        class]`` (depth cols).  The caller has already ordered ``source`` before this call.  ``panel``
        is the buffer for the gathered operand ``X[:, my row class]`` (``gathered``: it already holds it);
        it is returned for reuse.  Both pulls are pipelined with their products.
        """
        rows, cols = shape
        a = panel if panel is not None else self.planes("panel_a", rows, self.rows_of(cols))
        first_cols = max(1, first.cols)
        push = PUSH_PRODUCTS and not PIPELINE_GATHERS
        if push:
            # GEMM -> all-gather in one kernel: the epilogue of the first product stores every element of the middle
            # matrix, already split into operand planes, into the gathered operand of each rank that consumes it
            ta, targets = self.push_targets(cols, rows)

            def middle(c0: int, c1: int) -> None:
                k.gemm(a.sub(0, c0, rows, c1 - c0), first, mode=k.EPI_PUSH, push=targets)
        else:
            _, t_view, t_source = self.packed_segment("middle", (cols, rows))

            def middle(c0: int, c1: int) -> None:
                k.gemm(a.sub(0, c0, rows, c1 - c0), first, mode=k.EPI_STORE, out=t_view[c0:c1, :first_cols])

        if a.cols > 0:
            if gathered:
                middle(0, a.cols)
            elif push:
                dist_gather(source, IDENTITY, self.row_map(), rows, a.cols, planes=a)
                middle(0, a.cols)
            else:
                self.gather_then_multiply(source, self.row_map(), rows, a.cols, a, middle, other_cols=first.cols)
        self.comm.barrier()
        if not push:
            ta = self.planes("panel_t", cols, self.rows_of(rows))

        def last(c0: int, c1: int) -> None:
            window = dict(final)
            for name in ("out", "momentum", "variance"):
                if window.get(name) is not None:
                    window[name] = window[name][c0:c1]
            k.gemm(ta.sub(0, c0, cols, c1 - c0), second, **window)

        if ta.cols > 0:
            if push:
                last(0, ta.cols)
            else:
                self.gather_then_multiply(t_source, self.row_map(), cols, ta.cols, ta, last, other_cols=second.cols)
        return a

    def push_targets(self, depth: int, width: int) -> Tuple[k.Planes, dict]:
        """Operand planes of ``T[:, my row class]`` (``depth x rows_of(width)``) in symmetric memory, for the producers
        of ``T`` to fill through peer pointers, and the argument dictionary of the pushing product.  Two sets
        alternate from call to call: a rank may still be reading one set in the second product of a call while a
        faster peer, one barrier further, already pushes the next call's middle matrix."""
        self._push_calls = getattr(self, "_push_calls", 0) + 1
        parity = self._push_calls % 2
        mixed = k.MIXED_CORRECTIONS
        most = max(1, numroc(width, self.nb, 0, self.Pr))
        ld = max(4, k.round_up(depth, 4))
        ld16 = 2 * k.round_up(max(1, depth), 32)
        low_floats = most * (ld16 // 2 if mixed else ld)
        name = f"push{parity}:{depth}x{width}:{self.nb}:{self.Pr}x{self.Pc}:{int(mixed)}"
        fresh = name not in self.comm.segments
        segment = self.comm.segment(name, most * ld + low_floats)
        if fresh:
            segment.local.zero_()          # the bf16 plane's tail past `depth` has to read as zeros
            self.comm.barrier()            # ... before any peer starts to push into it
        hi = segment.local[: most * ld].view(most, ld)
        low = segment.local[most * ld: most * ld + low_floats]
        mine = self.rows_of(width)
        if mixed:
            planes = k.Planes(hi, None, depth, mine, ld, low.view(torch.bfloat16).view(most, ld16), ld16)
        else:
            planes = k.Planes(hi, low.view(most, ld), depth, mine, ld)
        key = ("push_table", name)
        table = self._leader_tables.get(key)
        if table is None:
            entries = []
            for base in segment.peer_ptrs:
                entries += [base, base + 4 * most * ld]
            table = self._leader_tables[key] = torch.tensor(entries, dtype=torch.int64, device=self.device)
        return planes, dict(table=table, ld=ld, ld16=ld16, nb=self.nb, Pr=self.Pr, Pc=self.Pc, pr=self.pr, pc=self.pc,
                            mixed=mixed)


_ENGINES: Dict[tuple, GridEngine] = {}


def engine_for(device: torch.device, grid, block_size: int, group=None) -> GridEngine:
    """The engine of a grid over ``group`` (default: the world).  The ops that take ``group=`` (the two
    redistributions and the permutation, as in the reference's ``src/soap_tp/ops/optimizer.py:71,229,404``)
    pass it on; ranks, peers and barriers are then those of the group."""
    key = (str(torch.device(device)), tuple(grid), int(block_size), group_key(group))
    engine = _ENGINES.get(key)
    if engine is None:
        engine = GridEngine(device, tuple(grid), int(block_size), group)
        _ENGINES[key] = engine
    return engine


def reset_engines() -> None:
    _ENGINES.clear()


# ---------------------------------------------------------------------------------------------
# Public-op entry points (each is collective and self-contained)
# ---------------------------------------------------------------------------------------------
def redistribute_tp_to_bc(matrix: Tensor, global_shape, block_size: int, grid, shard_dim: int, group=None) -> Tensor:
    e = engine_for(matrix.device, grid, block_size, group)
    rows, cols = global_shape
    source = e.stage_shard(matrix, global_shape, shard_dim)
    e.comm.barrier()
    lr, lc = e.rows_of(rows), e.cols_of(cols)
    packed = torch.empty((max(1, lc), max(1, lr)), dtype=torch.float32, device=matrix.device).T
    dist_gather(source, e.row_map(), e.col_map(), lr, lc, out=packed)
    e.comm.barrier()
    return packed if matrix.dtype == torch.float32 else packed.to(matrix.dtype)


def _pull_shard(e: GridEngine, source: Source, global_shape, shard_dim: int) -> Tensor:
    rows, cols = global_shape
    if shard_dim == 0:
        per = rows // e.world
        shard = torch.empty((per, cols), dtype=torch.float32, device=e.device)
        dist_gather(source, IndexMap(offset=e.rank * per), IDENTITY, per, cols, out=shard)
    else:
        per = cols // e.world
        shard = torch.empty((rows, per), dtype=torch.float32, device=e.device)
        dist_gather(source, IDENTITY, IndexMap(offset=e.rank * per), rows, per, out=shard)
    return shard


def redistribute_bc_to_tp(matrix: Tensor, global_shape, block_size: int, grid, shard_dim: int, group=None) -> Tensor:
    e = engine_for(matrix.device, grid, block_size, group)
    source = e.stage_packed("stage", matrix if matrix.dtype == torch.float32 else matrix.float(), global_shape)
    e.comm.barrier()
    shard = _pull_shard(e, source, global_shape, shard_dim)
    e.comm.barrier()
    return shard if matrix.dtype == torch.float32 else shard.to(matrix.dtype)


def rotate(matrix: Tensor, Q_left: Tensor, Q_right: Tensor, global_shape, block_size: int, grid, direction: str) -> Tensor:
    e = engine_for(matrix.device, grid, block_size)
    rows, cols = global_shape
    left_plain, left_t = e.basis_panels(Q_left, rows, "left")
    right_plain, right_t = e.basis_panels(Q_right, cols, "right")
    source = e.stage_packed("stage", matrix, global_shape)
    e.comm.barrier()
    lr, lc = e.rows_of(rows), e.cols_of(cols)
    first, second = (left_plain, right_plain) if direction == "forward" else (left_t, right_t)
    e.two_sided(source, global_shape, first, second, mode=k.EPI_STORE, out=matrix[: max(1, lr), : max(1, lc)])
    e.comm.barrier()
    return matrix


def gram_update(G_local: Tensor, preconditioner: Tensor, beta: float, block_size: int, grid, shard_dim: int, side: str) -> Tensor:
    e = engine_for(G_local.device, grid, block_size)
    dims = [tuple(d) for d in e.comm.gather_ints(list(G_local.shape))]
    replicated = 1 - shard_dim
    if any(d[replicated] != dims[0][replicated] for d in dims):
        raise ValueError(f"non-sharded dimension {replicated} must match on every rank.")
    if any(d[shard_dim] != dims[0][shard_dim] for d in dims):
        # unequal shards: bring them to equal contiguous shards on the host path of the control plane
        return _gram_update_unequal(e, G_local, preconditioner, beta, shard_dim, side, dims)
    global_shape = list(dims[0])
    global_shape[shard_dim] *= e.world
    rows, cols = global_shape
    size = rows if side == "left" else cols
    from ..layout import validate_2d_block_cyclic_buffer

    validate_2d_block_cyclic_buffer(f"{side}_preconditioner", preconditioner, (size, size), block_size, grid, e.rank)
    source = e.stage_shard(G_local, (rows, cols), shard_dim)
    e.comm.barrier()
    _gram_from_source(e, source, (rows, cols), preconditioner, beta, side)
    _mirror_upper(e, [(side, preconditioner, size)])
    e.comm.barrier()
    return preconditioner


def gram_rows_from_col_shards(G_local: Tensor, out: Tensor, beta: float, side: str) -> Tensor:
    """1-D row-sharded Gram EMA for column-sharded ``G`` (``ops/gram_1d.py``).

    ``side == "left"``: ``out`` is rows ``[r m/W, (r+1) m/W)`` of ``beta L + (1-beta) G G^T``;
    ``side == "right"``: the block row of ``G^T G`` of this rank's columns.  ``out`` is row-major, so
    its memory is the column-major transpose ``C' = (all rows) x (my rows)`` that the GEMM writes.
    """
    world = dist.get_world_size()
    e = engine_for(G_local.device, (1, world), 128)
    shapes = e.comm.gather_ints(list(G_local.shape))
    if any(s != shapes[0] for s in shapes):
        raise RuntimeError("every rank must hold a column shard of the same shape.")
    m, n_local = G_local.shape
    n = n_local * world
    source = e.stage_shard(G_local, (m, n), 1)
    e.comm.barrier()
    if side == "left":
        depth, size, mine, first = n, m, m // world, e.rank * (m // world)
        a = e.planes("gram1d_left", depth, size)
        dist_gather(source, IDENTITY, IDENTITY, depth, size, transpose=True, planes=a)   # G^T
    else:
        depth, size, mine, first = m, n, n_local, e.rank * n_local
        a = e.planes("gram1d_right", depth, size)
        dist_gather(source, IDENTITY, IDENTITY, depth, size, planes=a)                   # G
    b = a.sub(0, first, depth, mine)
    k.gemm(a, b, out=out.T, alpha=1.0 - beta, beta=beta)
    k.mark_written(out)
    e.comm.barrier()
    return out


def _gram_from_source(e: GridEngine, source: Source, shape, preconditioner: Tensor, beta: float, side: str,
                      gathered: Optional[k.Planes] = None) -> None:
    """Lower triangle (global indices) of ``beta P + (1 - beta) Gram`` on this rank's packed block.

    Operand panels: ``a`` = the Gram factor restricted to my local rows, ``b`` = to my local columns;
    ``gathered`` is ``a`` if the caller already holds it.  Whichever operand still has to come from the
    peers last is pulled in chunks that overlap with the products; `_mirror_upper` fills the other triangle.
    """
    rows, cols = shape
    if side == "left":    # L = G G^T: contraction over columns, operands are rows of G
        size, depth, transpose = rows, cols, True
    else:                 # R = G^T G: contraction over rows, operands are columns of G
        size, depth, transpose = cols, rows, False
    lr, lc = e.rows_of(size), e.cols_of(size)
    if lr == 0 or lc == 0:
        return
    triangle = (e.nb, e.pr, e.Pr, e.pc, e.Pc)
    weight = dict(alpha=1.0 - beta, beta=beta)
    b = e.planes("gram_b", depth, lc)
    if gathered is not None:
        a = gathered

        def columns(c0: int, c1: int) -> None:     # a window of my local columns
            k.gemm(a, b.sub(0, c0, depth, c1 - c0), out=preconditioner[:lr, c0:c1], lower_of_grid=triangle + (0, c0),
                   **weight)

        e.gather_then_multiply(source, e.col_map(), depth, lc, b, columns, transpose=transpose, other_cols=lr,
                               as_columns=True)
        return
    a = e.planes("gram_a", depth, lr)
    dist_gather(source, IDENTITY, e.col_map(), depth, lc, transpose=transpose, planes=b)

    def rows_window(c0: int, c1: int) -> None:      # a window of my local rows
        k.gemm(a.sub(0, c0, depth, c1 - c0), b, out=preconditioner[c0:c1, :lc], lower_of_grid=triangle + (c0, 0),
               **weight)

    e.gather_then_multiply(source, e.row_map(), depth, lr, a, rows_window, transpose=transpose, other_cols=lc)


def _mirror_upper(e: GridEngine, items, channel: int = 0) -> None:
    """Complete symmetric packed matrices whose lower triangles were just computed.

    ``items``: ``(tag, matrix, size)``.  Every rank publishes its packed block, and after one barrier
    pulls the entries above the global diagonal from the owners of the mirrored entries (a transposed,
    masked ``dist_gather``).  The result is exactly symmetric.  The published copies are overwritten
    only after a later barrier of the caller.
    """
    sources = [e.stage_packed(f"gram_{tag}", matrix, (size, size)) for tag, matrix, size in items]
    e.comm.barrier(channel=channel)
    for source, (tag, matrix, size) in zip(sources, items):
        lr, lc = e.rows_of(size), e.cols_of(size)
        if lr and lc:
            dist_gather(source, e.row_map(), e.col_map(), lr, lc, transpose=True, out=matrix[:lr, :lc], upper_only=True)


def _gram_update_unequal(e: GridEngine, G_local, preconditioner, beta, shard_dim, side, dims) -> Tensor:
    """Unequal ``tensor_split`` shards: pad every shard to the longest one with zero rows/columns
    (zeros add nothing to a Gram matrix) and run the equal-shard path on the padded matrix."""
    longest = max(d[shard_dim] for d in dims)
    padded_shape = list(G_local.shape)
    padded_shape[shard_dim] = longest
    padded = torch.zeros(padded_shape, dtype=torch.float32, device=G_local.device)
    padded.narrow(shard_dim, 0, G_local.shape[shard_dim]).copy_(G_local)
    rows, cols = padded_shape
    global_shape = [rows, cols]
    global_shape[shard_dim] = longest * e.world
    true_size = sum(d[shard_dim] for d in dims) if (side == "left") == (shard_dim == 0) else dims[0][1 - shard_dim]
    source = e.stage_shard(padded, tuple(global_shape), shard_dim)
    e.comm.barrier()
    if (side == "left") == (shard_dim == 0):
        # the Gram matrix is indexed by the padded dimension: map true indices to padded positions
        position = torch.cat([torch.arange(d[shard_dim]) + r * longest for r, d in enumerate(dims)]).to(e.device)
        size = true_size
        depth = global_shape[1 - shard_dim]
        transpose = side == "left"
        lr, lc = e.rows_of(size), e.cols_of(size)
        a, b = e.planes("gram_a", depth, lr), e.planes("gram_b", depth, lc)
        dist_gather(source, IDENTITY, e.row_map(position), depth, lr, transpose=transpose, planes=a)
        dist_gather(source, IDENTITY, e.col_map(position), depth, lc, transpose=transpose, planes=b)
        k.gemm(a, b, out=preconditioner[: max(1, lr), : max(1, lc)], alpha=1.0 - beta, beta=beta,
               lower_of_grid=(e.nb, e.pr, e.Pr, e.pc, e.Pc))
    else:
        _gram_from_source(e, source, tuple(global_shape), preconditioner, beta, side)
    _mirror_upper(e, [(side, preconditioner, true_size)])
    e.comm.barrier()
    return preconditioner


def _product_with_basis(e: GridEngine, P: Tensor, Q: Tensor, work: Tensor, size: int) -> None:
    """``work <- P Q`` for symmetric packed ``P`` (so ``P^T Q``)."""
    p_source = e.stage_packed("stage", P, (size, size))
    q_source = e.stage_packed("basis", Q, (size, size))
    e.comm.barrier()
    lr, lc = e.rows_of(size), e.cols_of(size)
    a, b = e.planes("power_a", size, lr, classic=True), e.planes("power_b", size, lc, classic=True)
    dist_gather(p_source, IDENTITY, e.row_map(), size, lr, planes=a)
    dist_gather(q_source, IDENTITY, e.col_map(), size, lc, planes=b)
    k.gemm(a, b, out=work[: max(1, lr), : max(1, lc)])
    e.comm.barrier()


def estimated_order(P: Tensor, Q: Tensor, work: Tensor, size: int, block_size: int, grid) -> Tensor:
    e = engine_for(P.device, grid, block_size)
    with TIMER.stage("refresh.power_iteration.product", P.device):
        _product_with_basis(e, P, Q, work, size)
    lr, lc = e.rows_of(size), e.cols_of(size)
    with TIMER.stage("refresh.power_iteration.estimates", P.device):
        # partial column dots over my rows, one row of a (Pr x size) block-cyclic matrix with row blocks of 1
        most_cols = numroc(size, e.nb, 0, e.Pc)
        segment = e.comm.segment(f"estimates:{size}:{e.nb}", max(1, most_cols))
        partial = segment.local[: max(1, lc)]
        partial.zero_()
        if lr and lc:
            k.column_dot(Q, work, lr, lc, out=partial)
        e.comm.barrier()
        source = Source(segment, KIND_BLOCK_CYCLIC, e.Pr, size, 1, e.nb, e.Pr, e.Pc, e.world)
        table = torch.empty((size, e.Pr), dtype=torch.float32, device=P.device).T   # Pr x size, column-major
        dist_gather(source, IDENTITY, IDENTITY, e.Pr, size, out=table)
        e.comm.barrier()
    with TIMER.stage("refresh.power_iteration.sort", P.device):
        order = k.order_by_estimate(table)   # column sums in fixed order over Pr -> identical on every rank
    return order


def _gather_dense(e: GridEngine, source: Source, size: int, column_order: Optional[Tensor] = None) -> Tensor:
    dense = torch.empty((size, size), dtype=torch.float32, device=e.device).T
    dist_gather(source, IDENTITY, IndexMap(perm=column_order), size, size, out=dense)
    return dense


def _scatter_owned(e: GridEngine, dense: Tensor, packed: Tensor, size: int) -> None:
    lr, lc = e.rows_of(size), e.cols_of(size)
    if lr and lc:
        rows = owned_indices(size, e.nb, e.pr, e.Pr, e.device)
        cols = owned_indices(size, e.nb, e.pc, e.Pc, e.device)
        k.gather2d(dense, packed[:lr, :lc], rows, cols)
        k.mark_written(packed)


def _leader_of(job: int, jobs: int, world: int) -> int:
    """Rank that runs job ``job`` of ``jobs`` independent dense factorisations."""
    return (job * world) // jobs


def _factor_on_leaders(e: GridEngine, jobs, run, long_running: bool = False) -> None:
    """Run independent dense factorisations concurrently, one per leader rank.

    ``jobs`` is a list of ``(packed input, packed output, size, column_order)``.  Every rank stages
    its part of every input; the leader of job ``i`` pulls the whole (column-permuted) matrix,
    calls ``run(i, dense_input, dense_output)`` with this package's single-GPU kernels, and leaves
    the dense result in a symmetric segment from which every rank then pulls the tiles it owns.
    With two jobs (left and right basis) and at least two ranks the two factorisations overlap
    completely; the factorisations are deterministic, so nothing has to be compared afterwards.
    """
    count = len(jobs)
    sources = []
    for index, (matrix, _, size, _) in enumerate(jobs):
        sources.append(e.stage_packed(f"factor_in{index}", matrix, (size, size)))
    e.comm.barrier()
    results = []
    for index, (matrix, output, size, order) in enumerate(jobs):
        leader = _leader_of(index, count, e.world)
        segment = e.comm.segment(f"factor_out{index}:{size}", size * size)
        results.append((segment, leader))
        if e.rank == leader:
            dense_in = _gather_dense(e, sources[index], size, order)
            dense_out = segment.local[: size * size].view(size, size).T
            run(index, dense_in, dense_out)
    # the other ranks wait here for the leaders' factorisations: on the host when those can outlast the
    # device barrier's spin budget (`long_running`: the eigensolver at initialisation)
    e.comm.barrier(after_long_work=long_running)
    for (matrix, output, size, order), (segment, leader) in zip(jobs, results):
        table = e.leader_table(segment, leader)
        source = Source(segment, KIND_BLOCK_CYCLIC, size, size, 1, 1, 1, 1, 1)
        lr, lc = e.rows_of(size), e.cols_of(size)
        if lr and lc:
            _dist_gather_table(table, source, e.row_map(), e.col_map(), lr, lc, output[:lr, :lc])
    e.comm.barrier()


def _dist_gather_table(table: Tensor, src: Source, map_i: IndexMap, map_j: IndexMap, rows_out: int, cols_out: int,
                       out: Tensor) -> None:
    """``dist_gather`` with an explicit peer table (here: a single entry, the leader's buffer)."""
    d_i = out.stride(0) if out.shape[0] > 1 else 1
    d_j = out.stride(1) if out.shape[1] > 1 else max(1, out.shape[0])
    k._C.dist_gather(table.data_ptr(), src.kind, src.rows, src.cols, src.nb_r, src.nb_c, src.Pr, src.Pc, src.world,
                     map_i.p, map_i.P, map_i.nb, map_i.offset, 0, map_j.p, map_j.P, map_j.nb, map_j.offset, 0, 0, 0, 0, 0,
                     out.data_ptr(), 0, d_i, d_j, rows_out, cols_out, k._stream())
    k._count("dist_gather_kernel")
    k.mark_written(out)


def qr_many(e: GridEngine, jobs) -> None:
    """``jobs``: list of ``(packed matrix, packed Q, size, column_order)``, factored concurrently.

    With at least two ranks per job the work of each factorisation is spread over the job's ranks
    (``engine/dist_qr.py``: panel chain on a leader, accumulation of ``Q`` on the others); with fewer ranks every
    job runs on one leader rank (:func:`_factor_on_leaders`)."""
    from ..ops.basis import count_qr_call
    from . import dist_qr

    if DISTRIBUTED_QR and all(workers for _, workers in (dist_qr.group_of(i, len(jobs), e.world) for i in range(len(jobs)))):
        sources = [e.stage_packed(f"factor_in{index}", matrix, (size, size))
                   for index, (matrix, _, size, _) in enumerate(jobs)]
        e.comm.barrier()

        def gather_input(index: int, planes: k.Planes) -> None:
            size, order = jobs[index][2], jobs[index][3]
            dist_gather(sources[index], IDENTITY, IndexMap(perm=order), size, size, planes=planes)

        dist_qr.qr_jobs(e, jobs, gather_input)
        return
    _factor_on_leaders(e, jobs, lambda index, dense_in, dense_out: factor.householder_qr(dense_in, dense_out))
    # the leader's factorisation counted itself; the other ranks took part in the same collective call
    for index in range(len(jobs)):
        if _leader_of(index, len(jobs), e.world) != e.rank:
            count_qr_call()


def qr(matrix: Tensor, Q: Tensor, size: int, block_size: int, grid, column_order: Optional[Tensor] = None) -> Tensor:
    """Householder QR of the packed ``matrix`` (columns optionally permuted on the way in).

    One rank pulls the whole (permuted) matrix and factors it with the single-GPU blocked
    Householder kernels; every rank then pulls the tiles of ``Q`` it owns from that rank.
    """
    e = engine_for(matrix.device, grid, block_size)
    qr_many(e, [(matrix, Q, size, column_order)])
    return Q


def power_iteration_qr(P: Tensor, Q: Tensor, work: Tensor, size: int, block_size: int, grid) -> Tensor:
    order = estimated_order(P, Q, work, size, block_size, grid)
    qr(work, Q, size, block_size, grid, column_order=order)
    return order


def initialize_bases(e: GridEngine, jobs) -> None:
    """``jobs``: list of ``(packed P, packed Q, size, eigenvalues, implementation)`` solved concurrently."""
    scratch = {}

    def run(index, dense_in, dense_out):
        _, _, size, values, implementation = jobs[index]
        work = torch.empty((size, size), dtype=torch.float32, device=e.device).T
        factor.symmetric_eigenbasis(dense_in, dense_out, work, values, implementation)
        scratch[index] = values

    _factor_on_leaders(e, [(P, Q, size, None) for P, Q, size, _, _ in jobs], run, long_running=True)
    # eigenvalues live on the leader; hand them to everybody through a small segment
    for index, (_, _, size, values, _) in enumerate(jobs):
        leader = _leader_of(index, len(jobs), e.world)
        segment = e.comm.segment(f"eigenvalues{index}:{size}", size)
        if e.rank == leader:
            segment.local[:size].copy_(values)
        e.comm.barrier()
        table = e.leader_table(segment, leader)
        out = values.view(size, 1)
        _dist_gather_table(table, Source(segment, KIND_BLOCK_CYCLIC, size, 1, 1, 1, 1, 1, 1), IDENTITY, IDENTITY, size, 1, out)
        e.comm.barrier()


def initialize_basis(P: Tensor, Q: Tensor, work: Tensor, eigenvalues: Tensor, size: int, block_size: int, grid,
                     implementation: str) -> Tensor:
    e = engine_for(P.device, grid, block_size)
    initialize_bases(e, [(P, Q, size, eigenvalues, implementation)])
    return Q


def permute(matrix: Tensor, global_shape, row_order: Tensor, column_order: Tensor, block_size: int, grid, group=None) -> Tensor:
    e = engine_for(matrix.device, grid, block_size, group)
    rows, cols = global_shape
    source = e.stage_packed("stage", matrix, global_shape)
    e.comm.barrier()
    lr, lc = e.rows_of(rows), e.cols_of(cols)
    dist_gather(source, e.row_map(row_order), e.col_map(column_order), lr, lc, out=matrix[: max(1, lr), : max(1, lc)])
    e.comm.barrier()
    return matrix


# ---------------------------------------------------------------------------------------------
# The fused step
# ---------------------------------------------------------------------------------------------
def soap_step(gradient_shard: Tensor, state: MutableMapping[str, Any], *, global_shape, shard_dim: int, block_size: int,
              grid, beta: float, beta1: float, beta2: float, eps: float, interval: int, implementation: str,
              initializing: bool) -> Tensor:
    e = engine_for(gradient_shard.device, grid, block_size)
    rows, cols = global_shape
    device = gradient_shard.device
    with TIMER.stage("stage_gradient", device):
        shard_source = e.stage_shard(gradient_shard, global_shape, shard_dim)
        e.comm.barrier()

    if initializing:
        _gram_from_source(e, shard_source, global_shape, state["left_preconditioner"], beta, "left")
        _gram_from_source(e, shard_source, global_shape, state["right_preconditioner"], beta, "right")
        _mirror_upper(e, [("left", state["left_preconditioner"], rows), ("right", state["right_preconditioner"], cols)])
        e.comm.barrier()
        initialize_bases(e, [
            (state[f"{side}_preconditioner"], state[f"{side}_basis"], size,
             torch.empty(size, dtype=torch.float32, device=device), implementation)
            for side, size in (("left", rows), ("right", cols))])
        prepare_refresh(e, global_shape)
        state["step"] = 0
        return torch.zeros(gradient_shard.shape, dtype=torch.float32, device=device)

    step = int(state["step"]) + 1
    with TIMER.stage("basis_panels", device):
        left_plain, left_t = e.basis_panels(state["left_basis"], rows, "left")
        right_plain, right_t = e.basis_panels(state["right_basis"], cols, "right")
    lr, lc = e.rows_of(rows), e.cols_of(cols)
    bias2 = 1.0 - beta2**step
    adam = dict(beta1=beta1, beta2=beta2, eps=eps / math.sqrt(bias2),
                bias_correction1=1.0 - beta1**step, bias_correction2=bias2)
    main = torch.cuda.current_stream(device)
    x_panel = e.planes("x_panel", rows, e.rows_of(cols))   # X[:, my row class]: forward rotation and right Gram
    with TIMER.stage("pull_gradient_panel", device):
        if x_panel.cols > 0:
            dist_gather(shard_source, IDENTITY, e.row_map(), rows, x_panel.cols, planes=x_panel)

    def gram_updates(channel: int) -> None:
        # Gram EMAs with the current gradient; the right Gram reuses the pulled panel X[:, my row class]
        with TIMER.stage("gram", device):
            _gram_from_source(e, shard_source, global_shape, state["left_preconditioner"], beta, "left")
            _gram_from_source(e, shard_source, global_shape, state["right_preconditioner"], beta, "right", gathered=x_panel)
            _mirror_upper(e, [("left", state["left_preconditioner"], rows), ("right", state["right_preconditioner"], cols)],
                          channel=channel)
            e.comm.barrier(channel=channel)

    # The Gram updates depend on the gradient only.  They run on a stream of their own (with their own barrier
    # channel) beside the rotations, so that their products fill the SMs while the rotations wait for pulls and
    # barriers and vice versa.
    gram_done = None
    if OVERLAP_GRAM:
        side = e.side_stream()
        pulled = torch.cuda.Event()
        pulled.record(main)
        side.wait_event(pulled)
        with torch.cuda.stream(side):
            gram_updates(channel=1)
            gram_done = torch.cuda.Event()
            gram_done.record(side)
    # forward rotation straight from the tensor-parallel shards, Adam in the epilogue, update -> segment
    with TIMER.stage("rotate_forward+adam", device):
        _, u_view, u_source = e.packed_segment("update", global_shape)
        e.two_sided(shard_source, global_shape, left_plain, right_plain, panel=x_panel, gathered=True, mode=k.EPI_ADAM,
                    out=u_view[: max(1, lr), : max(1, lc)],
                    momentum=state["momentum"][: max(1, lr), : max(1, lc)],
                    variance=state["variance"][: max(1, lr), : max(1, lc)], adam=adam)
        e.comm.barrier()
    # backward rotation, result -> segment, then every rank pulls its tensor-parallel shard
    with TIMER.stage("rotate_backward", device):
        _, o_view, o_source = e.packed_segment("output", global_shape)
        e.two_sided(u_source, global_shape, left_t, right_t, mode=k.EPI_STORE, out=o_view[: max(1, lr), : max(1, lc)])
        e.comm.barrier()
        update = _pull_shard(e, o_source, global_shape, shard_dim)
    if gram_done is not None:
        main.wait_event(gram_done)
    else:
        gram_updates(channel=0)
    if step % interval == 0:
        with TIMER.stage("refresh", device):
            refresh(e, state, global_shape)
    state["step"] = step
    return update


def prepare_refresh(e: GridEngine, global_shape) -> None:
    """Create (collectively) the segments and workspaces a refresh needs, so that the first refresh does
    not pay for allocations and IPC handle exchanges in the middle of training."""
    from . import qr as qr_driver

    rows, cols = global_shape
    for index, size in enumerate((rows, cols)):
        e.packed_segment(f"factor_in{index}", (size, size))
        e.comm.segment(f"factor_out{index}:{size}", size * size)
        e.packed_segment("stage", (size, size))
        e.packed_segment("basis", (size, size))
        e.comm.segment(f"estimates:{size}:{e.nb}", max(1, numroc(size, e.nb, 0, e.Pc)))
        if e.rank == _leader_of(index, 2, e.world):
            qr_driver._workspace(size, e.device)
    if DISTRIBUTED_QR:
        from . import dist_qr

        dist_qr.prepare(e, [rows, cols])
    e.packed_segment("stage", global_shape)
    e.packed_segment("middle", (cols, rows))
    from . import local

    local.warm_refresh_kernels(e.device, sizes={rows, cols})


def refresh(e: GridEngine, state: MutableMapping[str, Any], global_shape) -> Tuple[Tensor, Tensor]:
    rows, cols = global_shape
    grid, nb = e.grid, e.nb
    device = e.device
    with TIMER.stage("refresh.momentum_out", device):
        rotate(state["momentum"], state["left_basis"], state["right_basis"], global_shape, nb, grid, "backward")
    with TIMER.stage("refresh.power_iteration", device):
        left_order = estimated_order(state["left_preconditioner"], state["left_basis"], state["left_work"], rows, nb, grid)
        right_order = estimated_order(state["right_preconditioner"], state["right_basis"], state["right_work"], cols, nb, grid)
    with TIMER.stage("refresh.qr", device):
        # the two factorisations are independent: they run at the same time on two different ranks
        qr_many(e, [(state["left_work"], state["left_basis"], rows, left_order),
                    (state["right_work"], state["right_basis"], cols, right_order)])

    with TIMER.stage("refresh.permute_variance", device):
        permute(state["variance"], global_shape, left_order, right_order, nb, grid)
    with TIMER.stage("refresh.momentum_in", device):
        rotate(state["momentum"], state["left_basis"], state["right_basis"], global_shape, nb, grid, "forward")
    return left_order, right_order

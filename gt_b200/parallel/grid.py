"""Process grids for block-distributed sparse attention.

``P = P_d * P_o * P_i`` ranks form a grid of row blocks (destinations / queries, index ``r``), column blocks (sources /
keys and values, index ``c``) and an optional head axis (index ``h``, ``P_i = 1`` on a 2D grid).  The padded node id
space ``[0, n_pad)`` is cut into ``P`` contiguous chunks; rank ``(r, c, h)`` owns chunk ``(c * P_d + r) * P_i + h``.
Hence

* column block ``c`` = ids ``[c * P_d * P_i * chunk, (c + 1) * P_d * P_i * chunk)`` (contiguous); its owners are the
  ranks ``(., c, .)``;
* row block ``r`` = the ``P_o * P_i`` chunks owned by the ranks ``(r, ., .)`` in ``(c, h)`` order (what an all-gather
  over the row group returns).

Rank ``(r, c, h)`` computes the block ``A[row block r, column block c]`` for head group ``h``.  This is the ownership
rule of the reference's ``Grid2D`` / ``Grid3D`` (``gt3d/gt3d/dist/grid2d.py:1-23,154-206``, ``grid3d.py:1-18,89-138``),
so partitions and state dicts written for one are valid for the other.

``BlockGrid`` is pure index arithmetic and can be built for any rank without a process group (``BlockGrid.virtual``):
ownership, expander generation and communication plans are unit-testable on one CPU process.  ``Grid2D`` / ``Grid3D``
add the ``torch.distributed`` groups (``row_group``: ranks sharing ``(r, h)``; ``col_group``: ranks sharing ``(c, h)``;
``head_group``: ranks sharing ``(r, c)``).
"""
from typing import Optional

import torch
import torch.distributed as dist


class BlockGrid:
    def __init__(self, p_rows: int, p_cols: int, p_heads: int, num_nodes: int, rank: int, n_pad: Optional[int] = None,
                 layout: str = "row_major"):
        if layout not in ("row_major", "col_major"):
            raise ValueError(layout)
        self.p_rows, self.p_cols, self.p_heads, self.layout = int(p_rows), int(p_cols), int(p_heads), layout
        self.world = self.p_rows * self.p_cols * self.p_heads
        self.rank = int(rank)
        self.num_nodes = int(num_nodes)
        if n_pad is None:
            self.chunk = -(-self.num_nodes // self.world)
        else:
            if n_pad % self.world or n_pad < num_nodes:
                raise ValueError(f"n_pad={n_pad} must be a multiple of {self.world} and >= {num_nodes}")
            self.chunk = n_pad // self.world
        self.n_pad = self.chunk * self.world
        self.r, self.c, self.h = self.coords_of(self.rank)
        lo, hi = self.owned_range()
        self.valid_mask = torch.arange(lo, hi) < self.num_nodes
        self.row_group = self.col_group = self.head_group = None

    @classmethod
    def virtual(cls, p_rows, p_cols, num_nodes, rank, p_heads=1, n_pad=None, layout="row_major"):
        """Geometry of ``rank`` without any process group."""
        return cls(p_rows, p_cols, p_heads, num_nodes, rank, n_pad, layout)

    # ---- rank <-> coordinates ----------------------------------------------------------------------------------
    def rank_of(self, r, c, h=0):
        if self.layout == "row_major":
            return (r * self.p_cols + c) * self.p_heads + h
        return (c * self.p_rows + r) * self.p_heads + h

    def coords_of(self, rank):
        rc, h = divmod(rank, self.p_heads)
        if self.layout == "row_major":
            r, c = divmod(rc, self.p_cols)
        else:
            c, r = divmod(rc, self.p_rows)
        return r, c, h

    def to(self, device):
        self.valid_mask = self.valid_mask.to(device)
        return self

    # ---- ownership ---------------------------------------------------------------------------------------------
    def chunk_of(self, r, c, h=0):
        return (c * self.p_rows + r) * self.p_heads + h

    def owned_range(self, r=None, c=None, h=None):
        r = self.r if r is None else r
        c = self.c if c is None else c
        h = self.h if h is None else h
        k = self.chunk_of(r, c, h)
        return k * self.chunk, (k + 1) * self.chunk

    def owner_of(self, node_ids):
        """``(r, c, h)`` of the owner of every (padded) node id (tensors)."""
        k = node_ids // self.chunk
        h = k % self.p_heads
        rc = k // self.p_heads
        return rc % self.p_rows, rc // self.p_rows, h

    def col_block_range(self, c=None):
        c = self.c if c is None else c
        size = self.p_rows * self.p_heads * self.chunk
        return c * size, (c + 1) * size

    def row_block_ranges(self, r=None):
        r = self.r if r is None else r
        return [self.owned_range(r, c, h) for c in range(self.p_cols) for h in range(self.p_heads)]

    def row_block_ids(self, r=None):
        return torch.cat([torch.arange(lo, hi) for lo, hi in self.row_block_ranges(r)])

    @property
    def n_row_block(self):
        return self.p_cols * self.p_heads * self.chunk

    @property
    def n_col_block(self):
        return self.p_rows * self.p_heads * self.chunk

    @property
    def row_pos(self):
        """Index of my chunk inside my row block (all-gather order over the row group, then the head group)."""
        return self.c * self.p_heads + self.h

    @property
    def col_pos(self):
        return self.r * self.p_heads + self.h

    def global_to_row_local(self, gid):
        r, c, h = self.owner_of(gid)
        return (c * self.p_heads + h) * self.chunk + (gid - self.chunk_of(r, c, h) * self.chunk)

    def global_to_col_local(self, gid):
        _, c, _ = self.owner_of(gid)
        return gid - c * self.p_rows * self.p_heads * self.chunk

    def take_owned(self, x_global):
        """Owned chunk of a global per-node tensor, zero-padded past ``num_nodes``."""
        lo, hi = self.owned_range()
        out = x_global.new_zeros((self.chunk,) + tuple(x_global.shape[1:]))
        n = min(hi, self.num_nodes, x_global.shape[0]) - lo
        if n > 0:
            out[:n] = x_global[lo:lo + n]
        return out

    def local_block(self, edge_index, edge_type=None, weight=None):
        """Edges with destination in my row block and source in my column block, in local ``(col-local src, row-local
        dst)`` numbering.  For tests and graphs that fit on one host; large graphs arrive pre-partitioned."""
        src, dst = edge_index[0], edge_index[1]
        mine = (self.owner_of(dst)[0] == self.r) & (self.owner_of(src)[1] == self.c)
        ei = torch.stack([self.global_to_col_local(src[mine]), self.global_to_row_local(dst[mine])])
        out = (ei, edge_type[mine] if edge_type is not None else None)
        return out + (weight[mine],) if weight is not None else out

    def __repr__(self):
        return (f"{type(self).__name__}({self.p_rows}x{self.p_cols}x{self.p_heads}, rank {self.rank} = "
                f"(r={self.r}, c={self.c}, h={self.h}), N={self.num_nodes}, chunk={self.chunk})")


_GROUP_NAMES = {}


def group_name(group) -> str:
    """'row' / 'col' / 'head' / 'world' for the groups created by the grids (used by timers and statistics)."""
    return _GROUP_NAMES.get(id(group), "world" if group is None else "?")


def group_size(group) -> int:
    if group is None and not dist.is_initialized():
        return 1
    return dist.get_world_size(group)


class _DistGrid(BlockGrid):
    def __init__(self, p_rows, p_cols, p_heads, num_nodes, n_pad=None, layout="row_major"):
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised before a grid is built "
                               "(use BlockGrid.virtual for geometry without a process group)")
        world = dist.get_world_size()
        if world != p_rows * p_cols * p_heads:
            raise ValueError(f"grid {p_rows}x{p_cols}x{p_heads} does not match world size {world}")
        super().__init__(p_rows, p_cols, p_heads, num_nodes, dist.get_rank(), n_pad, layout)
        # every rank must create every group, in the same order
        rows, cols, heads = {}, {}, {}
        for r in range(p_rows):
            for h in range(p_heads):
                rows[(r, h)] = dist.new_group([self.rank_of(r, c, h) for c in range(p_cols)])
        for c in range(p_cols):
            for h in range(p_heads):
                cols[(c, h)] = dist.new_group([self.rank_of(r, c, h) for r in range(p_rows)])
        if p_heads > 1:
            for r in range(p_rows):
                for c in range(p_cols):
                    heads[(r, c)] = dist.new_group([self.rank_of(r, c, h) for h in range(p_heads)])
        self.row_group = rows[(self.r, self.h)]
        self.col_group = cols[(self.c, self.h)]
        self.head_group = heads.get((self.r, self.c))
        self.row_ranks = [self.rank_of(self.r, c, self.h) for c in range(p_cols)]
        self.col_ranks = [self.rank_of(r, self.c, self.h) for r in range(p_rows)]
        self.head_ranks = [self.rank_of(self.r, self.c, h) for h in range(p_heads)]
        _GROUP_NAMES[id(self.row_group)] = "row"
        _GROUP_NAMES[id(self.col_group)] = "col"
        if self.head_group is not None:
            _GROUP_NAMES[id(self.head_group)] = "head"


class Grid2D(_DistGrid):
    """``Grid2D(p_rows, p_cols, num_nodes, n_pad=None, layout='row_major')`` on the default process group."""

    def __init__(self, p_rows, p_cols, num_nodes, n_pad=None, layout="row_major", timers=False):
        super().__init__(p_rows, p_cols, 1, num_nodes, n_pad, layout)
        if timers:
            from ..utils.timers import enable_timers
            enable_timers(True)


class Grid3D(_DistGrid):
    """``Grid3D(p_rows, p_cols, p_heads, num_nodes, n_pad=None)``: the 2D block grid times a Ulysses head axis (the
    ``P_i`` ranks of a head group are consecutive)."""

    def __init__(self, p_rows, p_cols, p_heads, num_nodes, n_pad=None, timers=False):
        super().__init__(p_rows, p_cols, p_heads, num_nodes, n_pad, "row_major")
        if timers:
            from ..utils.timers import enable_timers
            enable_timers(True)


def make_grid(shape, num_nodes, n_pad=None, layout="row_major", timers=False):
    """Grid for ``--grid P_d P_o [P_i]``."""
    if len(shape) == 3:
        return Grid3D(shape[0], shape[1], shape[2], num_nodes, n_pad, timers=timers)
    return Grid2D(shape[0], shape[1], num_nodes, n_pad, layout, timers=timers)

"""Sparse structures of an attention / aggregation block.

A block is the sub-matrix ``A[rows, cols]`` of the attention mask a rank computes: destination (query) rows and
source (key / value) columns in block-local numbering.  ``BlockCSR`` owns every index array the kernels need:

* the CSR in canonical ``(dst, src)`` order (``crow``, ``col``, ``etype``) — the same canonical order as the
  reference's ``build_csr`` (``gt3d/gt3d/attention/backend_torch.py:24-42``) so results do not depend on the order
  edges arrive in;
* the transposed structure (CSC: ``ccol``, ``rowidx``, ``etype_t`` and the position of every CSC entry in the CSR)
  used by the atomic-free column pass of the backward (reference: ``build_csc``, ``triton_kernel.py:333``);
* *segment plans*: rows (columns) with more than ``seg_edges`` entries are cut into segments so that one warp never
  walks more than ``seg_edges`` edges; the partial results of a cut row are merged by a combine kernel
  (split-KV, reference ``build_row_segments`` ``triton_kernel.py:301``);
* the doubly-compressed row list (rows that own at least one edge) for hypersparse sub-blocks
  (reference ``build_dcsr`` ``triton_tiled.py:111``).

All index arrays are int32 (a block never holds 2^31 edges); construction works on CPU or CUDA tensors.
"""
import os
from dataclasses import dataclass, field
from typing import Optional

import torch


def build_csr(edge_index: torch.Tensor, num_rows: int, edge_type: Optional[torch.Tensor] = None):
    """Sort edges by (destination, edge type, source).  Returns ``(crow[int64 n+1], col[int64 E], etype or None, perm)``
    where ``perm`` maps CSR position -> position in the input edge list.  Grouping a row's edges by type lets the kernels
    keep the per-type gate slice in registers and reload it only when the type changes."""
    src, dst = edge_index[0].long(), edge_index[1].long()
    if src.numel() == 0:
        z = torch.zeros(0, dtype=torch.long, device=edge_index.device)
        return torch.zeros(num_rows + 1, dtype=torch.long, device=edge_index.device), z, (z if edge_type is not None else None), z
    width = int(src.max().item()) + 1
    if edge_type is not None:
        nt = int(edge_type.max().item()) + 1
        perm = torch.argsort((dst * nt + edge_type.long()) * width + src, stable=True)
    else:
        perm = torch.argsort(dst * width + src, stable=True)
    counts = torch.bincount(dst, minlength=num_rows)
    crow = torch.zeros(num_rows + 1, dtype=torch.long, device=edge_index.device)
    torch.cumsum(counts, 0, out=crow[1:])
    col = src[perm].contiguous()
    et = edge_type[perm].contiguous() if edge_type is not None else None
    return crow, col, et, perm


def rows_of_edges(crow: torch.Tensor) -> torch.Tensor:
    """Row index of every CSR entry (``[E]`` int64)."""
    n = crow.numel() - 1
    deg = (crow[1:] - crow[:-1]).long()
    return torch.repeat_interleave(torch.arange(n, device=crow.device), deg)


def _segments(ptr: torch.Tensor, seg_edges: int):
    """Cut every row of a pointer array into pieces of at most ``seg_edges`` entries.

    Returns ``(seg_row, seg_beg, seg_end, seg_slot, split_rows, split_ptr)``: ``seg_slot[s]`` is -1 when the row of
    segment ``s`` has a single segment (the kernel writes the row's result directly) and otherwise the index of the
    segment's scratch slot; ``split_rows`` lists the rows that were cut and ``split_ptr`` their slot ranges.
    Empty rows get one empty segment so that their outputs are still written (zeros)."""
    ptr = ptr.long()
    deg = ptr[1:] - ptr[:-1]
    nseg_row = torch.clamp((deg + seg_edges - 1) // seg_edges, min=1)
    seg_row = torch.repeat_interleave(torch.arange(deg.numel(), device=ptr.device), nseg_row)
    first = torch.zeros(deg.numel() + 1, dtype=torch.long, device=ptr.device)
    torch.cumsum(nseg_row, 0, out=first[1:])
    k = torch.arange(seg_row.numel(), device=ptr.device) - first[seg_row]          # index of the segment inside its row
    seg_beg = ptr[seg_row] + k * seg_edges
    seg_end = torch.minimum(seg_beg + seg_edges, ptr[seg_row + 1])
    is_split = nseg_row > 1
    split_rows = torch.nonzero(is_split).squeeze(1)
    split_cnt = nseg_row[split_rows]
    split_ptr = torch.zeros(split_rows.numel() + 1, dtype=torch.long, device=ptr.device)
    torch.cumsum(split_cnt, 0, out=split_ptr[1:])
    seg_slot = torch.full_like(seg_row, -1)
    if split_rows.numel():
        slot_first = torch.full((deg.numel(),), -1, dtype=torch.long, device=ptr.device)
        slot_first[split_rows] = split_ptr[:-1]
        sel = is_split[seg_row]
        seg_slot[sel] = slot_first[seg_row[sel]] + k[sel]
    if BALANCE_WARPS > 0 and seg_row.numel() > BALANCE_WARPS:
        perm = _balanced_order(seg_end - seg_beg, BALANCE_WARPS)
        seg_row, seg_beg, seg_end, seg_slot = seg_row[perm], seg_beg[perm], seg_end[perm], seg_slot[perm]
    i32 = torch.int32
    return (seg_row.to(i32), seg_beg.to(i32), seg_end.to(i32), seg_slot.to(i32), split_rows.to(i32), split_ptr.to(i32))


# The kernels are persistent: warp w of a grid of BALANCE_WARPS warps walks the segments w, w + W, w + 2 W, ...  Degrees of real
# graphs are heavy-tailed, so with the segments in row order a warp that happens to draw a few hub segments runs far longer than
# the average and the launch ends with most SMs idle.  The segments are therefore sorted by length (longest first) and dealt to
# the warps in serpentine order, which equalises the number of edges per warp to within one short segment (longest-processing-
# time scheduling done once on the host; the kernels need no work queue and stay deterministic).  0 keeps the row order.
BALANCE_WARPS = int(os.environ.get("GT_PLAN_BALANCE", str(148 * 24 * 4)))


def _balanced_order(length: torch.Tensor, n_warps: int) -> torch.Tensor:
    """Permutation ``perm`` such that ``segments[perm]`` walked with stride ``n_warps`` gives every warp the same work."""
    n = length.numel()
    order = torch.argsort(length, descending=True, stable=True)
    p = torch.arange(n, device=length.device)
    rnd, k = p // n_warps, p % n_warps
    full = (rnd + 1) * n_warps <= n                                  # the last, partial round is dealt forwards
    warp = torch.where(((rnd % 2) == 1) & full, n_warps - 1 - k, k)
    pos = rnd * n_warps + warp
    perm = torch.empty_like(order)
    perm[pos] = order
    return perm


@dataclass
class SegmentPlan:
    """Work list of one pass: one warp per segment (see ``_segments``)."""
    seg_row: torch.Tensor
    seg_beg: torch.Tensor
    seg_end: torch.Tensor
    seg_slot: torch.Tensor
    split_rows: torch.Tensor
    split_ptr: torch.Tensor
    seg_edges: int

    @property
    def num_segments(self) -> int:
        return int(self.seg_row.numel())

    @property
    def num_slots(self) -> int:
        # cached as a Python int at first use: the launch wrappers must not synchronise (CUDA-graph capture)
        if not hasattr(self, "_n_slots"):
            self._n_slots = int(self.split_ptr[-1].item()) if self.split_ptr.numel() else 0
        return self._n_slots

    def tensors(self):
        return [self.seg_row, self.seg_beg, self.seg_end, self.seg_slot, self.split_rows, self.split_ptr]


@dataclass
class BlockCSR:
    """CSR (+ lazily built CSC, segment plans, DCSR row list) of one block; see the module docstring."""
    n_rows: int
    n_cols: int
    crow: torch.Tensor                      # int32 [n_rows + 1]
    col: torch.Tensor                       # int32 [E]
    etype: Optional[torch.Tensor] = None    # int32 [E]
    weight: Optional[torch.Tensor] = None   # per-entry value (aggregation blocks), CSR order
    _cache: dict = field(default_factory=dict, repr=False)

    # ---- construction --------------------------------------------------------------------------------------
    @classmethod
    def from_edges(cls, edge_index, n_rows, n_cols, edge_type=None, weight=None, return_perm=False):
        crow, col, et, perm = build_csr(edge_index, n_rows, edge_type)
        if col.numel() >= 2 ** 31:
            raise ValueError("a block must hold fewer than 2^31 edges")
        if col.numel() and int(col.max().item()) >= n_cols:
            raise ValueError("source index outside the column block")
        blk = cls(int(n_rows), int(n_cols), crow.to(torch.int32).contiguous(), col.to(torch.int32).contiguous(),
                  et.to(torch.int32).contiguous() if et is not None else None,
                  weight[perm].contiguous() if weight is not None else None)
        return (blk, perm) if return_perm else blk

    @classmethod
    def from_csr(cls, crow, col, etype=None, n_cols=None, weight=None):
        n_cols = int(n_cols if n_cols is not None else (int(col.max().item()) + 1 if col.numel() else 1))
        return cls(int(crow.numel() - 1), n_cols, crow.to(torch.int32).contiguous(), col.to(torch.int32).contiguous(),
                   etype.to(torch.int32).contiguous() if etype is not None else None, weight)

    @property
    def num_edges(self) -> int:
        return int(self.col.numel())

    @property
    def device(self):
        return self.crow.device

    def to(self, device):
        dev = torch.device(device)
        if dev == self.crow.device:
            return self
        mv = lambda t: t.to(dev) if t is not None else None          # noqa: E731
        return BlockCSR(self.n_rows, self.n_cols, mv(self.crow), mv(self.col), mv(self.etype), mv(self.weight))

    # ---- derived structures ----------------------------------------------------------------------------------
    def rows(self) -> torch.Tensor:
        """Destination row of every CSR entry (int32 [E])."""
        if "rows" not in self._cache:
            self._cache["rows"] = rows_of_edges(self.crow).to(torch.int32)
        return self._cache["rows"]

    def csc(self):
        """``(ccol[int32 n_cols+1], rowidx[int32 E], etype_t, pos[int32 E], weight_t)``: entries grouped by source
        column, destinations ascending inside a column; ``pos`` is the CSR position of every CSC entry."""
        if "csc" not in self._cache:
            col = self.col.long()
            if self.etype is not None:                     # inside a column: grouped by type, then destination ascending
                nt = int(self.etype.max().item()) + 1 if self.etype.numel() else 1
                pos = torch.argsort(col * nt + self.etype.long(), stable=True)
            else:
                pos = torch.argsort(col, stable=True)
            ccol = torch.zeros(self.n_cols + 1, dtype=torch.long, device=self.device)
            torch.cumsum(torch.bincount(col, minlength=self.n_cols), 0, out=ccol[1:])
            rowidx = self.rows()[pos]
            et_t = self.etype[pos].contiguous() if self.etype is not None else None
            w_t = self.weight[pos].contiguous() if self.weight is not None else None
            self._cache["csc"] = (ccol.to(torch.int32), rowidx.contiguous(), et_t, pos.to(torch.int32), w_t)
        return self._cache["csc"]

    def row_plan(self, seg_edges: int = 256) -> SegmentPlan:
        key = ("row_plan", seg_edges)
        if key not in self._cache:
            self._cache[key] = SegmentPlan(*_segments(self.crow, seg_edges), seg_edges)
            self._cache[key].num_slots
        return self._cache[key]

    def col_plan(self, seg_edges: int = 256) -> SegmentPlan:
        key = ("col_plan", seg_edges)
        if key not in self._cache:
            self._cache[key] = SegmentPlan(*_segments(self.csc()[0], seg_edges), seg_edges)
            self._cache[key].num_slots
        return self._cache[key]

    def dcsr_rows(self) -> torch.Tensor:
        """Rows that own at least one edge (int32, ascending): the row list of the doubly-compressed CSR."""
        if "dcsr" not in self._cache:
            deg = self.crow[1:] - self.crow[:-1]
            self._cache["dcsr"] = torch.nonzero(deg > 0).squeeze(1).to(torch.int32)
        return self._cache["dcsr"]

    def need_sets(self):
        """(non-empty rows, referenced columns), sorted int64: the rows a sparsity-aware collective must move."""
        return self.dcsr_rows().long(), torch.unique(self.col.long())

    def compacted(self, rows_need: torch.Tensor, col_remap: torch.Tensor, n_cols_c: int) -> "BlockCSR":
        """The same entries over the row subset ``rows_need`` (which must include every non-empty row) with the
        columns renumbered through ``col_remap`` (block-local -> compact, -1 = absent)."""
        crow = self.crow.long()
        rows_need = rows_need.long()
        crow_c = torch.cat([crow[rows_need], crow[-1:]])
        col_c = col_remap.long()[self.col.long()]
        if col_c.numel() and int(col_c.min().item()) < 0:
            raise ValueError("a referenced column is missing from the column need set")
        return BlockCSR(int(rows_need.numel()), int(n_cols_c), crow_c.to(torch.int32).contiguous(),
                        col_c.to(torch.int32).contiguous(), self.etype, self.weight)

    def nbytes(self, seen: Optional[set] = None) -> int:
        """Bytes held by the structure including cached plans; storages listed in ``seen`` are skipped."""
        seen = set() if seen is None else seen
        total = 0

        def visit(obj):
            nonlocal total
            if torch.is_tensor(obj):
                if obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, SegmentPlan):
                for t in obj.tensors():
                    visit(t)
            elif isinstance(obj, (tuple, list)):
                for t in obj:
                    visit(t)

        for t in (self.crow, self.col, self.etype, self.weight):
            visit(t)
        for v in self._cache.values():
            visit(v)
        return total

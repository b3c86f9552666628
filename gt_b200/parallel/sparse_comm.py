"""Sparsity-aware row collectives: gather / reduce-scatter restricted to the rows a rank's tile references.

The graph is static, so the rows of a gathered block that a rank touches are known up front: the non-empty *columns* of
its tile for the K / V-side gather, the non-empty *rows* for the Q-side gather and the partials' reduce-scatter.  A
``SparseRowPlan`` stores these need sets in both directions (what I fetch from every peer, what every peer fetches from
me); the tile's CSR is renumbered once to the compact index space (``BlockCSR.compacted``).

Two transports implement a plan:

* ``transport="a2a"`` — an all-to-all-v with static split sizes (NCCL or gloo): the sender packs its rows with one
  ``index_select``; the reduce-scatter is the transposed all-to-all-v followed by a deterministic segmented sum.
  This is the reference's mechanism (``gt3d/gt3d/dist/sparse_comm.py:59-202``).
* ``transport="pull"`` — receiver-driven: every rank publishes its chunk in a symmetric buffer and a kernel reads
  exactly the needed rows from the peers' memory over NVLink (``pull_gather``), or sums the partial rows that the
  peers hold for my rows in a fixed peer order (``pull_reduce``).  No packing, no split sizes, no NCCL; this is the
  sm_100a replacement of the reference's NVSHMEM ``pullcomm`` prototype (``dist/pullcomm/pullcomm.cu:50-108``).

Inside one NVSwitch domain an all-to-all runs at the same per-rank rate as an all-gather, so ``worthwhile`` only
compares the share of rows moved against a margin (the reference's per-node-layout table collapses to one entry).
"""
import os

import torch
import torch.distributed as dist

from .grid import group_size

MARGIN = float(os.environ.get("GT_SPARSE_MARGIN", "0.9"))
A2A_OVER_AG = 1.0      # NVSwitch: every peer at full bandwidth, no intra / inter-node distinction


def _idt(n):
    return torch.int32 if n < 2 ** 31 else torch.int64


class SparseRowPlan:
    """Rows of a block gathered over ``group`` (every rank contributes ``rows_per_rank`` rows) that this rank needs.

    ``need_local``: sorted unique block-local row indices.  After construction: ``n_need``, ``remap`` (block-local ->
    compact, -1 = absent), ``recv_counts`` / ``send_counts`` per peer, ``send_idx`` (rows of my chunk the peers need,
    grouped by peer), ``share`` (= max over all ranks of rows moved / rows of the block), ``n_need_max`` (largest need set of any
    rank).  Plans are built collectively: every rank constructs the plan of its own group at the same point of the program."""

    def __init__(self, group, rows_per_rank: int, need_local: torch.Tensor, name: str = "?", transport: str = "a2a",
                 heap=None):
        self.group, self.rows_per_rank, self.name, self.transport, self.heap = group, int(rows_per_rank), name, transport, heap
        g = group_size(group)
        me = dist.get_rank(group) if g > 1 else 0
        self.g, self.me = g, me
        dev = need_local.device
        need_local = need_local.long()
        n_blk = g * self.rows_per_rank
        if need_local.numel() and (int(need_local.min()) < 0 or int(need_local.max()) >= n_blk):
            raise ValueError(f"plan {name}: need set outside the block")
        self.n_need = int(need_local.numel())
        owner = torch.div(need_local, self.rows_per_rank, rounding_mode="floor")
        local_idx = need_local - owner * self.rows_per_rank
        recv = torch.bincount(owner, minlength=g)
        if g == 1:
            send, send_idx = recv.clone(), local_idx
        else:
            send = torch.empty_like(recv)
            dist.all_to_all_single(send, recv, group=group)
            tot = int(send.sum().item())
            send_idx = torch.empty(tot, dtype=torch.long, device=dev)
            dist.all_to_all_single(send_idx, local_idx.contiguous(), output_split_sizes=send.tolist(),
                                   input_split_sizes=recv.tolist(), group=group)
        self.recv_counts, self.send_counts = recv.tolist(), send.tolist()
        self.n_send = int(sum(self.send_counts))
        self.send_idx = send_idx.to(_idt(self.rows_per_rank)).contiguous()
        # deterministic accumulation of the reduce-scatter: received rows sorted by the owned row they add to
        order = torch.argsort(send_idx, stable=True)
        self.acc_perm = order.to(torch.int32).contiguous()
        ptr = torch.zeros(self.rows_per_rank + 1, dtype=torch.long, device=dev)
        torch.cumsum(torch.bincount(send_idx, minlength=self.rows_per_rank), 0, out=ptr[1:])
        self.acc_ptr = ptr.to(torch.int32).contiguous()
        self.acc_row = send_idx[order].contiguous()
        remap = torch.full((n_blk,), -1, dtype=_idt(n_blk), device=dev)
        remap[need_local] = torch.arange(self.n_need, dtype=remap.dtype, device=dev)
        self.remap = remap
        self.need_local = need_local.to(_idt(n_blk)).contiguous()
        self.need_owner = owner.to(torch.int32).contiguous()              # pull transport: (peer, row) per compact row
        self.need_row = local_idx.to(torch.int32).contiguous()
        # Maxima over ALL ranks, not over this group: every rank builds the plan of its own group at the same point of the program,
        # and decisions and buffer sizes derived from a plan must agree across groups too.  A rank belongs to a row group and a
        # column group; if two row groups sized a symmetric-heap buffer differently (or one took the sparse and one the dense
        # path), the heap offsets of their members would differ from then on, and the column groups, whose members come from
        # different row groups, would no longer find their buffers at the same offset on every member.
        sh = torch.tensor([self.n_need / max(n_blk, 1), self.n_send / max(n_blk, 1), float(self.n_need)], dtype=torch.float64, device=dev)
        if g > 1:
            dist.all_reduce(sh, op=dist.ReduceOp.MAX)
        self.share, self.share_send, self.n_need_max = float(sh[0]), float(sh[1]), int(sh[2])
        self.ratio = A2A_OVER_AG

    def worthwhile(self, threshold=None):
        lim = self.ratio * MARGIN if threshold is None else threshold
        return max(self.share, self.share_send) <= lim

    def drop_remap(self):
        self.remap = None

    def nbytes(self, seen=None):
        seen = set() if seen is None else seen
        tot = 0
        for t in (self.send_idx, self.acc_perm, self.acc_ptr, self.acc_row, self.remap, self.need_local, self.need_owner,
                  self.need_row):
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                tot += t.numel() * t.element_size()
        return tot

    # ---- raw collectives -----------------------------------------------------------------------------------------
    @staticmethod
    def _pad16(x):
        """Rows padded to a multiple of 16 bytes (unaligned rows halve the transfer rate and break vector loads)."""
        unit = 16 // x.element_size()
        pad = (-x.shape[1]) % unit
        return (torch.nn.functional.pad(x, (0, pad)) if pad else x), x.shape[1]

    @staticmethod
    def _pad8(x):
        """Rows padded to a multiple of 8 elements (the peer-memory kernels move 8-element vectors)."""
        pad = (-x.shape[1]) % 8
        return (torch.nn.functional.pad(x, (0, pad)) if pad else x), x.shape[1]

    def gather(self, x, async_op=False):
        """``x [rows_per_rank, ...] -> [n_need, ...]``; ``async_op`` returns ``(work, finalize)``."""
        shp = tuple(x.shape[1:])
        x2 = x.contiguous().view(x.shape[0], -1)
        if self.g == 1:
            out = x2.index_select(0, self.send_idx.long()).view(-1, *shp)
            return (None, (lambda: out)) if async_op else out
        if self.transport == "pull" and self.heap.reaches(x, self.group):
            xp, width = self._pad8(x2)
            out = self.heap.pull_gather(xp, self)[:, :width].reshape(-1, *shp)
            return (None, (lambda: out)) if async_op else out
        x2, width = self._pad16(x2)
        send = x2.index_select(0, self.send_idx.long())
        out = x2.new_empty(self.n_need, x2.shape[1])
        work = dist.all_to_all_single(out, send, output_split_sizes=self.recv_counts, input_split_sizes=self.send_counts,
                                      group=self.group, async_op=async_op)
        fin = lambda _keep=send: out[:, :width].reshape(-1, *shp)          # noqa: E731  (send buffer outlives the op)
        return (work, fin) if async_op else fin()

    def reduce_scatter(self, y, async_op=False):
        """``y [n_need, ...]`` partial rows ``-> [rows_per_rank, ...]`` summed over the ranks that hold each row."""
        shp = tuple(y.shape[1:])
        y2 = y.contiguous().view(y.shape[0], -1)
        if self.g == 1:
            out = self._accumulate(y2).view(-1, *shp)
            return (None, (lambda: out)) if async_op else out
        if self.transport == "pull" and self.heap.reaches(y, self.group):
            yp, width = self._pad8(y2)
            out = self.heap.pull_reduce(yp, self)[:, :width].reshape(-1, *shp)
            return (None, (lambda: out)) if async_op else out
        y2, width = self._pad16(y2)
        recv = y2.new_empty(self.n_send, y2.shape[1])
        work = dist.all_to_all_single(recv, y2, output_split_sizes=self.send_counts, input_split_sizes=self.recv_counts,
                                      group=self.group, async_op=async_op)

        def fin(_keep=y2):
            return self._accumulate(recv)[:, :width].reshape(-1, *shp)

        return (work, fin) if async_op else fin()

    def _accumulate(self, rows):
        """``[n_send, F]`` received rows -> ``[rows_per_rank, F]``: a segmented sum in a fixed order (deterministic)."""
        out = torch.zeros(self.rows_per_rank, rows.shape[1], dtype=rows.dtype, device=rows.device)
        if self.n_send == 0:
            return out
        if rows.is_cuda:
            from ..ops import native
            return native.segment_sum_rows(rows, self.acc_perm, self.acc_ptr, out)
        adt = torch.float32 if rows.dtype in (torch.bfloat16, torch.float16) else rows.dtype
        acc = torch.zeros(self.rows_per_rank, rows.shape[1], dtype=adt, device=rows.device)
        acc.index_add_(0, self.acc_row, rows[self.acc_perm.long()].to(adt))
        return acc.to(rows.dtype)

    def __repr__(self):
        return (f"SparseRowPlan({self.name}: G={self.g} rows/rank={self.rows_per_rank} need {self.n_need} "
                f"share {self.share:.3f} send {self.share_send:.3f} transport {self.transport})")


def wait_work(work):
    if work is not None:
        work.wait()


class _SparseAllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan, wire):
        ctx.plan, ctx.wire, ctx.dtype = plan, wire, x.dtype
        return plan.gather(x if wire is None else x.to(wire)).to(x.dtype)

    @staticmethod
    def backward(ctx, grad):
        g = grad if ctx.wire is None else grad.to(ctx.wire)
        return ctx.plan.reduce_scatter(g).to(ctx.dtype), None, None


class _SparseReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, plan, wire):
        ctx.plan, ctx.wire, ctx.dtype = plan, wire, y.dtype
        return plan.reduce_scatter(y if wire is None else y.to(wire)).to(y.dtype)

    @staticmethod
    def backward(ctx, grad):
        g = grad if ctx.wire is None else grad.to(ctx.wire)
        return ctx.plan.gather(g).to(ctx.dtype), None, None


def sparse_all_gather(x, plan, wire=None):
    return _SparseAllGather.apply(x, plan, wire)


def sparse_reduce_scatter(y, plan, wire=None):
    return _SparseReduceScatter.apply(y, plan, wire)


def tile_need_sets(csr):
    """(non-empty rows, referenced columns) of a tile, sorted int64."""
    return csr.need_sets()


def build_sparse_comm(grid, attn_block, gcn_block, threshold=None, attn_subs=None, gcn_subs=None, transport="a2a",
                      heap=None):
    """Plans of the row group (Q-side gather, partials reduce-scatter) and the column group (K / V-side gather, dx
    reduce-scatter) for this rank's tile, plus the tiles renumbered to the plans' compact index spaces.  The need sets
    are the union of the attention and GCN tiles.  A plan is used only when ``worthwhile``; the other collective stays
    dense.  ``attn_subs`` / ``gcn_subs``: the column sub-blocks of the streamed layer (one column plan per sub-block).
    Returns ``(dict(row=, col=, cols=, attn=, gcn=) or None, info)`` (reference: ``exphormer_dist.py:299-367``)."""
    from .attention import AttentionBlock
    dev = attn_block.csr.device
    n_rows, n_cols = grid.n_row_block, grid.n_col_block
    g_row, g_col = group_size(grid.row_group), group_size(grid.col_group)

    def need(a_blk, g_blk):
        rows, cols = a_blk.csr.need_sets()
        if g_blk is not None:
            r2, c2 = g_blk.csr64.need_sets()
            rows, cols = torch.unique(torch.cat([rows, r2])), torch.unique(torch.cat([cols, c2]))
        return rows, cols

    rows, cols = need(attn_block, gcn_block)
    plan_row = SparseRowPlan(grid.row_group, n_rows // g_row, rows, "row", transport, heap)
    plan_col = SparseRowPlan(grid.col_group, n_cols // g_col, cols, "col", transport, heap)
    thr_row, thr_col = threshold if isinstance(threshold, (tuple, list)) else (threshold, threshold)
    use_row, use_col = plan_row.worthwhile(thr_row), plan_col.worthwhile(thr_col)
    info = dict(row_share=plan_row.share, col_share=plan_col.share, row_ratio=plan_row.ratio, col_ratio=plan_col.ratio,
                row_rows=plan_row.n_need, col_rows=plan_col.n_need, use_row=use_row, use_col=use_col,
                n_row_block=n_rows, n_col_block=n_cols)
    if not (use_row or use_col):
        return None, info
    rows_eff = rows if use_row else torch.arange(n_rows, device=dev)
    out = dict(row=plan_row if use_row else None, col=None, cols=None)
    ident = lambda n: torch.arange(n, device=dev)                                # noqa: E731
    if attn_subs is None:
        out["col"] = plan_col if use_col else None
        col_remap = plan_col.remap.long() if use_col else ident(n_cols)
        n_cols_c = plan_col.n_need if use_col else n_cols
        out["attn"] = attn_block.compacted(rows_eff, col_remap, n_cols_c)
        out["gcn"] = gcn_block.view(rows_eff, col_remap, n_cols_c) if gcn_block is not None else None
    else:
        n_sub = len(attn_subs)
        cs = (n_cols // g_col) // n_sub
        plans, attn_c, gcn_c = [], [], []
        for s in range(n_sub):
            if use_col:
                _, c_need = need(attn_subs[s], gcn_subs[s] if gcn_subs is not None else None)
                p = SparseRowPlan(grid.col_group, cs, c_need, f"col{s}", transport, heap)
                col_remap, n_cols_c = p.remap.long(), p.n_need
            else:
                p, col_remap, n_cols_c = None, ident(g_col * cs), g_col * cs
            plans.append(p)
            attn_c.append(attn_subs[s].compacted(rows_eff, col_remap, n_cols_c))
            gcn_c.append(gcn_subs[s].view(rows_eff, col_remap, n_cols_c) if gcn_subs is not None else None)
            if p is not None:
                p.drop_remap()
        out["cols"], out["attn"], out["gcn"] = plans, attn_c, gcn_c
    plan_row.drop_remap()
    plan_col.drop_remap()
    return out, info

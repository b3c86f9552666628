"""Distributed building blocks besides attention: GCN aggregation, BatchNorm with global statistics, loss / accuracy,
gradient all-reduce.  Dense inputs and outputs are the owned chunk ``[chunk, ...]``; padded rows are kept out of
statistics and losses through ``grid.valid_mask``.  Semantics follow ``gt3d/gt3d/dist/layers.py:67-324``.
"""
import os

import torch
import torch.distributed as dist

from ..attention.csr import BlockCSR
from ..ops.sparse import spmm
from .collectives import all_gather_rows, all_reduce_sum, reduce_scatter_rows
from .grid import group_size

_STEP = [0]


def set_step(i: int):
    """Training step counter: ``DistBatchNorm1d`` updates its running statistics at most once per step, so a forward
    recomputed under activation checkpointing does not update them twice."""
    _STEP[0] = int(i)


def current_step() -> int:
    return _STEP[0]


class GCNBlock:
    """Symmetrically normalised adjacency block ``A[r, c]`` (entries ``d_i^-1/2 d_j^-1/2``) shared by all GCN layers.

    The block's edges must already contain the self loops.  Without pre-computed ``edge_weight`` the global in-degree
    of every row-block node is the sum of the local counts over the row group, and the inverse square roots of the
    column block are gathered from their owners (head group first on a 3D grid, then the column group)."""

    def __init__(self, grid, block_edge_index, edge_weight=None, n_cols=None):
        self.grid = grid
        n_rows = grid.n_row_block
        n_cols = grid.n_col_block if n_cols is None else n_cols
        dev = block_edge_index.device
        if edge_weight is None:
            csr, perm = BlockCSR.from_edges(block_edge_index, n_rows, n_cols, return_perm=True)
            deg = (csr.crow[1:] - csr.crow[:-1]).to(torch.float64)
            if group_size(grid.row_group) > 1:
                dist.all_reduce(deg, group=grid.row_group)
            dis_rows = deg.pow(-0.5)
            dis_rows[torch.isinf(dis_rows)] = 0.0
            mine = dis_rows[grid.row_pos * grid.chunk:(grid.row_pos + 1) * grid.chunk].contiguous()
            if grid.p_heads > 1:
                buf = torch.empty(grid.p_heads * grid.chunk, dtype=torch.float64, device=dev)
                dist.all_gather_into_tensor(buf, mine, group=grid.head_group)
                mine = buf
            if group_size(grid.col_group) > 1:
                dis_cols = torch.empty(grid.n_col_block, dtype=torch.float64, device=dev)
                dist.all_gather_into_tensor(dis_cols, mine, group=grid.col_group)
            else:
                dis_cols = mine
            w = dis_rows[csr.rows().long()] * dis_cols[csr.col.long()]
            csr.weight = w
            self._perm = perm
        else:
            csr, perm = BlockCSR.from_edges(block_edge_index, n_rows, n_cols, weight=edge_weight.to(torch.float64),
                                            return_perm=True)
            self._perm = perm
        self.csr64 = csr
        self._typed = {}

    @property
    def n_rows(self):
        return self.csr64.n_rows

    @property
    def n_cols(self):
        return self.csr64.n_cols

    def weights_in_input_order(self):
        """Normalised weights aligned with the edge list the block was built from."""
        w = torch.empty_like(self.csr64.weight)
        w[self._perm] = self.csr64.weight
        return w

    def matrix(self, dtype, device=None) -> BlockCSR:
        """The block with weights in ``dtype`` (bf16 inputs aggregate with fp32 weights)."""
        wdt = torch.float32 if dtype in (torch.bfloat16, torch.float16) else dtype
        device = torch.device(device) if device is not None else self.csr64.device
        key = (wdt, device)
        if key not in self._typed:
            c = self.csr64.to(device)
            self._typed[key] = BlockCSR(c.n_rows, c.n_cols, c.crow, c.col, None, c.weight.to(wdt))
        return self._typed[key]

    def view(self, rows_need, col_remap, n_cols_c):
        """The block restricted to the compact index spaces of a sparse-communication plan pair."""
        out = GCNBlock.__new__(GCNBlock)
        out.grid, out._perm, out._typed = self.grid, None, {}
        out.csr64 = self.csr64.compacted(rows_need, col_remap, n_cols_c)
        return out

    def nbytes(self, seen=None):
        seen = set() if seen is None else seen
        return self.csr64.nbytes(seen) + sum(c.nbytes(seen) for c in self._typed.values())


class DistGCNConv(torch.nn.Module):
    """GCNConv(dim, dim): ``X W`` on the owned chunk, gathered over the column group, aggregated on the block,
    reduce-scattered over the row group, plus bias."""

    def __init__(self, grid, block: GCNBlock, dim_in, dim_out):
        super().__init__()
        self.grid, self.block = grid, block
        self.lin = torch.nn.Linear(dim_in, dim_out, bias=False)
        self.bias = torch.nn.Parameter(torch.zeros(dim_out))

    def forward(self, x_loc):
        from ..ops import functional as K
        h_blk = all_gather_rows(K.linear(x_loc, self.lin.weight), self.grid.col_group)
        agg = spmm(self.block.matrix(h_blk.dtype, h_blk.device), h_blk)
        return reduce_scatter_rows(agg, self.grid.row_group) + self.bias


class DistBatchNorm1d(torch.nn.Module):
    """BatchNorm1d whose batch statistics run over all valid nodes of all ranks (one all-reduce of ``[2 dim]``)."""

    def __init__(self, grid, dim, eps=1e-5, momentum=0.1):
        super().__init__()
        self.grid, self.eps, self.momentum = grid, eps, momentum
        self.weight = torch.nn.Parameter(torch.ones(dim))
        self.bias = torch.nn.Parameter(torch.zeros(dim))
        self.register_buffer("running_mean", torch.zeros(dim))
        self.register_buffer("running_var", torch.ones(dim))
        self.register_buffer("num_batches_tracked", torch.tensor(0, dtype=torch.long))
        self._stats_step = -1

    def local_stats(self, x):
        xm = x * self.grid.valid_mask.to(device=x.device, dtype=x.dtype).unsqueeze(-1)
        return torch.cat([xm.sum(0), (xm * x).sum(0)])

    def apply_stats(self, x, stats):
        n = float(self.grid.num_nodes)
        d = x.shape[1]
        mean = stats[:d] / n
        var = stats[d:] / n - mean * mean
        if self._stats_step != _STEP[0]:
            self._stats_step = _STEP[0]
            with torch.no_grad():
                unbiased = var * (n / max(n - 1.0, 1.0))
                self.running_mean.lerp_(mean.detach().to(self.running_mean.dtype), self.momentum)
                self.running_var.lerp_(unbiased.detach().to(self.running_var.dtype), self.momentum)
                self.num_batches_tracked += 1
        return (x - mean) * torch.rsqrt(var + self.eps) * self.weight.to(x.dtype) + self.bias.to(x.dtype)

    def forward(self, x):
        if self.training:
            return self.apply_stats(x, _stats_sum(self.local_stats(x)))
        mean, var = self.running_mean.to(x.dtype), self.running_var.to(x.dtype)
        return (x - mean) * torch.rsqrt(var + self.eps) * self.weight.to(x.dtype) + self.bias.to(x.dtype)


def _stats_sum(stats):
    """Sum of the BatchNorm statistics over all ranks.  ``GT_BN_NO_SYNC=1`` skips the all-reduces (forward and backward): a timing
    ablation with rank-local, i.e. wrong, statistics (the reference's ``GT3D_BN_NO_SYNC``, ``gt3d/gt3d/dist/layers.py:44-45``)."""
    if os.environ.get("GT_BN_NO_SYNC", "0") == "1":
        return stats
    return all_reduce_sum(stats)


def dist_batchnorm_pair(bn_a, x_a, bn_b, x_b):
    """Two independent ``DistBatchNorm1d`` applications that share one statistics all-reduce (forward and backward)."""
    if not bn_a.training:
        return bn_a(x_a), bn_b(x_b)
    d = x_a.shape[1]
    stats = _stats_sum(torch.cat([bn_a.local_stats(x_a), bn_b.local_stats(x_b)]))
    return bn_a.apply_stats(x_a, stats[:2 * d]), bn_b.apply_stats(x_b, stats[2 * d:])


def dist_cross_entropy(logits_loc, y_loc, mask_loc, num_total):
    """This rank's share of the mean cross-entropy over the masked nodes of all ranks (``num_total`` of them)."""
    if logits_loc.is_cuda and logits_loc.dtype in (torch.float32, torch.bfloat16):
        from ..ops.loss import masked_cross_entropy
        return masked_cross_entropy(logits_loc, y_loc, mask_loc, float(num_total))
    w = mask_loc.to(logits_loc.dtype)
    nll = torch.nn.functional.cross_entropy(logits_loc.float() if logits_loc.dtype == torch.bfloat16 else logits_loc,
                                            y_loc.clamp_min(0), reduction="none")
    return (nll * w).sum() / num_total


@torch.no_grad()
def dist_accuracy(logits_loc, y_loc, masks_loc: dict):
    """Accuracy per split over all ranks; ``masks_loc``: name -> bool mask over the owned chunk."""
    pred = logits_loc.argmax(-1)
    hit = pred == y_loc
    stats = torch.stack([torch.stack([(hit & m).sum(), m.sum()]) for m in masks_loc.values()]).double()
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(stats)
    stats = stats.cpu()
    return {k: (stats[i, 0] / stats[i, 1].clamp_min(1)).item() for i, k in enumerate(masks_loc)}


def allreduce_grads(params, group=None):
    """One flat sum-all-reduce of every gradient (parameters are replicated on all ranks).  Parameters without a
    gradient on this rank contribute zeros so that all ranks reduce the same buffer."""
    params = [p for p in params if p.requires_grad]
    if not params or group_size(group) == 1:
        return
    for p in params:
        if p.grad is None:
            p.grad = torch.zeros_like(p)
    flat = torch.cat([p.grad.reshape(-1) for p in params])
    dist.all_reduce(flat, group=group)
    off = 0
    for p in params:
        p.grad.copy_(flat[off:off + p.numel()].view_as(p))
        off += p.numel()

"""Distributed Exphormer on a 2D grid (or a 3D grid with a head axis).

Parameters, their names and the mathematics are those of :class:`~gt_b200.models.exphormer_ref.ExphormerRef`; a
state dict of one loads into the other.  ``DistExphormer`` picks the layer implementation from its flags (the layer
kinds of the reference, ``gt3d/gt3d/models/exphormer_dist.py:94-208``):

==============  =====================================================================================================
plain           owner projects Q/K/V; Q/K/V gathered; split-KV combine; GCN has its own gather + reduce-scatter
fused           x gathered ONCE per block (row block for Q, column block for K/V/GCN), projected locally, ONE
                reduce-scatter carrying ``[acc | l | gcn partial]``; ``gather_proj``: owner projects, projections move
pipelined       fused, column block gathered in ``n_sub`` sub-blocks, gather of s+1 overlaps compute of s
streamed        fused, sub-blocks discarded after use and re-gathered / re-projected in backward (memory
                ``O(N/P_d + N/(P_o n_sub))``); explicit backward with asynchronous dx reduce-scatters
head            3D grid: owner projects, rows<->heads all-to-all, head-slice gathers, kernel on ``H/P_i`` heads
ring            (P, 1) grid, input chunks rotate (:mod:`gt_b200.parallel.ring`)
==============  =====================================================================================================

Every layer shares ``_LayerBase.tail`` (dropout, the norms, FFN), and on CUDA the dense pieces run on the native
kernels through :mod:`gt_b200.ops.functional`.
"""
import os

import torch
import torch.nn as nn
import torch.nn.functional as F
import torch.utils.checkpoint

from ..ops import functional as K
from ..ops.sparse import spmm, spmm_raw
from ..parallel.attention import (AttentionBlock, DistAttentionPartial, DistMaskedSparseAttention, combine_partials,
                                  split_block_by_column_subblocks, split_block_by_source_chunk)
from ..parallel.collectives import (all_gather_rows, all_gather_rows_start, heads_to_rows, raw_all_gather_rows,
                                    raw_reduce_scatter_rows, rows_to_heads, wait_gather)
from ..parallel.fused_comm import fused_ok, linear_gather
from ..parallel.grid import group_size
from ..parallel.layers import DistBatchNorm1d, DistGCNConv, GCNBlock, dist_batchnorm_pair
from ..parallel.sparse_comm import build_sparse_comm, sparse_all_gather, wait_work
from ..utils.timers import timers
from .exphormer_ref import RMSNorm, gcn_edges_with_self_loops  # noqa: F401  (re-exported for the trainer)

BN_PAIR = os.environ.get("GT_BN_PAIR", "1") == "1"          # one statistics all-reduce for the two branch BatchNorms


def make_norm(kind, grid, dim, eps=1e-5, momentum=0.1):
    """``bn``: BatchNorm over all nodes of all ranks (one all-reduce); ``ln`` / ``rms``: per node, no collective."""
    if kind == "ln":
        return K.LayerNorm(dim, eps=eps)
    if kind == "rms":
        return RMSNorm(dim, eps=eps)
    if kind == "bn":
        return DistBatchNorm1d(grid, dim, eps, momentum)
    raise ValueError(kind)


def _gather_rows(t, group, plan=None, wire=None):
    return all_gather_rows(t, group, wire) if plan is None else sparse_all_gather(t, plan, wire)


class _LayerBase(nn.Module):
    """Parameters of one Exphormer layer (reference names) and the owned-row tail."""

    def __init__(self, grid, dim_h, num_heads, dropout, bn_eps, bn_momentum, norm, with_gcn=True, with_attn=True,
                 gcn_module=None):
        super().__init__()
        if not (with_gcn or with_attn):
            raise ValueError("a layer needs the GCN branch, the attention branch or both")
        self.grid, self.dim_h, self.num_heads, self.d_head, self.dropout = grid, dim_h, num_heads, dim_h // num_heads, dropout
        self.with_gcn, self.with_attn = with_gcn, with_attn
        if with_gcn:
            if gcn_module is not None:
                self.gcn = gcn_module
            else:                                   # same names as GCNConvRef: gcn.lin.weight, gcn.bias
                self.gcn = nn.Module()
                self.gcn.lin = nn.Linear(dim_h, dim_h, bias=False)
                self.gcn.bias = nn.Parameter(torch.zeros(dim_h))
            self.bn_local = make_norm(norm, grid, dim_h, bn_eps, bn_momentum)
        if with_attn:
            self.q, self.k, self.v, self.e = (nn.Linear(dim_h, dim_h, bias=False) for _ in range(4))
            self.bn_attn = make_norm(norm, grid, dim_h, bn_eps, bn_momentum)
        self.ff1 = nn.Linear(dim_h, 2 * dim_h)
        self.ff2 = nn.Linear(2 * dim_h, dim_h)
        self.bn_ff = make_norm(norm, grid, dim_h, bn_eps, bn_momentum)

    def gate(self, edge_type_emb):
        return K.linear(edge_type_emb, self.e.weight).view(-1, self.num_heads, self.d_head)

    def tail(self, x, o=None, agg=None, agg_has_bias=False, l=None):
        """``o [n, dim]``: normalised attention output, or with ``l [n, H]`` the unnormalised accumulator (clamp-exp:
        ``o / (l + 1e-6)`` is then fused into the norm kernel); ``agg [n, dim]``: GCN aggregation (bias added here)."""
        p, tr = self.dropout, self.training
        h_attn = h_local = None
        if l is not None and not isinstance(self.bn_attn, K.LayerNorm):
            o = (o.reshape(o.shape[0], l.shape[1], -1) / (l + 1e-6).unsqueeze(-1)).reshape(o.shape[0], -1)
            l = None
        if self.with_attn and self.with_gcn and BN_PAIR and isinstance(self.bn_local, DistBatchNorm1d):
            a = x + F.dropout(o.to(x.dtype), p, tr)
            b = x + F.dropout(agg.to(x.dtype) if agg_has_bias else agg.to(x.dtype) + self.gcn.bias.to(x.dtype), p, tr)
            h_local, h_attn = dist_batchnorm_pair(self.bn_local, b, self.bn_attn, a)
        else:
            if self.with_attn:
                h_attn = K.dropout_add_norm(self.bn_attn, o, x, None, p, tr, l=l)
            if self.with_gcn:
                h_local = K.dropout_add_norm(self.bn_local, agg, x, None if agg_has_bias else self.gcn.bias, p, tr)
        hh = h_attn if h_local is None else (h_local if h_attn is None else h_local + h_attn)
        ff = K.linear(hh, self.ff1.weight, self.ff1.bias, activation="relu", dropout=p, training=tr)
        ff = K.linear(ff, self.ff2.weight, self.ff2.bias)
        return K.dropout_add_norm(self.bn_ff, ff, hh, None, p, tr)


class DistExphormerLayer(_LayerBase):
    """Plain layer: projections on the owned chunk, the attention operator and the GCN do their own collectives."""

    def __init__(self, grid, gcn_block, attn_block, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                 comm_dtype=None, with_gcn=True, with_attn=True, norm="bn"):
        gcn_mod = DistGCNConv(grid, gcn_block, dim_h, dim_h) if with_gcn else None
        super().__init__(grid, dim_h, num_heads, dropout, bn_eps, bn_momentum, norm, with_gcn, with_attn, gcn_mod)
        if with_attn:
            self.attn = DistMaskedSparseAttention(grid, attn_block, num_heads, self.d_head, backend=backend,
                                                  score="gated", norm="clampexp", comm_dtype=comm_dtype)

    def forward(self, x, edge_type_emb):
        n, h, d = x.shape[0], self.num_heads, self.d_head
        o = agg = None
        if self.with_gcn:
            agg = self.gcn(x)                                       # includes the bias
        if self.with_attn:
            o = self.attn(K.linear(x, self.q.weight).view(n, h, d), K.linear(x, self.k.weight).view(n, h, d),
                          K.linear(x, self.v.weight).view(n, h, d), self.gate(edge_type_emb)).reshape(n, h * d)
        return self.tail(x, o, agg, agg_has_bias=True)


class DistExphormerLayerFused(_LayerBase):
    """Fused-communication layer: 2 gathers of x + 1 reduce-scatter per direction."""

    def __init__(self, grid, gcn_block, attn_block, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                 comm_dtype=None, rs_dtype=None, with_gcn=True, gather_proj=False, kernel_dtype=None, sparse=None, norm="bn"):
        super().__init__(grid, dim_h, num_heads, dropout, bn_eps, bn_momentum, norm, with_gcn, True)
        self.comm_dtype, self.rs_dtype, self.kernel_dtype, self.gather_proj = comm_dtype, rs_dtype, kernel_dtype, gather_proj
        self.sp_row = sparse["row"] if sparse is not None else None
        self.sp_col = sparse["col"] if sparse is not None else None
        self.gcn_block = gcn_block
        self.token = None                                    # a parallel.token_dense.DenseToken: the global token outside the sparse structure
        self.attn = DistAttentionPartial(grid, attn_block, num_heads, self.d_head, backend=backend, score="gated",
                                         norm="clampexp")

    def branches(self, x, edge_type_emb):
        g, h, d = self.grid, self.num_heads, self.d_head
        hd = h * d
        kdt = self.kernel_dtype or x.dtype
        t = timers()
        gate = self.gate(edge_type_emb)
        agg = None
        if self.gather_proj:
            t.start("qkv proj")
            q_loc = K.linear(x, self.q.weight)
            ws = [self.k.weight, self.v.weight] + ([self.gcn.lin.weight] if self.with_gcn else [])
            kvg_loc = K.linear(x, torch.cat(ws, dim=0))
            t.stop("qkv proj")
            t.start("gather x")
            q = _gather_rows(q_loc, g.row_group, self.sp_row, self.comm_dtype).to(kdt).view(-1, h, d)
            kvg = _gather_rows(kvg_loc, g.col_group, self.sp_col, self.comm_dtype)
            t.stop("gather x")
            pieces = K.split_columns(kvg, [hd, hd] + ([kvg.shape[1] - 2 * hd] if self.with_gcn else []))
            k, v = pieces[0].to(kdt).view(-1, h, d), pieces[1].to(kdt).view(-1, h, d)
            if self.with_gcn:
                msg = pieces[2]
                agg = spmm(self.gcn_block.matrix(msg.dtype, msg.device), msg)
        else:
            ws = [self.k.weight, self.v.weight] + ([self.gcn.lin.weight] if self.with_gcn else [])
            w_kvg = torch.cat(ws, dim=0)                               # one GEMM for K | V | GCN message
            t.start("gather x + qkv proj")
            # dense groups on the peer-memory transport: the all-gather happens inside the GEMM (TMA loads from the owners)
            if self.sp_col is None and fused_ok(x, w_kvg, g.col_group):
                kvg = linear_gather(x, w_kvg, g.col_group)
            else:
                kvg = K.linear(_gather_rows(x, g.col_group, self.sp_col, self.comm_dtype), w_kvg)
            if self.sp_row is None and fused_ok(x, self.q.weight, g.row_group):
                q = linear_gather(x, self.q.weight, g.row_group).to(kdt).view(-1, h, d)
            else:
                q = K.linear(_gather_rows(x, g.row_group, self.sp_row, self.comm_dtype), self.q.weight).to(kdt).view(-1, h, d)
            t.stop("gather x + qkv proj")
            pieces = K.split_columns(kvg, [hd, hd] + ([kvg.shape[1] - 2 * hd] if self.with_gcn else []))
            k, v = pieces[0].to(kdt).view(-1, h, d), pieces[1].to(kdt).view(-1, h, d)
            if self.with_gcn:
                t.start("gcn spmm")
                msg = pieces[2]
                agg = spmm(self.gcn_block.matrix(msg.dtype, msg.device), msg)
                t.stop("gcn spmm")
        t.start("attention partial")
        acc, l, m = self.attn(q, k, v, gate)
        t.stop("attention partial")
        t.start("reduce-scatter")
        (acc_o, l_o), agg_o = combine_partials(acc, l, m, g, "clampexp", 1e-6, extra=agg, rs_dtype=self.rs_dtype, plan=self.sp_row,
                                               normalize=False)
        t.stop("reduce-scatter")
        return (acc_o, l_o), agg_o

    def forward(self, x, edge_type_emb):
        if type(self) is DistExphormerLayerFused:
            # the whole branch as one explicit-backward operator on the native kernels (collectives inside the kernels)
            from ..parallel.fused_layer import fused_branch
            gate = self.gate(edge_type_emb)
            out = fused_branch(self, x, gate)
            if out is not None:
                acc_o, l_o, agg_o = out
                if self.token is not None:
                    acc_o, l_o = self.token.add(self, x, gate, acc_o, l_o)
                return self.tail(x, acc_o, agg_o, l=l_o)
        (acc_o, l_o), agg_o = self.branches(x, edge_type_emb)
        if self.token is not None:
            acc_o, l_o = self.token.add(self, x, self.gate(edge_type_emb), acc_o, l_o)
        return self.tail(x, acc_o, agg_o, l=l_o)

    def stacked_params(self):
        """Parameters the fused operator reads as one stacked matrix (rows K | V | message | Q)."""
        return [self.k.weight, self.v.weight] + ([self.gcn.lin.weight] if self.with_gcn else []) + [self.q.weight]


class DistExphormerLayerHead(_LayerBase):
    """3D-grid layer: owner projects all heads (and the GCN message) once, ONE all-to-all + ONE gather move
    ``[K_j | V_j | G_j]`` per head group j, ONE reduce-scatter, ONE all-to-all back carrying ``[o | gcn]``."""

    def __init__(self, grid, attn_block, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend, comm_dtype=None,
                 rs_dtype=None, kernel_dtype=None, gcn_block=None, with_gcn=False, sparse=None, norm="bn"):
        super().__init__(grid, dim_h, num_heads, dropout, bn_eps, bn_momentum, norm, with_gcn, True)
        if num_heads % grid.p_heads or dim_h % grid.p_heads:
            raise ValueError("the head axis must divide the heads and the hidden size")
        self.hg, self.ds = num_heads // grid.p_heads, dim_h // grid.p_heads
        self.comm_dtype, self.rs_dtype, self.kernel_dtype, self.gcn_block = comm_dtype, rs_dtype, kernel_dtype, gcn_block
        self.sp_row = sparse["row"] if sparse is not None else None
        self.sp_col = sparse["col"] if sparse is not None else None
        self.attn = DistAttentionPartial(grid, attn_block, self.hg, self.d_head, backend=backend, score="gated",
                                         norm="clampexp")

    def forward(self, x, edge_type_emb):
        g = self.grid
        n, h, d, p_i, hg, ds = x.shape[0], self.num_heads, self.d_head, g.p_heads, self.hg, self.ds
        kdt = self.kernel_dtype or x.dtype
        t = timers()
        gate = self.gate(edge_type_emb)
        if not self.with_gcn and os.environ.get("GT_HEAD_MERGED", "1") == "0":
            return self.tail(x, self._attention_separate(x, gate), None)
        t.start("qkv proj")
        q = K.linear(x, self.q.weight).view(n, p_i, ds)
        # weight rows interleaved per head group so that the all-to-all input [n, P_i, (2|3) ds] is a view
        ws = [self.k.weight.view(p_i, ds, self.dim_h), self.v.weight.view(p_i, ds, self.dim_h)]
        if self.with_gcn:
            ws.append(self.gcn.lin.weight.view(p_i, ds, self.dim_h))
        kvg = K.linear(x, torch.cat(ws, dim=1).reshape(-1, self.dim_h)).view(n, p_i, -1)
        t.stop("qkv proj")
        t.start("head: a2a + gather q/k/v")
        wire = self.comm_dtype
        q_h = rows_to_heads(q if wire is None else q.to(wire), g.head_group, p_i)
        kvg_h = rows_to_heads(kvg if wire is None else kvg.to(wire), g.head_group, p_i)
        q_blk = _gather_rows(q_h, g.row_group, self.sp_row).to(kdt).reshape(-1, hg, d)
        kvg_blk = _gather_rows(kvg_h, g.col_group, self.sp_col).reshape(-1, kvg.shape[2])
        t.stop("head: a2a + gather q/k/v")
        k_blk = kvg_blk[:, :ds].to(kdt).contiguous().view(-1, hg, d)
        v_blk = kvg_blk[:, ds:2 * ds].to(kdt).contiguous().view(-1, hg, d)
        agg = None
        if self.with_gcn:
            msg = kvg_blk[:, 2 * ds:].to(x.dtype).contiguous()
            agg = spmm(self.gcn_block.matrix(msg.dtype, msg.device), msg)
        acc, l, m = self.attn(q_blk, k_blk, v_blk, gate[:, g.h * hg:(g.h + 1) * hg].contiguous())
        t.start("reduce-scatter")
        o_h, agg_o = combine_partials(acc, l, m, g, "clampexp", 1e-6, extra=agg, rs_dtype=self.rs_dtype, plan=self.sp_row)
        t.stop("reduce-scatter")
        t.start("head: a2a back")
        back = o_h.reshape(-1, ds) if agg_o is None else torch.cat([o_h.reshape(-1, ds), agg_o.to(o_h.dtype)], dim=1)
        back = back if wire is None else back.to(wire)
        back = heads_to_rows(back.view(-1, 1, back.shape[1]).contiguous(), g.head_group, p_i).to(x.dtype)   # [n, P_i, (1|2) ds]
        t.stop("head: a2a back")
        o = back[:, :, :ds].reshape(n, h * d)
        agg_rows = back[:, :, ds:].reshape(n, self.dim_h) if self.with_gcn else None
        return self.tail(x, o, agg_rows)


    def _attention_separate(self, x, gate):
        """``GT_HEAD_MERGED=0``, attention-only layers: Q, K and V travel separately (three all-to-alls and three gathers instead of
        one for Q and one for the merged ``[K | V]`` tensor): the A/B switch of the layer's communication pattern
        (``gt3d/gt3d/models/exphormer_dist.py:484-505``)."""
        if self.sp_row is not None or self.sp_col is not None:
            raise ValueError("GT_HEAD_MERGED=0 has no sparse-communication path")
        g = self.grid
        n, d, p_i, hg, ds = x.shape[0], self.d_head, g.p_heads, self.hg, self.ds
        kdt = self.kernel_dtype or x.dtype
        wire = self.comm_dtype
        t = timers()

        def to_block(w, group):
            y = K.linear(x, w).view(n, p_i, ds)
            y = rows_to_heads(y if wire is None else y.to(wire), g.head_group, p_i)
            return _gather_rows(y, group, None).to(kdt).reshape(-1, hg, d)
        t.start("head: a2a + gather q/k/v")
        q_blk, k_blk, v_blk = to_block(self.q.weight, g.row_group), to_block(self.k.weight, g.col_group), to_block(self.v.weight, g.col_group)
        t.stop("head: a2a + gather q/k/v")
        acc, l, m = self.attn(q_blk, k_blk, v_blk, gate[:, g.h * hg:(g.h + 1) * hg].contiguous())
        o_h, _ = combine_partials(acc, l, m, g, "clampexp", 1e-6, rs_dtype=self.rs_dtype)
        back = o_h.reshape(-1, 1, ds)
        back = heads_to_rows((back if wire is None else back.to(wire)).contiguous(), g.head_group, p_i).to(x.dtype)
        return back.reshape(n, self.num_heads * d)


class DistExphormerLayerPipelined(DistExphormerLayerFused):
    """Fused layer whose column block arrives in ``n_sub`` sub-blocks; the asynchronous gather of sub-block s+1 overlaps
    the projections / SpMM / attention of sub-block s.  Clamp-exp partials of the sub-blocks add without rescaling."""

    def __init__(self, grid, gcn_blocks, attn_blocks, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                 comm_dtype=None, rs_dtype=None, kernel_dtype=None, with_gcn=True, norm="bn"):
        super().__init__(grid, gcn_blocks[0] if with_gcn else None, attn_blocks[0], dim_h, num_heads, dropout, bn_eps,
                         bn_momentum, backend, comm_dtype=comm_dtype, rs_dtype=rs_dtype, kernel_dtype=kernel_dtype,
                         with_gcn=with_gcn, norm=norm)
        self.gcn_blocks = gcn_blocks
        self.attns = nn.ModuleList([DistAttentionPartial(grid, b, num_heads, self.d_head, backend=backend, score="gated",
                                                         norm="clampexp") for b in attn_blocks])
        self.n_sub = len(attn_blocks)
        self.cs = grid.chunk // self.n_sub

    def branches(self, x, edge_type_emb):
        g, h, d, cs = self.grid, self.num_heads, self.d_head, self.cs
        hd = h * d
        kdt = self.kernel_dtype or x.dtype
        row_handle = all_gather_rows_start(x, g.row_group, self.comm_dtype)
        pending = all_gather_rows_start(x[0:cs], g.col_group, self.comm_dtype)
        gate = self.gate(edge_type_emb)
        ws = torch.cat([self.k.weight, self.v.weight] + ([self.gcn.lin.weight] if self.with_gcn else []), dim=0)
        q = acc = l = agg = None
        for s in range(self.n_sub):
            xs = wait_gather(pending)
            if s + 1 < self.n_sub:
                pending = all_gather_rows_start(x[(s + 1) * cs:(s + 2) * cs], g.col_group, self.comm_dtype)
            kvg = K.linear(xs, ws)
            if q is None:
                q = K.linear(wait_gather(row_handle), self.q.weight).to(kdt).view(-1, h, d)
            pieces = K.split_columns(kvg, [hd, hd] + ([kvg.shape[1] - 2 * hd] if self.with_gcn else []))
            acc_s, l_s, _ = self.attns[s](q, pieces[0].to(kdt).view(-1, h, d), pieces[1].to(kdt).view(-1, h, d), gate)
            acc = acc_s if acc is None else acc + acc_s
            l = l_s if l is None else l + l_s
            if self.with_gcn:
                msg = pieces[2]
                agg_s = spmm(self.gcn_blocks[s].matrix(msg.dtype, msg.device), msg)
                agg = agg_s if agg is None else agg + agg_s
        return combine_partials(acc, l, torch.zeros_like(l), g, "clampexp", 1e-6, extra=agg, rs_dtype=self.rs_dtype, normalize=False)


class _StreamedAttnGCN(torch.autograd.Function):
    """Owned rows of the reduce-scattered payload ``[acc | l | gcn partial]`` (``[chunk, h d + h + dim]``).

    Forward: for every column sub-block: gather (optionally prefetched), project K / V / GCN message, accumulate the
    partials into the row-block payload, drop the sub-block.  Saved for backward: the owned input only.  Backward:
    gather the payload gradient over the row group, then per sub-block re-gather, re-project, run the backward kernels,
    form the weight gradients and ``dx_s = dK W_k + dV W_v + dP W_g`` and reduce-scatter it (asynchronously, overlapped
    with the next sub-block).  Mirrors the algorithm of ``gt3d/gt3d/models/exphormer_dist.py:763-933``."""

    @staticmethod
    def _gather(x, group, plan=None):
        return raw_all_gather_rows(x, group) if plan is None else plan.gather(x)

    @staticmethod
    def _gather_start(x, group, plan=None):
        if plan is not None:
            return plan.gather(x, async_op=True)
        work, out = raw_all_gather_rows(x.contiguous(), group, async_op=True)
        return work, (lambda: out)

    @staticmethod
    def _finish(pend):
        work, fin = pend
        wait_work(work)
        return fin()

    @staticmethod
    def _rs_start(x, group, plan=None):
        if plan is not None:
            return plan.reduce_scatter(x, async_op=True)
        work, out = raw_reduce_scatter_rows(x, group, async_op=True)
        return work, (lambda _keep=x: out)

    @staticmethod
    def _reduce_scatter(x, group, plan=None):
        return raw_reduce_scatter_rows(x, group) if plan is None else plan.reduce_scatter(x)

    @staticmethod
    def forward(ctx, x, wq, wk, wv, wg, gate, layer):
        from ..attention import get_backend
        L, g = layer, layer.grid
        be = get_backend(L.backend)
        h, d, cs, n_sub = L.num_heads, L.d_head, L.cs, L.n_sub
        hd = h * d
        wire = L.comm_dtype or x.dtype
        kdt = L.kernel_dtype or x.dtype
        gate_c = gate.to(x.dtype if L.backend == "torch" else torch.float32)
        sp_row, sp_cols = L.sp_row, L.sp_cols
        spc = (lambda s: sp_cols[s]) if sp_cols is not None else (lambda s: None)
        accum = L.compact and hasattr(be, "attn_fwd_partial_accum") and x.is_cuda
        S = _StreamedAttnGCN
        t = timers()
        with torch.no_grad():
            xc = x.to(wire).contiguous()
            pend = S._gather_start(xc[0:cs], g.col_group, spc(0)) if L.overlap else None
            t.start("stream fwd: gather x_row + q")
            x_row = S._gather(xc, g.row_group, sp_row)
            q = K.linear_nograd(x_row.to(x.dtype), wq).to(kdt).view(-1, h, d)
            del x_row
            t.stop("stream fwd: gather x_row + q")
            rows, dim = q.shape[0], x.shape[1]
            pdt = torch.float64 if x.dtype == torch.float64 else torch.float32
            packed = torch.zeros(rows, hd + h + (dim if L.with_gcn else 0), dtype=pdt, device=x.device)
            for s in range(n_sub):
                t.start("stream fwd: gather sub-block")
                if L.overlap:
                    xs = S._finish(pend).to(x.dtype)
                    pend = S._gather_start(xc[(s + 1) * cs:(s + 2) * cs], g.col_group, spc(s + 1)) if s + 1 < n_sub else None
                else:
                    xs = S._gather(xc[s * cs:(s + 1) * cs], g.col_group, spc(s)).to(x.dtype)
                t.stop("stream fwd: gather sub-block")
                t.start("stream fwd: gcn + kv proj")
                ks = K.linear_nograd(xs, wk).to(kdt).view(-1, h, d)
                vs = K.linear_nograd(xs, wv).to(kdt).view(-1, h, d)
                if L.with_gcn:
                    msg = K.linear_nograd(xs, wg)
                    gm = L.gcn_blocks[s].matrix(msg.dtype, msg.device)
                    packed[:, hd + h:] += spmm_raw(gm, msg).to(pdt)
                del xs
                t.stop("stream fwd: gcn + kv proj")
                t.start("stream fwd: attention")
                blk = L.attns[s].block.csr
                if accum:
                    be.attn_fwd_partial_accum(q, ks, vs, blk, gate_c, None, packed, hd, score="gated", norm="clampexp",
                                              clamp=L.attn_clamp, scale=L.attn_scale)
                elif blk.num_edges:
                    acc_s, l_s, _ = be.attn_fwd_partial(q, ks, vs, blk, gate_c, None, score="gated", norm="clampexp",
                                                        clamp=L.attn_clamp, scale=L.attn_scale)
                    packed[:, :hd] += acc_s.reshape(rows, hd).to(pdt)
                    packed[:, hd:hd + h] += l_s.to(pdt)
                t.stop("stream fwd: attention")
                del ks, vs
            del q
            ctx.packed_dtype = pdt
            if L.rs_dtype is not None:
                packed = packed.to(L.rs_dtype)
            t.start("stream fwd: reduce-scatter")
            packed_o = S._reduce_scatter(packed, g.row_group, sp_row).to(pdt)
            t.stop("stream fwd: reduce-scatter")
        ctx.save_for_backward(x, wq, wk, wv, wg, gate)
        ctx.layer, ctx.gate_c_dtype = L, gate_c.dtype
        return packed_o

    @staticmethod
    def backward(ctx, dpo):
        from ..attention import get_backend
        x, wq, wk, wv, wg, gate = ctx.saved_tensors
        L, g = ctx.layer, ctx.layer.grid
        be = get_backend(L.backend)
        h, d, cs, n_sub = L.num_heads, L.d_head, L.cs, L.n_sub
        hd = h * d
        wire = L.comm_dtype or x.dtype
        kdt = L.kernel_dtype or x.dtype
        pdt = ctx.packed_dtype
        gate_c = gate.to(ctx.gate_c_dtype)
        sp_row, sp_cols = L.sp_row, L.sp_cols
        spc = (lambda s: sp_cols[s]) if sp_cols is not None else (lambda s: None)
        S = _StreamedAttnGCN
        t = timers()
        t.start("stream bwd")
        with torch.no_grad():
            dpo = dpo.contiguous()
            dacc = S._gather(dpo[:, :hd].contiguous(), g.row_group, sp_row).to(pdt)
            dl = S._gather(dpo[:, hd:hd + h].contiguous(), g.row_group, sp_row).to(pdt)
            dagg = S._gather(dpo[:, hd + h:].contiguous(), g.row_group, sp_row).to(x.dtype) if L.with_gcn else None
            rows = dacc.shape[0]
            dacc = dacc.view(rows, h, d)
            xc = x.to(wire).contiguous()
            pend = S._gather_start(xc[0:cs], g.col_group, spc(0)) if L.overlap else None
            rs_pend = None
            x_row = S._gather(xc, g.row_group, sp_row)
            q = K.linear_nograd(x_row.to(x.dtype), wq).to(kdt).view(-1, h, d)
            m0 = torch.zeros_like(dl)
            dq = torch.zeros(q.shape, dtype=pdt, device=q.device)
            dwk, dwv = torch.zeros_like(wk), torch.zeros_like(wv)
            dwg = torch.zeros_like(wg) if L.with_gcn else None
            dgate = None
            dx = torch.zeros_like(x)

            def finish_rs(p):
                s_, pend_ = p
                dx[s_ * cs:(s_ + 1) * cs] += S._finish(pend_).to(x.dtype)

            for s in range(n_sub):
                if L.overlap:
                    xs = S._finish(pend).to(x.dtype)
                    pend = S._gather_start(xc[(s + 1) * cs:(s + 2) * cs], g.col_group, spc(s + 1)) if s + 1 < n_sub else None
                else:
                    xs = S._gather(xc[s * cs:(s + 1) * cs], g.col_group, spc(s)).to(x.dtype)
                ks = K.linear_nograd(xs, wk).to(kdt).view(-1, h, d)
                vs = K.linear_nograd(xs, wv).to(kdt).view(-1, h, d)
                blk = L.attns[s].block.csr
                dxs = torch.zeros(xs.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
                if blk.num_edges:
                    if L.compact and hasattr(be, "attn_bwd_partial_accum") and x.is_cuda and pdt == torch.float32:
                        # compact-accumulate backward: dq of the rows that own an edge in this sub-block is added in place
                        dks, dvs, dgate_s, _ = be.attn_bwd_partial_accum(q, ks, vs, blk, gate_c, None, m0, dacc, dl, dq.view(rows, hd),
                                                                         score="gated", norm="clampexp", clamp=L.attn_clamp,
                                                                         scale=L.attn_scale)
                    else:
                        dq_s, dks, dvs, dgate_s, _ = be.attn_bwd_partial(q, ks, vs, blk, gate_c, None, m0, dacc, dl, score="gated",
                                                                         norm="clampexp", clamp=L.attn_clamp, scale=L.attn_scale)
                        dq += dq_s.to(pdt)
                        del dq_s
                    if dgate_s is not None:
                        dgate = dgate_s if dgate is None else dgate + dgate_s
                    dks, dvs = dks.to(x.dtype).view(-1, hd), dvs.to(x.dtype).view(-1, hd)
                    dwk += K.matmul_tn(dks, xs).to(dwk.dtype)
                    dwv += K.matmul_tn(dvs, xs).to(dwv.dtype)
                    dxs += K.matmul_nn(dks, wk)
                    dxs += K.matmul_nn(dvs, wv)
                    del dks, dvs
                del ks, vs
                if L.with_gcn:
                    gm = L.gcn_blocks[s].matrix(dagg.dtype, dagg.device)
                    dp_s = spmm_raw(gm, dagg, transpose=True)
                    dwg += K.matmul_tn(dp_s, xs).to(dwg.dtype)
                    dxs += K.matmul_nn(dp_s, wg)
                    del dp_s
                del xs
                if L.overlap:
                    if rs_pend is not None:
                        finish_rs(rs_pend)
                    rs_pend = (s, S._rs_start(dxs.to(wire), g.col_group, spc(s)))
                else:
                    dx[s * cs:(s + 1) * cs] += S._reduce_scatter(dxs.to(wire), g.col_group, spc(s)).to(x.dtype)
                del dxs
            if rs_pend is not None:
                finish_rs(rs_pend)
            dq2 = dq.view(rows, hd).to(x.dtype)
            xr = x_row.to(x.dtype)
            dwq = K.matmul_tn(dq2, xr).to(wq.dtype)
            dxr = K.matmul_nn(dq2, wq).to(wire)
            dx += S._reduce_scatter(dxr, g.row_group, sp_row).to(x.dtype)
        t.stop("stream bwd")
        return dx, dwq, dwk, dwv, dwg, (dgate.to(gate.dtype) if dgate is not None else None), None


class DistExphormerLayerStreamed(DistExphormerLayerPipelined):
    """Fused layer with the column block streamed in ``n_sub`` sub-blocks and recomputed in backward.  With
    ``tail_checkpoint`` the owned-row tail is recomputed too, so the layer keeps only its input and the payload."""

    self_checkpointing = True

    def __init__(self, grid, gcn_blocks, attn_blocks, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                 comm_dtype=None, rs_dtype=None, tail_checkpoint=False, kernel_dtype=None, with_gcn=True, norm="bn"):
        super().__init__(grid, gcn_blocks, attn_blocks, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                         comm_dtype=comm_dtype, rs_dtype=rs_dtype, kernel_dtype=kernel_dtype, with_gcn=with_gcn, norm=norm)
        self.backend, self.tail_checkpoint = backend, tail_checkpoint
        self.attn_clamp, self.attn_scale = self.attns[0].clamp, self.attns[0].scale
        self.overlap, self.compact = True, True
        self.sp_cols = None

    def _tail(self, x, packed_o):
        n, h, d = x.shape[0], self.num_heads, self.d_head
        hd = h * d
        l_o = packed_o[:, hd:hd + h]
        o = (packed_o[:, :hd].reshape(n, h, d) / (l_o + 1e-6).unsqueeze(-1)).reshape(n, hd).to(x.dtype)
        agg_o = packed_o[:, hd + h:].to(x.dtype) if self.with_gcn else None
        return self.tail(x, o, agg_o)

    def forward(self, x, edge_type_emb):
        gate = self.gate(edge_type_emb)
        wg = self.gcn.lin.weight if self.with_gcn else None
        packed_o = _StreamedAttnGCN.apply(x, self.q.weight, self.k.weight, self.v.weight, wg, gate, self)
        if self.tail_checkpoint and self.training:
            return torch.utils.checkpoint.checkpoint(self._tail, x, packed_o, use_reentrant=False)
        return self._tail(x, packed_o)


class DistExphormer(nn.Module):
    """``DistExphormer(grid, gcn_block_ei, attn_block_ei, attn_block_et, dim_in, dim_hidden, dim_out, num_layers,
    num_heads, ...)``: blocks are local ``(col-local src, row-local dst)`` edge lists (``grid.local_block`` or a
    partition loader); the GCN block must already contain the self loops."""

    def __init__(self, grid, gcn_block_ei, attn_block_ei, attn_block_et, dim_in, dim_hidden, dim_out, num_layers, num_heads,
                 dropout=0.3, gnn_dropout=0.3, num_edge_types=2, bn_eps=1e-5, bn_momentum=0.1, pre_l2norm=True,
                 backend="cuda", gcn_weight=None, checkpoint=False, comm_dtype=None, fused=False, rs_dtype=None,
                 pipeline_sub=1, stream_sub=1, norm="bn", ring=False, with_gcn=True, with_attn=True, gather_proj=False,
                 stream_overlap=True, stream_compact=True, kernel_dtype=None, sparse_comm=False, sparse_threshold=None,
                 sparse_transport="a2a", heap=None, token_node=None):
        super().__init__()
        self.grid = grid
        head_grid = grid.p_heads > 1 or getattr(grid, "head_group", None) is not None
        n_sub = max(pipeline_sub, stream_sub)
        if gather_proj and not (fused and n_sub == 1 and not ring):
            raise ValueError("gather_proj is implemented for the fused (non-streamed) layer")
        if not with_gcn and n_sub > 1 and not ring and stream_sub <= 1:
            raise ValueError("attention-only is implemented for the plain, fused, streamed, head and ring layers")
        if not with_attn and (fused or ring or head_grid):
            raise ValueError("GCN-only is implemented for the plain layer")
        if head_grid and (fused or ring or n_sub > 1 or gather_proj):
            raise ValueError("the head grid has its own layer: no fused / ring / streamed / gather_proj")
        if sparse_comm and not (with_attn and not ring and pipeline_sub <= 1 and (fused or head_grid)):
            raise ValueError("sparse communication is implemented for the fused, streamed and head-grid layers")
        self.with_gcn, self.with_attn = with_gcn, with_attn
        self.gnn_dropout, self.pre_l2norm, self.checkpoint = gnn_dropout, pre_l2norm, checkpoint
        self.sparse_comm, self.sparse_info = None, None
        gcn_block = GCNBlock(grid, gcn_block_ei, gcn_weight) if with_gcn else None
        attn_block = AttentionBlock(grid, attn_block_ei, attn_block_et)
        self.edge_type_emb = nn.Embedding(num_edge_types, dim_hidden)
        self.pre_lin = nn.Linear(dim_in, dim_hidden, bias=False)
        self.pre_bn = make_norm(norm, grid, dim_hidden, bn_eps, bn_momentum)
        common = (dim_hidden, num_heads, dropout, bn_eps, bn_momentum, backend)
        sp_kw = dict(transport=sparse_transport, heap=heap)
        if head_grid:
            sp = None
            if sparse_comm:
                sp, self.sparse_info = build_sparse_comm(grid, attn_block, gcn_block, sparse_threshold, **sp_kw)
                if sp is not None:
                    attn_block, gcn_block, self.sparse_comm = sp["attn"], sp["gcn"], sp
            mk = lambda: DistExphormerLayerHead(grid, attn_block, *common, comm_dtype=comm_dtype, rs_dtype=rs_dtype,   # noqa: E731
                                                kernel_dtype=kernel_dtype, gcn_block=gcn_block, with_gcn=with_gcn,
                                                sparse=sp, norm=norm)
        elif ring:
            from ..parallel.ring import DistExphormerLayerRing
            if grid.p_cols != 1:
                raise ValueError("ring attention needs a (P, 1) grid")
            p = grid.p_rows
            if with_gcn:
                w_full = gcn_block.weights_in_input_order()
                gcn_blocks = [GCNBlock(grid, ei, w, n_cols=grid.chunk)
                              for ei, _, w in split_block_by_source_chunk(gcn_block_ei, p, grid.chunk, None, w_full)]
            else:
                gcn_blocks = [None] * p
            attn_blocks = [AttentionBlock(grid, ei, et, n_cols=grid.chunk)
                           for ei, et, _ in split_block_by_source_chunk(attn_block_ei, p, grid.chunk, attn_block_et)]
            mk = lambda: DistExphormerLayerRing(grid, gcn_blocks, attn_blocks, *common, comm_dtype=comm_dtype,   # noqa: E731
                                                tail_checkpoint=checkpoint, with_gcn=with_gcn, norm=norm)
        elif fused and n_sub > 1:
            n_cols_sub = grid.p_rows * grid.p_heads * (grid.chunk // n_sub)
            if with_gcn:
                w_full = gcn_block.weights_in_input_order()
                gcn_blocks = [GCNBlock(grid, ei, w, n_cols=n_cols_sub)
                              for ei, _, w in split_block_by_column_subblocks(gcn_block_ei, n_sub, grid.chunk, None, w_full)]
            else:
                gcn_blocks = None
            attn_blocks = [AttentionBlock(grid, ei, et, n_cols=n_cols_sub)
                           for ei, et, _ in split_block_by_column_subblocks(attn_block_ei, n_sub, grid.chunk, attn_block_et)]
            sp = None
            if sparse_comm:
                sp, self.sparse_info = build_sparse_comm(grid, attn_block, gcn_block, sparse_threshold, attn_subs=attn_blocks,
                                                         gcn_subs=gcn_blocks, **sp_kw)
                if sp is not None:
                    attn_blocks, gcn_blocks, self.sparse_comm = sp["attn"], sp["gcn"], sp
            if stream_sub > 1:
                def mk():
                    layer = DistExphormerLayerStreamed(grid, gcn_blocks, attn_blocks, *common, comm_dtype=comm_dtype,
                                                       rs_dtype=rs_dtype, tail_checkpoint=checkpoint,
                                                       kernel_dtype=kernel_dtype, with_gcn=with_gcn, norm=norm)
                    layer.overlap, layer.compact = stream_overlap, stream_compact
                    layer.sp_row = sp["row"] if sp is not None else None
                    layer.sp_cols = sp["cols"] if sp is not None else None
                    return layer
            else:
                mk = lambda: DistExphormerLayerPipelined(grid, gcn_blocks, attn_blocks, *common, comm_dtype=comm_dtype,   # noqa: E731
                                                         rs_dtype=rs_dtype, kernel_dtype=kernel_dtype, with_gcn=with_gcn, norm=norm)
        elif fused:
            sp = None
            if sparse_comm:
                sp, self.sparse_info = build_sparse_comm(grid, attn_block, gcn_block, sparse_threshold, **sp_kw)
                if sp is not None:
                    attn_block, gcn_block, self.sparse_comm = sp["attn"], sp["gcn"], sp
            mk = lambda: DistExphormerLayerFused(grid, gcn_block, attn_block, *common, comm_dtype=comm_dtype, rs_dtype=rs_dtype,   # noqa: E731
                                                 with_gcn=with_gcn, gather_proj=gather_proj, kernel_dtype=kernel_dtype,
                                                 sparse=sp, norm=norm)
        else:
            mk = lambda: DistExphormerLayer(grid, gcn_block, attn_block, *common, comm_dtype=comm_dtype, with_gcn=with_gcn,   # noqa: E731
                                            with_attn=with_attn, norm=norm)
        self.layers = nn.ModuleList([mk() for _ in range(num_layers)])
        if token_node is not None:
            # the global token's row and column as dense terms on the owned rows; the blocks must then not contain its edges
            if not (fused and stream_sub <= 1 and not ring and not head_grid):
                raise ValueError("a dense global token is implemented for the fused and pipelined layers")
            from ..parallel.token_dense import DenseToken
            for layer in self.layers:
                layer.token = DenseToken(grid, token_node)
        self.head = nn.Linear(dim_hidden, dim_out)

    def pre_mp(self, x):
        h = K.linear(x, self.pre_lin.weight)
        if isinstance(self.pre_bn, K.LayerNorm) and K.native_ok(h):
            # LayerNorm -> dropout -> ReLU -> L2 normalise in one kernel per direction
            return K.pre_mp(h, self.pre_bn, self.gnn_dropout if self.training else 0.0, self.pre_l2norm)
        h = F.relu(F.dropout(self.pre_bn(h), self.gnn_dropout, self.training))
        return F.normalize(h, p=2, dim=1) if self.pre_l2norm else h

    def forward(self, x_loc):
        h = self.pre_mp(x_loc)
        for layer in self.layers:
            if self.checkpoint and self.training and not getattr(layer, "self_checkpointing", False):
                h = torch.utils.checkpoint.checkpoint(layer, h, self.edge_type_emb.weight, use_reentrant=False)
            else:
                h = layer(h, self.edge_type_emb.weight)
        return K.linear(h, self.head.weight, self.head.bias)

    def flat_param_order(self):
        """Parameters that must be adjacent in the training engine's flat buffers, group by group."""
        out = []
        for layer in self.layers:
            if hasattr(layer, "stacked_params"):
                out += layer.stacked_params()
        return out

    def on_flat_layout(self, engine):
        """Called by the training engine once its flat buffers exist: hand every fused layer the stacked views."""
        if engine.flat_p_bf16 is None:
            return
        for layer in self.layers:
            if hasattr(layer, "stacked_params"):
                ps = layer.stacked_params()
                try:
                    layer._w_stack = (engine.span(ps, "bf16"), engine.span(ps, "grad"))
                except ValueError:
                    layer._w_stack = None

    def compaction_stats(self):
        """(row-block rows x sub-blocks, (row, sub-block) pairs owning an edge) of the first layer."""
        attns = getattr(self.layers[0], "attns", None)
        if attns is None:
            return 0, 0
        tot = ne = 0
        for a in attns:
            deg = a.block.crow[1:] - a.block.crow[:-1]
            tot += deg.numel()
            ne += int((deg > 0).sum())
        return tot, ne

    def structure_bytes(self):
        """Bytes of graph structures (blocks, cached plans, communication plans) reachable from the model."""
        from ..parallel.sparse_comm import SparseRowPlan
        seen, seen_obj, total = set(), set(), 0

        def walk(obj, depth):
            nonlocal total
            if id(obj) in seen_obj or depth > 6:
                return
            seen_obj.add(id(obj))
            if isinstance(obj, (GCNBlock, AttentionBlock, SparseRowPlan)):
                total += obj.nbytes(seen)
            elif isinstance(obj, dict):
                for v in obj.values():
                    walk(v, depth + 1)
            elif isinstance(obj, (list, tuple, nn.ModuleList)):
                for v in obj:
                    walk(v, depth + 1)
            elif isinstance(obj, nn.Module):
                for v in list(vars(obj).values()) + list(obj._modules.values()):
                    walk(v, depth + 1)
        walk(self, 0)
        return total

    @torch.no_grad()
    def load_ref_state_dict(self, sd):
        own = self.state_dict()
        for k, v in sd.items():
            if k not in own:
                raise KeyError(k)
            own[k].copy_(v)
        self.load_state_dict(own)

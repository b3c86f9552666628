"""Distributed masked sparse attention on the block grids.

``AttentionBlock``            the CSR of my block ``A[r, c]`` (shared by all layers of a model)
``DistMaskedSparseAttention`` "plain" operator: gathers Q / K / V, runs the block kernel, split-KV combine over the
                              row group, backward with global row statistics (5-6 collectives per direction)
``DistAttentionPartial``      block kernel on already gathered operands returning the unnormalised ``(acc, l, m)``;
                              its backward takes ``(dacc, dl)`` so no statistics gather is needed (fused layers)
``combine_partials``          the split-KV combine: optional softmax max all-reduce, ONE reduce-scatter carrying
                              ``[acc | l | extra]``, normalisation on the owner
``DistHeadSparseAttention``   the same on a 3D grid: Ulysses all-to-all inside the head group around the operator
``split_block_by_column_subblocks``  block -> per-sub-block edge lists for the pipelined / streamed layers

Semantics follow the reference (``gt3d/gt3d/dist/sparse_attention.py:59-437``).
"""
import torch
import torch.distributed as dist

from ..attention import BlockCSR, get_backend
from ..utils.timers import timers
from .collectives import (all_gather_rows, heads_to_rows, raw_all_gather_rows, raw_reduce_scatter_rows,
                          reduce_scatter_rows, rows_to_heads)
from .grid import group_size


class AttentionBlock:
    """CSR of the attention block of this rank: rows = row block (row-local dst), columns = column block."""

    def __init__(self, grid, block_edge_index, block_edge_type=None, n_cols=None):
        n_cols = grid.n_col_block if n_cols is None else n_cols
        self.csr = BlockCSR.from_edges(block_edge_index, grid.n_row_block, n_cols, block_edge_type)

    @classmethod
    def from_csr(cls, csr: BlockCSR):
        self = cls.__new__(cls)
        self.csr = csr
        return self

    # convenience views -----------------------------------------------------------------------------------------
    @property
    def crow(self):
        return self.csr.crow

    @property
    def col(self):
        return self.csr.col

    @property
    def etype(self):
        return self.csr.etype

    @property
    def num_edges(self):
        return self.csr.num_edges

    def to(self, device):
        self.csr = self.csr.to(device)
        return self

    def compacted(self, rows_need, col_remap, n_cols_c):
        return AttentionBlock.from_csr(self.csr.compacted(rows_need, col_remap, n_cols_c))

    def nbytes(self, seen=None):
        return self.csr.nbytes(seen)


def _as_block(grid, block):
    if isinstance(block, AttentionBlock):
        return block
    if isinstance(block, BlockCSR):
        return AttentionBlock.from_csr(block)
    return AttentionBlock(grid, *block)


def _stat_dtype(dtype):
    return torch.float64 if dtype == torch.float64 else torch.float32


class _DistAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_loc, k_loc, v_loc, gate, bias, mod):
        g, be = mod.grid, get_backend(mod.backend)
        wire = mod.comm_dtype or q_loc.dtype
        k_blk = raw_all_gather_rows(k_loc.to(wire), g.col_group)
        v_blk = raw_all_gather_rows(v_loc.to(wire), g.col_group)
        q_blk = raw_all_gather_rows(q_loc.to(wire), g.row_group)
        if mod.backend == "torch":
            q_blk, k_blk, v_blk = q_blk.to(q_loc.dtype), k_blk.to(q_loc.dtype), v_blk.to(q_loc.dtype)
        sdt = _stat_dtype(q_loc.dtype)
        gate_c = gate.to(sdt if mod.backend != "torch" else q_loc.dtype) if gate is not None else None
        bias_c = bias.to(sdt if mod.backend != "torch" else q_loc.dtype) if bias is not None else None
        acc, l, m = be.attn_fwd_partial(q_blk, k_blk, v_blk, mod.block.csr, gate_c, bias_c, score=mod.score,
                                        norm=mod.norm, clamp=mod.clamp, scale=mod.scale)
        acc, l, m = acc.to(sdt), l.to(sdt), m.to(sdt)
        if mod.norm == "softmax" and group_size(g.row_group) > 1:
            m_glob = m.clone()
            dist.all_reduce(m_glob, op=dist.ReduceOp.MAX, group=g.row_group)
            w = torch.exp(m - m_glob)
            acc, l, m = acc * w.unsqueeze(-1), l * w, m_glob
        n_rows, h, d = acc.shape
        packed = raw_reduce_scatter_rows(torch.cat([acc.reshape(n_rows, h * d), l], dim=1), g.row_group)
        acc_o, l_o = packed[:, :h * d].reshape(-1, h, d), packed[:, h * d:].contiguous()
        m_o = m[g.row_pos * g.chunk:(g.row_pos + 1) * g.chunk].contiguous()
        o_loc = be.normalize(acc_o, l_o, mod.norm, mod.eps).to(q_loc.dtype)
        ctx.mod, ctx.in_dtype = mod, q_loc.dtype
        ctx.gate_dtype = gate.dtype if gate is not None else None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.save_for_backward(q_blk, k_blk, v_blk, o_loc, l_o, m_o, gate_c, bias_c)
        return o_loc

    @staticmethod
    def backward(ctx, do_loc):
        mod = ctx.mod
        g, be = mod.grid, get_backend(mod.backend)
        q_blk, k_blk, v_blk, o_loc, l_o, m_o, gate_c, bias_c = ctx.saved_tensors
        h, d = q_blk.shape[1], q_blk.shape[2]
        sdt = l_o.dtype
        wire = mod.comm_dtype or ctx.in_dtype
        n = o_loc.shape[0]
        # the row block's (o, dO) in the wire dtype and its statistics (l, m) in the statistics dtype
        odo = raw_all_gather_rows(torch.cat([o_loc.reshape(n, -1), do_loc.reshape(n, -1)], dim=1).to(wire), g.row_group)
        lm = raw_all_gather_rows(torch.cat([l_o, m_o], dim=1), g.row_group)
        o_blk, do_blk = odo[:, :h * d].reshape(-1, h, d), odo[:, h * d:].reshape(-1, h, d)
        if mod.backend == "torch":
            o_blk, do_blk = o_blk.to(ctx.in_dtype), do_blk.to(ctx.in_dtype)
        l_blk, m_blk = lm[:, :h].contiguous().to(sdt), lm[:, h:].contiguous().to(sdt)
        if mod.backend == "torch":
            l_blk, m_blk = l_blk.to(ctx.in_dtype), m_blk.to(ctx.in_dtype)
        dq, dk, dv, dgate, dbias = be.attn_bwd(q_blk, k_blk, v_blk, mod.block.csr, gate_c, bias_c, o_blk, l_blk, m_blk,
                                               do_blk, score=mod.score, norm=mod.norm, clamp=mod.clamp, eps=mod.eps,
                                               scale=mod.scale)
        rdt = ctx.in_dtype
        dq_loc = raw_reduce_scatter_rows(dq.to(rdt), g.row_group)
        dk_loc = raw_reduce_scatter_rows(dk.to(rdt), g.col_group)
        dv_loc = raw_reduce_scatter_rows(dv.to(rdt), g.col_group)
        # dgate / dbias are this rank's partial sums; the trainer's gradient all-reduce adds the ranks
        return (dq_loc, dk_loc, dv_loc, dgate.to(ctx.gate_dtype) if dgate is not None else None,
                dbias.to(ctx.bias_dtype) if dbias is not None else None, None)


class _OpBase(torch.nn.Module):
    def __init__(self, grid, block, num_heads, head_dim, backend, score, norm, clamp, eps):
        super().__init__()
        self.grid, self.block = grid, _as_block(grid, block)
        self.h, self.d = num_heads, head_dim
        self.backend, self.score, self.norm, self.clamp, self.eps = backend, score, norm, tuple(clamp), eps
        self.scale = 1.0 / (head_dim ** 0.5)

    def _apply(self, fn, *a, **kw):          # move the block with the module (.to / .cuda)
        out = super()._apply(fn, *a, **kw)
        probe = fn(torch.zeros(0, device=self.block.csr.device))
        self.block.to(probe.device)
        return out


class DistMaskedSparseAttention(_OpBase):
    """Inputs / output: the owned chunk ``[chunk, H, d]``."""

    def __init__(self, grid, block, num_heads, head_dim, backend="cuda", score="gated", norm="clampexp",
                 clamp=(-5.0, 5.0), eps=1e-6, comm_dtype=None):
        super().__init__(grid, block, num_heads, head_dim, backend, score, norm, clamp, eps)
        self.comm_dtype = comm_dtype

    def forward(self, q_local, k_local, v_local, gate=None, bias=None):
        return _DistAttention.apply(q_local.contiguous(), k_local.contiguous(), v_local.contiguous(), gate, bias, self)


class _AttnPartial(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q_blk, k_blk, v_blk, gate, bias, mod):
        be = get_backend(mod.backend)
        tdt = q_blk.dtype if mod.backend == "torch" else torch.float32
        gate_c = gate.to(tdt) if gate is not None else None
        bias_c = bias.to(tdt) if bias is not None else None
        t = timers()
        t.start("attn fwd kernel")
        acc, l, m = be.attn_fwd_partial(q_blk, k_blk, v_blk, mod.block.csr, gate_c, bias_c, score=mod.score,
                                        norm=mod.norm, clamp=mod.clamp, scale=mod.scale)
        t.stop("attn fwd kernel")
        ctx.mod = mod
        ctx.gate_dtype = gate.dtype if gate is not None else None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        ctx.save_for_backward(q_blk, k_blk, v_blk, m, gate_c, bias_c)
        ctx.mark_non_differentiable(m)
        return acc, l, m

    @staticmethod
    def backward(ctx, dacc, dl, _dm):
        mod = ctx.mod
        be = get_backend(mod.backend)
        q_blk, k_blk, v_blk, m, gate_c, bias_c = ctx.saved_tensors
        t = timers()
        t.start("attn bwd kernel")
        dq, dk, dv, dgate, dbias = be.attn_bwd_partial(q_blk, k_blk, v_blk, mod.block.csr, gate_c, bias_c, m,
                                                       dacc.contiguous(), dl.contiguous(), score=mod.score,
                                                       norm=mod.norm, clamp=mod.clamp, scale=mod.scale)
        t.stop("attn bwd kernel")
        return (dq.to(q_blk.dtype), dk.to(k_blk.dtype), dv.to(v_blk.dtype),
                dgate.to(ctx.gate_dtype) if dgate is not None and ctx.gate_dtype is not None else None,
                dbias.to(ctx.bias_dtype) if dbias is not None and ctx.bias_dtype is not None else None, None)


class _AttnPullKV(torch.autograd.Function):
    """Block attention whose forward kernel reads the K / V rows it needs straight from the owners' memory (receiver-driven
    pull over NVLink inside the gather loop): the column-group all-gather of K and V does not exist in the forward.
    Backward gathers K and V once (peer-memory all-gather) for the row and column passes and reduce-scatters dK, dV.
    Worth it when a tile references few of the block's rows (each needed row crosses the link once per referencing edge)."""

    @staticmethod
    def forward(ctx, q_blk, k_loc, v_loc, gate, mod):
        from ..attention import backend_cuda as bc
        heap, g = mod.heap, mod.grid
        _, k_tab = heap.publish(k_loc, g.col_group, "pull_k")
        _, v_tab = heap.publish(v_loc, g.col_group, "pull_v")
        gate_c = gate.float() if gate is not None else None
        acc, l, m = bc.attn_fwd_partial_pull(q_blk, k_tab, v_tab, k_loc.shape[0], mod.block.csr, gate_c, None, score=mod.score,
                                             norm=mod.norm, clamp=mod.clamp, scale=mod.scale)
        ctx.mod, ctx.gate_dtype = mod, gate.dtype if gate is not None else None
        ctx.save_for_backward(q_blk, k_loc, v_loc, m, gate_c)
        ctx.mark_non_differentiable(m)
        return acc, l, m

    @staticmethod
    def backward(ctx, dacc, dl, _dm):
        from ..attention import backend_cuda as bc
        mod = ctx.mod
        q_blk, k_loc, v_loc, m, gate_c = ctx.saved_tensors
        g = mod.grid
        k_blk, v_blk = raw_all_gather_rows(k_loc, g.col_group), raw_all_gather_rows(v_loc, g.col_group)
        dq, dk, dv, dgate, _ = bc.attn_bwd_partial(q_blk, k_blk, v_blk, mod.block.csr, gate_c, None, m, dacc.contiguous(), dl.contiguous(),
                                                   score=mod.score, norm=mod.norm, clamp=mod.clamp, scale=mod.scale)
        dk = raw_reduce_scatter_rows(dk.to(k_loc.dtype), g.col_group)
        dv = raw_reduce_scatter_rows(dv.to(v_loc.dtype), g.col_group)
        return dq.to(q_blk.dtype), dk, dv, (dgate.to(ctx.gate_dtype) if dgate is not None and ctx.gate_dtype is not None else None), None


class DistAttentionPullKV(_OpBase):
    """``q_blk [rows, H, d]`` (gathered over the row group), ``k_loc, v_loc [chunk, H, d]`` (OWNED rows, projected by the
    owner) -> unnormalised ``(acc, l, m)`` of the block; K / V rows are pulled from peer memory inside the kernel."""

    def __init__(self, grid, block, num_heads, head_dim, heap, score="gated", norm="clampexp", clamp=(-5.0, 5.0)):
        super().__init__(grid, block, num_heads, head_dim, "cuda", score, norm, clamp, 1e-6)
        if not heap.group_is_local(grid.col_group):
            raise ValueError("K / V rows are pulled from peer memory: the column group must lie within one machine")
        self.heap = heap

    def forward(self, q_blk, k_loc, v_loc, gate=None):
        return _AttnPullKV.apply(q_blk.contiguous(), k_loc.contiguous(), v_loc.contiguous(), gate, self)


class DistAttentionPartial(_OpBase):
    """Unnormalised block attention on gathered operands: ``q [rows, H, d]``, ``k, v [cols, H, d]`` -> ``(acc, l, m)``."""

    def __init__(self, grid, block, num_heads, head_dim, backend="cuda", score="gated", norm="clampexp",
                 clamp=(-5.0, 5.0)):
        super().__init__(grid, block, num_heads, head_dim, backend, score, norm, clamp, 1e-6)

    def forward(self, q_blk, k_blk, v_blk, gate=None, bias=None):
        return _AttnPartial.apply(q_blk.contiguous(), k_blk.contiguous(), v_blk.contiguous(), gate, bias, self)


def _pack_ok(parts):
    if not parts[0].is_cuda:
        return False
    from ..ops import native
    return native.pack_ok(parts)


class _PackedReduceScatter(torch.autograd.Function):
    """Reduce-scatter of several column blocks in ONE payload: ``parts [rows, w_i]`` are packed into the wire dtype by one
    kernel, reduced over the group, and unpacked to the parts' own dtypes; backward is pack -> all-gather -> unpack."""

    @staticmethod
    def forward(ctx, group, wire, *parts):
        from ..ops import native
        wire = wire or torch.float32
        ctx.group, ctx.wire = group, wire
        ctx.widths, ctx.dtypes = [p.shape[1] for p in parts], [p.dtype for p in parts]
        packed = native.pack_columns([p.detach() for p in parts], wire)
        out = raw_reduce_scatter_rows(packed, group)
        return tuple(native.unpack_columns(out, ctx.widths, ctx.dtypes))

    @staticmethod
    def backward(ctx, *grads):
        from ..ops import native
        ref = next(g for g in grads if g is not None)
        grads = [g if g is not None else ref.new_zeros(ref.shape[0], w) for g, w in zip(grads, ctx.widths)]
        packed = native.pack_columns(grads, ctx.wire)
        full = raw_all_gather_rows(packed, ctx.group)
        return (None, None) + tuple(native.unpack_columns(full, ctx.widths, ctx.dtypes))


def combine_partials(acc, l, m, grid, norm, eps, extra=None, rs_dtype=None, plan=None, normalize=True):
    """Merge the block partials of a row group onto the owner of every row; returns ``(o_owned, extra_owned)``.

    softmax: the partials are first rescaled to the row-group maximum of ``m`` (one MAX all-reduce; no gradient flows
    through ``m``).  ``extra [rows, F]`` (e.g. the GCN aggregation partial) rides in the same reduce-scatter.
    ``rs_dtype`` reduces the payload in low precision.  ``plan``: a :class:`~gt_b200.parallel.sparse_comm.SparseRowPlan`
    of the row group; the partials are then given for the plan's compact rows only.  ``normalize=False`` returns
    ``((acc_owned [n, H d], l_owned [n, H]), extra_owned)`` so that the division can be fused into the consumer."""
    if norm == "softmax" and group_size(grid.row_group) > 1:
        if plan is None:
            m_glob = m.detach().clone()
        else:
            m_glob = torch.full((plan.g * plan.rows_per_rank, m.shape[1]), float("-inf"), dtype=m.dtype, device=m.device)
            m_glob[plan.need_local.long()] = m.detach()
        dist.all_reduce(m_glob, op=dist.ReduceOp.MAX, group=grid.row_group)
        if plan is not None:
            m_glob = m_glob[plan.need_local.long()]
        w = torch.exp(m.detach() - m_glob)
        acc, l = acc * w.unsqueeze(-1), l * w
    n_rows, h, d = acc.shape
    if group_size(grid.row_group) == 1 and plan is None:
        # one rank per row group: nothing to reduce, so the [acc | l | extra] payload is never built
        acc_o, l_o, extra_o = acc, l, extra
        if not normalize:
            return (acc_o.reshape(n_rows, h * d), l_o), extra_o
        o = acc_o / (torch.where(l_o > 0, l_o, torch.ones_like(l_o)) if norm == "softmax" else (l_o + eps)).unsqueeze(-1)
        return o, extra_o
    if plan is None and _pack_ok([acc.reshape(n_rows, h * d), l] + ([extra] if extra is not None else [])):
        # one packing pass into the wire dtype, the collective, one unpacking pass (instead of cat / cast / slice / cast)
        outs = _PackedReduceScatter.apply(grid.row_group, rs_dtype, acc.reshape(n_rows, h * d), l, *([extra] if extra is not None else []))
        acc_o, l_o, extra_o = outs[0], outs[1], (outs[2] if extra is not None else None)
        if not normalize:
            return (acc_o, l_o), extra_o
        acc_o = acc_o.reshape(-1, h, d)
        o = acc_o / (torch.where(l_o > 0, l_o, torch.ones_like(l_o)) if norm == "softmax" else (l_o + eps)).unsqueeze(-1)
        return o, extra_o
    parts, width = [acc.reshape(n_rows, h * d), l], h * d + h
    if extra is not None:
        parts.append(extra.to(acc.dtype))
        width += extra.shape[1]
    packed = torch.cat(parts, dim=1)
    if plan is None:
        packed = reduce_scatter_rows(packed, grid.row_group, rs_dtype)
    else:
        from .sparse_comm import sparse_reduce_scatter
        packed = sparse_reduce_scatter(packed, plan, rs_dtype)
    acc_o, l_o = packed[:, :h * d].reshape(-1, h, d), packed[:, h * d:h * d + h]
    if not normalize:
        return (packed[:, :h * d], l_o.contiguous()), (packed[:, h * d + h:width] if extra is not None else None)
    if norm == "softmax":
        o = acc_o / torch.where(l_o > 0, l_o, torch.ones_like(l_o)).unsqueeze(-1)
    else:
        o = acc_o / (l_o + eps).unsqueeze(-1)
    return o, (packed[:, h * d + h:width] if extra is not None else None)


def split_block_by_column_subblocks(edge_index_local, n_sub, chunk, etype=None, weight=None):
    """Cut a local block by column sub-block ``s = (src % chunk) // (chunk / n_sub)`` and renumber the sources to the
    order of the gathered sub-block (``owner * cs + offset``).  Returns a list of ``(edge_index, etype, weight)``."""
    if chunk % n_sub:
        raise ValueError(f"chunk {chunk} must be divisible by n_sub {n_sub}")
    cs = chunk // n_sub
    src, dst = edge_index_local[0], edge_index_local[1]
    owner, off = src // chunk, src % chunk
    sub = off // cs
    out = []
    for s in range(n_sub):
        sel = sub == s
        out.append((torch.stack([owner[sel] * cs + (off[sel] - s * cs), dst[sel]]),
                    etype[sel] if etype is not None else None, weight[sel] if weight is not None else None))
    return out


def split_block_by_source_chunk(edge_index_local, p, chunk, etype=None, weight=None):
    """Cut a (P, 1)-grid block by the chunk that owns the source (one piece per ring step), sources renumbered to the
    chunk.  Returns a list of ``(edge_index, etype, weight)``."""
    src, dst = edge_index_local[0], edge_index_local[1]
    owner = src // chunk
    out = []
    for s in range(p):
        sel = owner == s
        out.append((torch.stack([src[sel] - s * chunk, dst[sel]]), etype[sel] if etype is not None else None,
                    weight[sel] if weight is not None else None))
    return out


class DistHeadSparseAttention(torch.nn.Module):
    """Attention on a 3D grid: owners project all heads, rows <-> heads all-to-all inside the head group, gather of the
    head slice over the row (Q) / column (K, V) group, block kernel on ``H / P_i`` heads, split-KV combine over the row
    group, all-to-all back.  ``(1, 1, P)`` is pure head parallelism (DeepSpeed-Ulysses)."""

    def __init__(self, grid, block, num_heads, head_dim, backend="cuda", score="gated", norm="clampexp",
                 clamp=(-5.0, 5.0), eps=1e-6, comm_dtype=None, rs_dtype=None, no_comm=False):
        super().__init__()
        if num_heads % grid.p_heads:
            raise ValueError("the head axis must divide the number of heads")
        self.grid, self.h, self.d, self.hg = grid, num_heads, head_dim, num_heads // grid.p_heads
        self.norm, self.eps, self.comm_dtype, self.rs_dtype, self.no_comm = norm, eps, comm_dtype, rs_dtype, no_comm
        self.partial = DistAttentionPartial(grid, block, self.hg, head_dim, backend=backend, score=score, norm=norm,
                                            clamp=clamp)

    def _to_block(self, t, group):
        g = self.grid
        if self.no_comm:                                  # timing stand-in of the same shape
            reps = g.p_heads * group_size(group)
            return t[:, g.h * self.hg:(g.h + 1) * self.hg].repeat(reps, 1, 1)
        wire = t.to(self.comm_dtype) if self.comm_dtype is not None else t
        return all_gather_rows(rows_to_heads(wire, g.head_group, g.p_heads), group).to(t.dtype)

    def forward(self, q_loc, k_loc, v_loc, gate=None, bias=None):
        g, t = self.grid, timers()
        t.start("head: a2a + gather q/k/v")
        q_blk = self._to_block(q_loc.contiguous(), g.row_group)
        k_blk = self._to_block(k_loc.contiguous(), g.col_group)
        v_blk = self._to_block(v_loc.contiguous(), g.col_group)
        t.stop("head: a2a + gather q/k/v")
        sl = slice(g.h * self.hg, (g.h + 1) * self.hg)
        gate_h = gate[:, sl].contiguous() if gate is not None else None
        bias_h = bias[:, sl].contiguous() if bias is not None else None
        acc, l, m = self.partial(q_blk, k_blk, v_blk, gate_h, bias_h)
        if self.no_comm:
            n_rows, hg, d = acc.shape
            gr = group_size(g.row_group)
            packed = torch.cat([acc.reshape(n_rows, -1), l], dim=1).view(gr, n_rows // gr, -1).sum(0)
            o_h = packed[:, :hg * d].view(-1, hg, d) / (packed[:, hg * d:] + self.eps).unsqueeze(-1)
            chunk = o_h.shape[0] // g.p_heads
            return o_h.view(g.p_heads, chunk, hg, d).transpose(0, 1).reshape(chunk, self.h, d).to(q_loc.dtype)
        t.start("reduce-scatter")
        o_h, _ = combine_partials(acc, l, m, g, self.norm, self.eps, rs_dtype=self.rs_dtype)
        t.stop("reduce-scatter")
        t.start("head: a2a back")
        wire = o_h.to(self.comm_dtype) if self.comm_dtype is not None else o_h
        out = heads_to_rows(wire.contiguous(), g.head_group, g.p_heads).to(q_loc.dtype)
        t.stop("head: a2a back")
        return out

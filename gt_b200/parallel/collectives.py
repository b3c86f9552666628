"""Row collectives of the grids, paired for autograd.

Every dense tensor is node-sharded ``[chunk, ...]``; the layers move rows with

* ``all_gather_rows(x, group)``       ``[chunk, ...] -> [G * chunk, ...]``; backward = reduce-scatter
* ``reduce_scatter_rows(x, group)``   ``[G * chunk, ...] -> [chunk, ...]`` (sum); backward = all-gather
* ``all_gather_rows_start`` / ``wait_gather``   asynchronous gather (prefetch of the next column sub-block)
* ``rows_to_heads`` / ``heads_to_rows``         the Ulysses all-to-all of the head axis and its inverse
* ``all_reduce_sum``                  sum with the all-reduced gradient (statistics consumed by every rank)

(reference: ``gt3d/gt3d/dist/grid2d.py:209-323``, ``grid3d.py:141-206``, ``layers.py:24-50``).  A ``wire`` dtype
(e.g. bf16) may be given: the payload is cast for the transfer and cast back.  The raw functions run on NCCL (GPU) or
gloo (CPU tests; gloo has no reduce-scatter, so it is emulated with an all-reduce).  The B200 fast path replaces these
NCCL calls by kernels that read / write peer memory directly (:mod:`gt_b200.parallel.symm`); the layers select it with
``comm="p2p"``.  Unlike the reference there is no host synchronisation before a collective by default: inside one NVSwitch
domain concurrent row- and column-group traffic does not share a NIC (``GT_SYNC_COLLECTIVES`` switches it on).
"""
import os

import torch
import torch.distributed as dist

from ..utils.timers import timers
from .grid import group_name, group_size

_STATS_HOOK = [None]          # set by utils.collstats to time every raw collective
_HEAP = [None]                # symmetric heap: when set, CUDA row collectives run on the package's peer-memory kernels


def set_transport(heap):
    """Route the dense row collectives of CUDA tensors through ``heap`` (a :class:`~gt_b200.parallel.symm.SymmetricHeap`);
    ``None`` restores NCCL."""
    _HEAP[0] = heap


def _p2p_ok(x, group, rows_out):
    h = _HEAP[0]
    if h is None or not h.reaches(x, group) or x.dtype not in h._float_types():
        return False
    per_rank = x.numel() // (group_size(group) if rows_out else 1)
    return (per_rank * x.element_size()) % 16 == 0 and per_rank % 8 == 0


def _a2a_p2p_ok(x, slab_elems, group):
    h = _HEAP[0]
    return h is not None and h.reaches(x, group) and x.dtype in h._float_types() and (slab_elems * x.element_size()) % 16 == 0


# GT_SYNC_COLLECTIVES (default 0): 1 = host-synchronise the current stream before every synchronous collective, so that the previous
# collective, possibly on another communicator, has completed before this one is posted; 2 = also a barrier over the group.  On
# one NVSwitch node communicators do not share a NIC and the default is off; the reference needs the synchronisation when two
# cross-node groups share a network interface (``gt3d/gt3d/dist/grid2d.py:55-69``, default on there), and multi-node runs of this
# package on NCCL can switch it on for the same reason.  Asynchronous gathers are never synchronised.
SYNC_COLLECTIVES = int(os.environ.get("GT_SYNC_COLLECTIVES", "0"))


def _pre_collective(group):
    if SYNC_COLLECTIVES and torch.cuda.is_available() and not torch.cuda.is_current_stream_capturing():
        torch.cuda.current_stream().synchronize()
        if SYNC_COLLECTIVES >= 2 and group_size(group) > 1:
            dist.barrier(group=group)


def _instrument(kind, group, nbytes, fn):
    if SYNC_COLLECTIVES:
        _pre_collective(group)
    hook = _STATS_HOOK[0]
    if hook is None:
        return fn()
    return hook(kind, group, nbytes, fn)


def _is_gloo(group):
    return dist.get_backend(group) == "gloo"


def raw_all_gather_rows(x, group, async_op=False):
    """``[chunk, ...] -> [G * chunk, ...]`` in group-rank order.  ``async_op`` returns ``(work, out)``."""
    g = group_size(group)
    if g == 1:
        return (None, x) if async_op else x
    x = x.contiguous()
    if _p2p_ok(x, group, False):
        out = _instrument("all_gather", group, g * x.numel() * x.element_size(), lambda: _HEAP[0].all_gather(x, group))
        return (None, out) if async_op else out
    out = x.new_empty((g * x.shape[0],) + tuple(x.shape[1:]))
    if async_op:
        return dist.all_gather_into_tensor(out, x, group=group, async_op=True), out
    _instrument("all_gather", group, out.numel() * out.element_size(),
                lambda: dist.all_gather_into_tensor(out, x, group=group))
    return out


def raw_reduce_scatter_rows(x, group, async_op=False):
    """``[G * chunk, ...]`` partial sums ``-> [chunk, ...]`` (the rows of my group rank)."""
    g = group_size(group)
    if g == 1:
        return (None, x) if async_op else x
    x = x.contiguous()
    n = x.shape[0] // g
    if _p2p_ok(x, group, True):
        out = _instrument("reduce_scatter", group, x.numel() * x.element_size(), lambda: _HEAP[0].reduce_scatter(x, group))
        return (None, out) if async_op else out
    if _is_gloo(group):
        def run():
            y = x.clone() if x.dtype != torch.bfloat16 else x.float()
            dist.all_reduce(y, group=group)
            me = dist.get_rank(group)
            return y[me * n:(me + 1) * n].to(x.dtype).contiguous()
        out = _instrument("reduce_scatter", group, x.numel() * x.element_size(), run)
        return (None, out) if async_op else out
    out = x.new_empty((n,) + tuple(x.shape[1:]))
    if async_op:
        return dist.reduce_scatter_tensor(out, x, group=group, async_op=True), out
    _instrument("reduce_scatter", group, x.numel() * x.element_size(),
                lambda: dist.reduce_scatter_tensor(out, x, group=group))
    return out


def raw_all_to_all(x, group):
    """Equal-split all-to-all over dim 0."""
    if group_size(group) == 1:
        return x
    x = x.contiguous()
    out = torch.empty_like(x)
    _instrument("all_to_all", group, x.numel() * x.element_size(), lambda: dist.all_to_all_single(out, x, group=group))
    return out


def raw_rows_to_heads(x, group, p):
    """``[chunk, H, d]`` (my rows, all heads) ``-> [p * chunk, H / p, d]`` (the rows of my head group, my heads)."""
    if p == 1:
        return x
    chunk, h, d = x.shape
    if _a2a_p2p_ok(x, (h // p) * d, group):
        return _HEAP[0].rows_to_heads(x.contiguous(), group)
    send = x.view(chunk, p, h // p, d).transpose(0, 1).contiguous()
    return raw_all_to_all(send, group).view(p * chunk, h // p, d)


def raw_heads_to_rows(y, group, p):
    """Inverse of ``raw_rows_to_heads``: ``[p * chunk, H / p, d] -> [chunk, H, d]``."""
    if p == 1:
        return y
    n, hg, d = y.shape
    chunk = n // p
    if _a2a_p2p_ok(y, hg * d, group):
        return _HEAP[0].heads_to_rows(y.contiguous(), group)
    recv = raw_all_to_all(y.contiguous().view(p, chunk, hg, d), group)
    return recv.transpose(0, 1).contiguous().view(chunk, p * hg, d)


def _wire(x, wire):
    return x if wire is None or wire == x.dtype else x.to(wire)


class _AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, wire):
        ctx.group, ctx.wire, ctx.dtype = group, wire, x.dtype
        return raw_all_gather_rows(_wire(x, wire), group).to(x.dtype)

    @staticmethod
    def backward(ctx, grad):
        t = timers()
        name = f"bwd reduce-scatter ({group_name(ctx.group)})"
        t.start(name)
        out = raw_reduce_scatter_rows(_wire(grad, ctx.wire), ctx.group).to(ctx.dtype)
        t.stop(name)
        return out, None, None


class _ReduceScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, wire):
        ctx.group, ctx.wire, ctx.dtype = group, wire, x.dtype
        return raw_reduce_scatter_rows(_wire(x, wire), group).to(x.dtype)

    @staticmethod
    def backward(ctx, grad):
        t = timers()
        name = f"bwd all-gather ({group_name(ctx.group)})"
        t.start(name)
        out = raw_all_gather_rows(_wire(grad, ctx.wire), ctx.group).to(ctx.dtype)
        t.stop(name)
        return out, None, None


def all_gather_rows(x, group, wire=None):
    return _AllGatherRows.apply(x, group, wire)


def reduce_scatter_rows(x, group, wire=None):
    return _ReduceScatterRows.apply(x, group, wire)


class PendingGather:
    """Handle of an asynchronous gather: ``buf`` becomes valid after ``wait()``."""

    def __init__(self, work, buf, keep=None):
        self.work, self.buf, self.keep = work, buf, keep

    def wait(self):
        if self.work is not None:
            self.work.wait()
            self.work = None
        self.keep = None
        return self.buf


class _GatherStart(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, wire, holder):
        ctx.group, ctx.wire, ctx.dtype = group, wire, x.dtype
        xs = _wire(x, wire).contiguous()
        work, buf = raw_all_gather_rows(xs, group, async_op=True)
        holder.append(PendingGather(work, buf, keep=xs))
        return buf

    @staticmethod
    def backward(ctx, grad):
        return raw_reduce_scatter_rows(_wire(grad, ctx.wire), ctx.group).to(ctx.dtype), None, None, None


class _GatherWait(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, pending, dtype):
        pending.wait()
        return buf.to(dtype) if buf.dtype != dtype else buf.view_as(buf)

    @staticmethod
    def backward(ctx, grad):
        return grad, None, None


def all_gather_rows_start(x, group, wire=None):
    """Start an asynchronous gather; returns an opaque handle for ``wait_gather``."""
    holder = []
    buf = _GatherStart.apply(x, group, wire, holder)
    return buf, holder[0], x.dtype


def wait_gather(handle):
    buf, pending, dtype = handle
    return _GatherWait.apply(buf, pending, dtype)


class _RowsToHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, p):
        ctx.group, ctx.p = group, p
        return raw_rows_to_heads(x, group, p)

    @staticmethod
    def backward(ctx, grad):
        t = timers()
        t.start("bwd all-to-all (head)")
        out = raw_heads_to_rows(grad.contiguous(), ctx.group, ctx.p)
        t.stop("bwd all-to-all (head)")
        return out, None, None


class _HeadsToRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, group, p):
        ctx.group, ctx.p = group, p
        return raw_heads_to_rows(y, group, p)

    @staticmethod
    def backward(ctx, grad):
        t = timers()
        t.start("bwd all-to-all (head)")
        out = raw_rows_to_heads(grad.contiguous(), ctx.group, ctx.p)
        t.stop("bwd all-to-all (head)")
        return out, None, None


def rows_to_heads(x, group, p):
    return _RowsToHeads.apply(x, group, p)


def heads_to_rows(y, group, p):
    return _HeadsToRows.apply(y, group, p)


def _sum_over_ranks(x, group):
    """Sum of ``x`` over the group in a new tensor.  Small CUDA payloads (normalisation statistics, loss terms) take the
    one-shot peer-memory all-reduce when the peer-memory transport is on: one kernel that reads every rank's buffer."""
    if group_size(group) == 1:
        return x.clone()
    h = _HEAP[0]
    if h is not None and h.reaches(x, group) and x.dtype in h._float_types() and x.numel() % 8 == 0 and x.numel() > 0:
        x = x.contiguous()
        return _instrument("all_reduce", group, x.numel() * x.element_size(), lambda: h.all_reduce(x, torch.empty_like(x), group=group))
    y = x.clone()
    dist.all_reduce(y, group=group)
    return y


class _AllReduceSum(torch.autograd.Function):
    """``y = sum over ranks of x`` where every rank consumes ``y``: the gradient w.r.t. the local ``x`` is the sum over
    ranks of the upstream gradients."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _sum_over_ranks(x, group)

    @staticmethod
    def backward(ctx, g):
        return _sum_over_ranks(g.contiguous(), ctx.group), None


def all_reduce_sum(x, group=None):
    return _AllReduceSum.apply(x, group)

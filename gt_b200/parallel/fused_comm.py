"""Projections with their collective inside the GEMM kernel (peer memory over NVLink, symmetric heap).

``linear_gather(x, W, group)`` is ``all_gather_rows(x, group) @ W^T`` and its backward, with

* forward: ONE tcgen05 kernel whose TMA loads fetch every rank's rows of ``x`` from the owner's memory (the all-gather
  never exists as a separate step; the gathered ``x`` is written as a by-product for the weight gradient),
* backward: the input-gradient GEMM stores each finished tile into the owning rank's memory from its epilogue (the
  reduce-scatter's transfer overlaps the MMAs), followed by a barrier and a local sum of the ``G`` slots.

The reference issues these as separate NCCL collectives around cuBLAS GEMMs (``gt3d/gt3d/models/exphormer_dist.py:
440-447`` forward gathers + projections, ``gt3d/gt3d/dist/grid2d.py`` all-gather / reduce-scatter autograd pairs).
Falls back to the unfused pair when no heap is active, the group has one rank, or the shape is outside the fused
kernel's limits (K <= 512, bf16).
"""
import torch

from ..ops import functional as K
from ..ops import native
from .collectives import _HEAP, all_gather_rows
from .grid import group_size


def fused_ok(x, weight, group):
    heap = _HEAP[0]
    return (heap is not None and x.is_cuda and heap.group_is_local(group) and x.dtype == torch.bfloat16 and group_size(group) > 1 and x.dim() == 2
            and x.shape[1] % 8 == 0 and x.shape[1] <= 512 and weight.shape[0] % 8 == 0 and group_size(group) <= 8)


class _LinearGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, group):
        heap = _HEAP[0]
        wb = weight.to(torch.bfloat16).contiguous()
        y, xg = heap.linear_gather(x, wb, group, want_gathered=True)
        ctx.save_for_backward(xg, wb)
        ctx.group, ctx.heap, ctx.wdt = group, heap, weight.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        xg, wb = ctx.saved_tensors
        dy = dy.contiguous()
        dw = native.gemm_tn(dy, xg).to(ctx.wdt) if ctx.needs_input_grad[1] else None
        dx = ctx.heap.linear_scatter(dy, wb.t().contiguous(), ctx.group) if ctx.needs_input_grad[0] else None
        return dx, dw, None


def linear_gather(x, weight, group, wire=None):
    """``all_gather_rows(x, group) @ weight^T`` (no bias)."""
    if fused_ok(x, weight, group):
        return _LinearGather.apply(x, weight, group)
    return K.linear(all_gather_rows(x, group, wire), weight)

"""Sparse aggregation ``out = A @ x`` over a :class:`~gt_b200.attention.csr.BlockCSR` with values ``blk.weight``.

Forward walks the CSR, backward walks the cached transpose (``dx = A^T @ dout``), so neither direction needs atomics or
an ``[E, d]`` temporary.  On CUDA tensors the native warp-per-row kernel runs (:mod:`gt_b200.ops.native`); on CPU the
same sums are formed with ``index_add_`` over edge chunks.  Replaces the reference's cuSPARSE path
(``gt3d/gt3d/dist/layers.py:53-64``); ``rows=`` restricts the product to a doubly-compressed row list and adds into an
existing buffer (``layers.py:132-146`` and the streamed layer's ``index_add_``).
"""
import torch

from ..attention.csr import BlockCSR

_CHUNK = 8_000_000


def _spmm_torch(ptr_rows, cols, w, x, n_out, out=None):
    out = torch.zeros(n_out, x.shape[1], dtype=x.dtype, device=x.device) if out is None else out
    e = cols.numel()
    for e0 in range(0, e, _CHUNK):
        e1 = min(e0 + _CHUNK, e)
        out.index_add_(0, ptr_rows[e0:e1], x[cols[e0:e1]] * w[e0:e1, None].to(x.dtype))
    return out


def spmm_raw(blk: BlockCSR, x: torch.Tensor, transpose: bool = False, out: torch.Tensor = None) -> torch.Tensor:
    """``A @ x`` (or ``A^T @ x``) without autograd; ``out`` (if given) is accumulated into."""
    if blk.weight is None:
        raise ValueError("aggregation block has no weights")
    if x.is_cuda:
        from . import native
        return native.spmm(blk, x, transpose, out)
    if not transpose:
        return _spmm_torch(blk.rows().long(), blk.col.long(), blk.weight, x, blk.n_rows, out)
    ccol, rowidx, _, _, w_t = blk.csc()
    cols_of = torch.repeat_interleave(torch.arange(blk.n_cols, device=x.device), (ccol[1:] - ccol[:-1]).long())
    return _spmm_torch(cols_of, rowidx.long(), w_t, x, blk.n_cols, out)


class _SpMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, blk):
        ctx.blk = blk
        return spmm_raw(blk, x.contiguous())

    @staticmethod
    def backward(ctx, dout):
        return spmm_raw(ctx.blk, dout.contiguous(), transpose=True), None


def spmm(blk: BlockCSR, x: torch.Tensor) -> torch.Tensor:
    """Differentiable ``A @ x``: ``x [n_cols, d] -> [n_rows, d]``."""
    return _SpMM.apply(x, blk)

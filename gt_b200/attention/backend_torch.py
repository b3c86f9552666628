"""CSR attention backend written with plain PyTorch ops (CPU or CUDA, any float dtype).

It is the plumbing / oracle backend: the distributed layers run on it under ``gloo`` on CPU, and the CUDA kernels
are checked against it.  Contract shared with :mod:`gt_b200.attention.backend_cuda` (and, semantically, with the
reference's ``attn_fwd_partial`` / ``attn_bwd_partial`` / ``attn_bwd`` / ``normalize``,
``gt3d/gt3d/attention/triton_kernel.py:544-602`` and ``backend_torch.py:76-211``):

``attn_fwd_partial(q, k, v, blk, gate, bias, score=, norm=, clamp=, scale=) -> (acc, l, m)``
    unnormalised block partials: ``acc[i] = sum_j p_ij v_j``, ``l[i] = sum_j p_ij`` with ``p_ij = exp(s_ij - m_i)``
    (``m`` = block row maximum for softmax, 0 for clamp-exp and for empty rows).
``attn_bwd_partial(q, k, v, blk, gate, bias, m, dacc, dl, ...) -> (dq, dk, dv, dgate, dbias)``
    gradient of the partials: ``ds_ij = p_ij (dacc_i . v_j + dl_i)`` (times the clamp mask), ``dv_j += p_ij dacc_i``.
``attn_bwd(q, k, v, blk, gate, bias, o, l, m, do, ...)``
    gradient of the normalised output given (possibly global) row statistics.
``normalize(acc, l, norm, eps)``

Edges are processed in chunks so that the peak temporary is ``O(chunk_edges * H * d)``; reductions over the edges
of a row use ``index_add_`` / ``scatter_reduce`` on the cached row index of every edge.
"""
import math

import torch

from .csr import BlockCSR

_CHUNK = 4_000_000


def _edge_chunks(num_edges, chunk_edges):
    step = num_edges if not chunk_edges or chunk_edges <= 0 else chunk_edges
    step = max(step, 1)
    return [(e0, min(e0 + step, num_edges)) for e0 in range(0, num_edges, step)]


def _score(qe, ke, et, gate, bias, score, scale):
    """scores [e, H] and the raw product q*k*scale (needed by the gate gradient)."""
    prod = qe * ke * scale
    if score == "dot":
        return prod.sum(-1), prod
    if score == "gated":
        return (prod * gate[et]).sum(-1), prod
    if score == "biased":
        return prod.sum(-1) + bias[et], prod
    raise ValueError(score)


def _prep(blk: BlockCSR, q, scale):
    rows = blk.rows().long()
    cols = blk.col.long()
    et = blk.etype.long() if blk.etype is not None else None
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    return rows, cols, et, scale


def attn_fwd_partial(q, k, v, blk: BlockCSR, gate=None, bias=None, *, score="dot", norm="softmax",
                     clamp=(-5.0, 5.0), scale=None, chunk_edges=_CHUNK):
    rows, cols, et, scale = _prep(blk, q, scale)
    n, h, d = q.shape
    acc = torch.zeros(n, h, d, dtype=q.dtype, device=q.device)
    l = torch.zeros(n, h, dtype=q.dtype, device=q.device)
    m = torch.zeros(n, h, dtype=q.dtype, device=q.device)
    chunks = _edge_chunks(blk.num_edges, chunk_edges)
    if norm == "softmax" and blk.num_edges:
        mx = torch.full((n, h), float("-inf"), dtype=q.dtype, device=q.device)
        for e0, e1 in chunks:
            r, c = rows[e0:e1], cols[e0:e1]
            s, _ = _score(q[r], k[c], et[e0:e1] if et is not None else None, gate, bias, score, scale)
            mx.scatter_reduce_(0, r[:, None].expand(-1, h), s, reduce="amax", include_self=True)
        m = torch.where(torch.isfinite(mx), mx, torch.zeros_like(mx))
    for e0, e1 in chunks:
        r, c = rows[e0:e1], cols[e0:e1]
        s, _ = _score(q[r], k[c], et[e0:e1] if et is not None else None, gate, bias, score, scale)
        p = torch.exp(s - m[r]) if norm == "softmax" else torch.exp(s.clamp(clamp[0], clamp[1]))
        l.index_add_(0, r, p)
        acc.index_add_(0, r, p.unsqueeze(-1) * v[c])
    return acc, l, m


def normalize(acc, l, norm, eps=1e-6, dtype=None):
    if norm == "softmax":
        o = acc / torch.where(l > 0, l, torch.ones_like(l)).unsqueeze(-1)
    else:
        o = acc / (l + eps).unsqueeze(-1)
    return o.to(dtype) if dtype is not None else o


def _bwd_core(q, k, v, blk, gate, bias, m, row_vec, row_bias, p_scale, *, score, norm, clamp, scale, chunk_edges):
    """Shared body of the two backward forms.

    With ``p_ij`` the unnormalised weight, ``P_ij = p_ij * p_scale_i``; ``ds_ij = P_ij (row_vec_i . v_j + row_bias_i)``
    (times the clamp mask) and ``dv_j += P_ij row_vec_i``.
    partial form : row_vec = dacc, row_bias = dl,  p_scale = 1
    normalised   : row_vec = dO,   row_bias = -D,  p_scale = 1 / l (or 1 / (l + eps))."""
    rows, cols, et, scale = _prep(blk, q, scale)
    adt = torch.float32 if q.dtype in (torch.float16, torch.bfloat16) else q.dtype
    dq = torch.zeros(q.shape, dtype=adt, device=q.device)
    dk = torch.zeros(k.shape, dtype=adt, device=k.device)
    dv = torch.zeros(v.shape, dtype=adt, device=v.device)
    dgate = torch.zeros(gate.shape, dtype=adt, device=q.device) if (score == "gated" and gate is not None) else None
    dbias = torch.zeros(bias.shape, dtype=adt, device=q.device) if (score == "biased" and bias is not None) else None
    for e0, e1 in _edge_chunks(blk.num_edges, chunk_edges):
        r, c = rows[e0:e1], cols[e0:e1]
        t = et[e0:e1] if et is not None else None
        qe, ke, ve = q[r], k[c], v[c]
        s, prod = _score(qe, ke, t, gate, bias, score, scale)
        if norm == "softmax":
            pw = torch.exp(s - m[r])
            mask = None
        else:
            pw = torch.exp(s.clamp(clamp[0], clamp[1]))
            mask = ((s >= clamp[0]) & (s <= clamp[1])).to(pw.dtype)
        if p_scale is not None:
            pw = pw * p_scale[r]
        ds = pw * ((row_vec[r] * ve).sum(-1) + row_bias[r])
        if mask is not None:
            ds = ds * mask
        dv.index_add_(0, c, (pw.unsqueeze(-1) * row_vec[r]).to(adt))
        dss = (ds * scale).unsqueeze(-1)
        if score == "gated":
            g = gate[t]
            dq.index_add_(0, r, (dss * ke * g).to(adt))
            dk.index_add_(0, c, (dss * qe * g).to(adt))
            dgate.index_add_(0, t, (ds.unsqueeze(-1) * prod).to(adt))
        else:
            dq.index_add_(0, r, (dss * ke).to(adt))
            dk.index_add_(0, c, (dss * qe).to(adt))
            if score == "biased":
                dbias.index_add_(0, t, ds.to(adt))
    return dq, dk, dv, dgate, dbias


def attn_bwd_partial(q, k, v, blk: BlockCSR, gate, bias, m, dacc, dl, *, score="dot", norm="softmax",
                     clamp=(-5.0, 5.0), scale=None, chunk_edges=_CHUNK):
    return _bwd_core(q, k, v, blk, gate, bias, m, dacc, dl, None, score=score, norm=norm, clamp=clamp, scale=scale,
                     chunk_edges=chunk_edges)


def attn_bwd(q, k, v, blk: BlockCSR, gate, bias, o, l, m, do, *, score="dot", norm="softmax", clamp=(-5.0, 5.0),
             eps=1e-6, scale=None, chunk_edges=_CHUNK):
    dd = (do * o).sum(-1)
    inv = 1.0 / torch.where(l > 0, l, torch.ones_like(l)) if norm == "softmax" else 1.0 / (l + eps)
    return _bwd_core(q, k, v, blk, gate, bias, m, do, -dd, inv, score=score, norm=norm, clamp=clamp, scale=scale,
                     chunk_edges=chunk_edges)


class _MaskedSparseAttentionTorch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gate, bias, blk, cfg):
        score, norm, clamp, eps, scale, chunk = cfg
        acc, l, m = attn_fwd_partial(q, k, v, blk, gate, bias, score=score, norm=norm, clamp=clamp, scale=scale,
                                     chunk_edges=chunk)
        o = normalize(acc, l, norm, eps)
        ctx.blk, ctx.cfg = blk, cfg
        ctx.save_for_backward(q, k, v, gate, bias, o, l, m)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, gate, bias, o, l, m = ctx.saved_tensors
        score, norm, clamp, eps, scale, chunk = ctx.cfg
        dq, dk, dv, dgate, dbias = attn_bwd(q, k, v, ctx.blk, gate, bias, o, l, m, do, score=score, norm=norm,
                                            clamp=clamp, eps=eps, scale=scale, chunk_edges=chunk)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype),
                dgate.to(gate.dtype) if dgate is not None else None,
                dbias.to(bias.dtype) if dbias is not None else None, None, None)


def masked_sparse_attention_torch(q, k, v, blk: BlockCSR, *, gate=None, bias=None, score="dot", norm="softmax",
                                  clamp=(-5.0, 5.0), eps=1e-6, scale=None, chunk_edges=_CHUNK):
    """Differentiable normalised attention over ``blk`` (q on the rows, k / v on the columns)."""
    if score in ("gated", "biased") and blk.etype is None:
        raise ValueError(f"score={score!r} needs edge types in the block")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    cfg = (score, norm, (float(clamp[0]), float(clamp[1])), float(eps), scale, chunk_edges)
    return _MaskedSparseAttentionTorch.apply(q, k, v, gate, bias, blk, cfg)

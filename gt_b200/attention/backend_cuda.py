"""Attention back-end on the hand-written sm_100a kernels (``csrc/attn.cu``).

Same contract as :mod:`gt_b200.attention.backend_torch`.  ``q / k / v`` are bf16 or fp32 ``[n, H, d]`` (fp32
accumulation inside), the partials ``(acc, l, m)`` are fp32.  A head dim that is not a power of two (2 x 40 of the
GraphGPS recipe) runs on the kernels with zero-padded heads.  Shapes the kernels do not tile even then (``H * d`` not
in {32, 64, 128, 256, 512}, more than 4 edge types) run on the torch-op backend on
the same device; that is a shape restriction, not a missing-extension fallback: if the extension is not built, every
call raises.

Extra entry points:
``attn_fwd_partial_accum``   compact-accumulate forward of the streamed layer: partials of the rows that own an edge
                             are added in place into the strided reduce-scatter payload (DCSR row list)
``attn_fwd_partial_pull``    forward that fetches K / V rows from the owners' symmetric buffers over NVLink
"""
import math
import os

import torch

from ..ops import native
from . import backend_torch as _bt
from . import tiles as _tiles
from .csr import BlockCSR

SEG_EDGES = 256
_SCORE = {"dot": 0, "gated": 1, "biased": 2}
_NORM = {"softmax": 0, "clampexp": 1}


def _supported(q, gate, bias):
    h, d = q.shape[1], q.shape[2]
    t = gate.shape[0] if gate is not None else (bias.shape[0] if bias is not None else 1)
    return q.dtype in (torch.bfloat16, torch.float32) and native.ext().attn_shape_supported(h, d, t)


def _padded_dim(q, gate, bias):
    """Head dims that are not a power of two (e.g. 2 x 40) run on the kernels with zero-padded heads: padded K columns add
    nothing to the scores and padded V columns produce zeros that are sliced away.  Returns the padded dim or None."""
    h, d = q.shape[1], q.shape[2]
    dp = max(8, 1 << (d - 1).bit_length())
    t = gate.shape[0] if gate is not None else (bias.shape[0] if bias is not None else 1)
    if dp != d and q.dtype in (torch.bfloat16, torch.float32) and native.ext().attn_shape_supported(h, dp, t):
        return dp
    return None


def _pad(t, dp):
    return torch.nn.functional.pad(t, (0, dp - t.shape[-1])) if t is not None else None


def _cfg(q, score, norm, clamp, scale):
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    return _SCORE[score], _NORM[norm], scale, float(clamp[0]), float(clamp[1])


def _plan_list(plan):
    return [plan.seg_row, plan.seg_beg, plan.seg_end, plan.seg_slot, plan.split_rows, plan.split_ptr]


def _tables(gate, bias, score):
    g = gate.float().contiguous().view(gate.shape[0], -1) if (score == "gated" and gate is not None) else None
    b = bias.float().contiguous() if (score == "biased" and bias is not None) else None
    return g, b


def _dcsr_plan(blk: BlockCSR, seg_edges):
    """Plan over the rows that own an edge, plus the map from plan row to block row."""
    key = ("dcsr_plan", seg_edges)
    if key not in blk._cache:
        rows = blk.dcsr_rows()
        crow = blk.crow.long()
        ptr = torch.stack([crow[rows.long()], crow[rows.long() + 1]], 1)
        # pointer array of the compressed rows: edges stay contiguous because the skipped rows are empty
        cptr = torch.cat([ptr[:, 0], crow[-1:]]) if rows.numel() else crow[:1]
        from .csr import SegmentPlan, _segments
        blk._cache[key] = (SegmentPlan(*_segments(cptr, seg_edges), seg_edges), rows)
        blk._cache[key][0].num_slots
    return blk._cache[key]


def attn_fwd_partial(q, k, v, blk: BlockCSR, gate=None, bias=None, *, score="dot", norm="softmax", clamp=(-5.0, 5.0),
                     scale=None, seg_edges=SEG_EDGES, k_peers=None, v_peers=None, rows_per_peer=0):
    if not _supported(q, gate, bias) and k is not None and _padded_dim(q, gate, bias):
        dp, d0 = _padded_dim(q, gate, bias), q.shape[-1]
        acc, l, m = attn_fwd_partial(_pad(q, dp), _pad(k, dp), _pad(v, dp), blk, _pad(gate, dp) if score == "gated" else gate, bias, score=score,
                                     norm=norm, clamp=clamp, scale=(1.0 / math.sqrt(d0) if scale is None else scale), seg_edges=seg_edges)
        return acc[..., :d0].contiguous(), l, m
    if not _supported(q, gate, bias):
        acc, l, m = _bt.attn_fwd_partial(q.float(), k.float(), v.float(), blk, gate.float() if gate is not None else None,
                                         bias.float() if bias is not None else None, score=score, norm=norm, clamp=clamp, scale=scale)
        return acc, l, m
    n, h, d = q.shape
    sc, nm, scale, lo, hi = _cfg(q, score, norm, clamp, scale)
    # density dispatch: dense 128 x 128 tiles of the mask go to the tensor-core kernel, everything else stays on the gathers
    tiles = _tile_plan_for(q, k, blk, bias, score, k_peers)
    if tiles is not None:
        blk = tiles.residual
    g, b = _tables(gate, bias, score)
    if tiles is not None and blk.num_edges == 0:
        acc = torch.zeros(n, h, d, dtype=torch.float32, device=q.device)
        l = torch.zeros(n, h, dtype=torch.float32, device=q.device)
        m = torch.zeros(n, h, dtype=torch.float32, device=q.device)
    else:
        plan = blk.row_plan(seg_edges)
        acc = torch.empty(n, h, d, dtype=torch.float32, device=q.device)
        l = torch.empty(n, h, dtype=torch.float32, device=q.device)
        m = torch.empty(n, h, dtype=torch.float32, device=q.device)
        scratch = torch.empty(plan.num_slots, (h * d + 2 * h + 3) // 4 * 4, dtype=torch.float32, device=q.device) if plan.num_slots else None
        native.ext().attn_fwd(q.contiguous(), k.contiguous() if k is not None else None, v.contiguous() if v is not None else None,
                              blk.col, blk.etype, g, b, _plan_list(plan), None, acc, l, m, scratch, h, d, sc, nm, scale, lo, hi,
                              h * d, h, False, k_peers, v_peers, int(rows_per_peer), 0, 0, [], 0, 0, 0)
    if tiles is not None:
        attn_tile_accumulate(q, k, v, tiles, b, acc, l, m, score=score, norm=norm, clamp=(lo, hi), scale=scale)
    return acc, l, m


def _tile_plan_for(q, k, blk, bias, score, k_peers=None):
    """The dense-tile split of ``blk`` when the tensor-core kernel can take it: bf16, heads of 32 in pairs, plain or biased
    dot-product scores, K / V in local memory."""
    if score == "gated" or k is None or k_peers is not None or q.dtype != torch.bfloat16:
        return None
    if q.shape[2] != 32 or q.shape[1] % 2 or (bias is not None and bias.shape[0] > _tiles.MAX_TYPES):
        return None
    return _tiles.tile_plan(blk)


def attn_tile_accumulate(q, k, v, tiles, bias, acc, l, m, *, score="dot", norm="softmax", clamp=(-5.0, 5.0), scale=None, debug_scores=None):
    """Merge the contribution of the dense tiles into the partial states ``(acc, l, m)`` in place (``csrc/attn_tile.cu``).
    ``debug_scores``: optional fp32 ``[2, 128, 128]`` that receives the raw ``Q K^T`` of the first tile of the first head pair."""
    n, h, d = q.shape
    sc, nm, scale, lo, hi = _cfg(q, score, norm, clamp, scale)
    b = bias.float().contiguous() if (score == "biased" and bias is not None) else None
    native.ext().attn_tile_fwd(q.contiguous(), k.contiguous(), v.contiguous(), tiles.rb_ids, tiles.rb_ptr, tiles.tile_cb, tiles.mask, b,
                               acc.view(n, h * d), l, m, h, sc, nm, scale, lo, hi, 0, 0, native.status(q.device), debug_scores)


def attn_fwd_partial_pull(q, k_peers, v_peers, rows_per_peer, blk, gate=None, bias=None, **kw):
    """Forward with K / V read from peer memory: ``k_peers`` / ``v_peers`` are int64 device tensors of buffer addresses."""
    return attn_fwd_partial(q, None, None, blk, gate, bias, k_peers=k_peers, v_peers=v_peers, rows_per_peer=rows_per_peer, **kw)


def attn_fwd_partial_accum(q, k, v, blk: BlockCSR, gate, bias, packed, hd, *, score="gated", norm="clampexp",
                           clamp=(-5.0, 5.0), scale=None, seg_edges=SEG_EDGES):
    """Add the block's clamp-exp partials into ``packed[:, :hd]`` (acc) and ``packed[:, hd:hd + H]`` (l) in place."""
    if norm != "clampexp":
        raise ValueError("in-place accumulation of partials is only valid for clamp-exp")
    if blk.num_edges == 0:
        return
    n, h, d = q.shape
    if not _supported(q, gate, bias) or packed.dtype != torch.float32:
        acc, l, _ = attn_fwd_partial(q, k, v, blk, gate, bias, score=score, norm=norm, clamp=clamp, scale=scale)
        packed[:, :hd] += acc.reshape(n, hd).to(packed.dtype)
        packed[:, hd:hd + h] += l.to(packed.dtype)
        return
    sc, nm, scale, lo, hi = _cfg(q, score, norm, clamp, scale)
    plan, rows = _dcsr_plan(blk, seg_edges)
    scratch = torch.empty(plan.num_slots, (h * d + 2 * h + 3) // 4 * 4, dtype=torch.float32, device=q.device) if plan.num_slots else None
    g, b = _tables(gate, bias, score)
    # q rows are addressed through the plan row; the kernel reads q[row] so hand it the compressed q
    qc = q.reshape(n, hd)[rows.long()].contiguous()
    stride = packed.stride(0)
    native.ext().attn_fwd(qc, k.contiguous(), v.contiguous(), blk.col, blk.etype, g, b, _plan_list(plan), rows,
                          packed, packed[:, hd:], None, scratch, h, d, sc, nm, scale, lo, hi, stride, stride, True, None, None, 0, 0, 0, [], 0, 0, 0)


def normalize(acc, l, norm, eps=1e-6, dtype=None):
    return _bt.normalize(acc, l, norm, eps, dtype)


def _pack_stat(m, row_bias, p_scale):
    z = torch.zeros_like(m)
    ps = p_scale if p_scale is not None else torch.ones_like(m)
    return torch.stack([m.float(), row_bias.float(), ps.float(), z.float()], dim=-1).contiguous()


# Score gradients handed from the column pass to the row pass (fp32 [E, H]): the row pass then gathers K only.  GT_ATTN_DS=0
# restores the independent passes; blocks whose buffer would exceed GT_ATTN_DS_MAX_MB (default 4096) keep them as well.
_DS_ON = os.environ.get("GT_ATTN_DS", "1") != "0"
_DS_MAX_BYTES = int(os.environ.get("GT_ATTN_DS_MAX_MB", "4096")) << 20


def ds_buffer(blk, h, dtype, device):
    """The hand-off buffer of a block, or ``None`` when the passes run independently."""
    if not _DS_ON or dtype != torch.bfloat16 or blk.num_edges == 0 or blk.num_edges * h * 4 > _DS_MAX_BYTES:
        return None
    return torch.empty(blk.num_edges, h, dtype=torch.float32, device=device)


def _bwd(q, k, v, blk, gate, bias, row_vec, stat, score, norm, clamp, scale, seg_edges, row_map=None, dq_accum=None, plan=None):
    """Both backward passes.  ``row_map`` / ``dq_accum`` / ``plan``: the compact-accumulate row pass (rows of the plan are
    ``row_map``; dq is added into the fp32 ``dq_accum``)."""
    n, h, d = q.shape
    nc = k.shape[0]
    e = native.ext()
    sc, nm, scale, lo, hi = _cfg(q, score, norm, clamp, scale)
    g, b = _tables(gate, bias, score)
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    rv = row_vec.to(q.dtype).contiguous()
    ds = ds_buffer(blk, h, q.dtype, q.device)
    # column pass over the transposed structure (first: it leaves the score gradients for the row pass)
    _, rowidx, et_t, pos, _ = blk.csc()
    cplan = blk.col_plan(seg_edges)
    dk, dv = torch.empty(nc, h, d, dtype=q.dtype, device=q.device), torch.empty(nc, h, d, dtype=q.dtype, device=q.device)
    cscratch = torch.empty(cplan.num_slots, 2 * h * d, dtype=torch.float32, device=q.device) if cplan.num_slots else None
    e.attn_bwd_col(q, k, v, rv, stat, rowidx, et_t, g, b, _plan_list(cplan), dk, dv, cscratch, h, d, sc, nm, scale, lo, hi, 0, 0, 0, 0,
                   ds, pos if ds is not None else None)
    # row pass
    plan = plan if plan is not None else blk.row_plan(seg_edges)
    nb = e.attn_bwd_row_blocks(plan.num_segments)
    dq = torch.empty_like(q) if dq_accum is None else dq_accum
    t = g.shape[0] if g is not None else (b.shape[0] if b is not None else 0)
    dgp = torch.empty(nb, t * h * d, dtype=torch.float32, device=q.device) if g is not None else None
    dbp = torch.empty(nb, t * h, dtype=torch.float32, device=q.device) if b is not None else None
    scratch = torch.empty(plan.num_slots, h * d, dtype=torch.float32, device=q.device) if plan.num_slots else None
    e.attn_bwd_row(q, k, v, rv, stat, blk.col, blk.etype, g, b, _plan_list(plan), row_map, dq, dq_accum is not None, dgp, dbp, nb, scratch,
                   h, d, sc, nm, scale, lo, hi, 0, 0, 0, 0, ds)
    dgate = dbias = None
    if g is not None:
        dgate = torch.empty(t * h * d, dtype=torch.float32, device=q.device)
        e.reduce_partials(dgp, dgate, False)
        dgate = dgate.view(t, h, d)
    if b is not None:
        dbias = torch.empty(t * h, dtype=torch.float32, device=q.device)
        e.reduce_partials(dbp, dbias, False)
        dbias = dbias.view(t, h)
    return dq, dk, dv, dgate, dbias


def attn_bwd_partial_accum(q, k, v, blk: BlockCSR, gate, bias, m, dacc, dl, dq_accum, *, score="gated", norm="clampexp",
                           clamp=(-5.0, 5.0), scale=None, seg_edges=SEG_EDGES):
    """Backward of one (hypersparse) sub-block whose query gradient is ADDED in place into ``dq_accum [rows, H d]`` (fp32):
    the row pass walks the doubly-compressed row list, so rows without an edge in this sub-block are neither read nor written
    and no ``[rows, H d]`` temporary + add exists per sub-block (the compact-accumulate backward of the reference,
    ``gt3d/gt3d/attention/triton_tiled.py:566-590``, used by its streamed layer ``gt3d/gt3d/models/exphormer_dist.py:892-893``).
    Returns ``(dk, dv, dgate, dbias)``."""
    n, h, d = q.shape
    if blk.num_edges == 0:
        z = torch.zeros(k.shape, dtype=k.dtype, device=k.device)
        return z, z.clone(), (torch.zeros_like(gate, dtype=torch.float32) if gate is not None else None), \
            (torch.zeros_like(bias, dtype=torch.float32) if bias is not None else None)
    if not _supported(q, gate, bias) or dq_accum.dtype != torch.float32 or not dq_accum.is_contiguous():
        dq, dk, dv, dgate, dbias = attn_bwd_partial(q, k, v, blk, gate, bias, m, dacc, dl, score=score, norm=norm, clamp=clamp, scale=scale,
                                                    seg_edges=seg_edges)
        dq_accum += dq.reshape(dq_accum.shape).to(dq_accum.dtype)
        return dk, dv, dgate, dbias
    plan, rows = _dcsr_plan(blk, seg_edges)
    _, dk, dv, dgate, dbias = _bwd(q, k, v, blk, gate, bias, dacc.reshape(q.shape), _pack_stat(m, dl, None), score, norm, clamp, scale, seg_edges,
                                   row_map=rows, dq_accum=dq_accum, plan=plan)
    return dk, dv, dgate, dbias


def attn_bwd_partial(q, k, v, blk: BlockCSR, gate, bias, m, dacc, dl, *, score="dot", norm="softmax", clamp=(-5.0, 5.0),
                     scale=None, seg_edges=SEG_EDGES):
    if not _supported(q, gate, bias) and _padded_dim(q, gate, bias):
        dp, d0 = _padded_dim(q, gate, bias), q.shape[-1]
        dq, dk, dv, dgate, dbias = attn_bwd_partial(_pad(q, dp), _pad(k, dp), _pad(v, dp), blk, _pad(gate, dp) if score == "gated" else gate, bias, m,
                                                    _pad(dacc.reshape(q.shape), dp), dl, score=score, norm=norm, clamp=clamp,
                                                    scale=(1.0 / math.sqrt(d0) if scale is None else scale), seg_edges=seg_edges)
        return (dq[..., :d0].contiguous(), dk[..., :d0].contiguous(), dv[..., :d0].contiguous(),
                dgate[..., :d0].contiguous() if dgate is not None else None, dbias)
    if not _supported(q, gate, bias):
        f = lambda t: t.float() if t is not None else None          # noqa: E731
        return _bt.attn_bwd_partial(f(q), f(k), f(v), blk, f(gate), f(bias), f(m), f(dacc), f(dl), score=score, norm=norm,
                                    clamp=clamp, scale=scale)
    stat = _pack_stat(m, dl, None)
    return _bwd(q, k, v, blk, gate, bias, dacc.reshape(q.shape), stat, score, norm, clamp, scale, seg_edges)


def attn_bwd(q, k, v, blk: BlockCSR, gate, bias, o, l, m, do, *, score="dot", norm="softmax", clamp=(-5.0, 5.0), eps=1e-6,
             scale=None, seg_edges=SEG_EDGES):
    if not _supported(q, gate, bias) and _padded_dim(q, gate, bias):
        dp, d0 = _padded_dim(q, gate, bias), q.shape[-1]
        dq, dk, dv, dgate, dbias = attn_bwd(_pad(q, dp), _pad(k, dp), _pad(v, dp), blk, _pad(gate, dp) if score == "gated" else gate, bias,
                                            _pad(o, dp), l, m, _pad(do.reshape(q.shape), dp), score=score, norm=norm, clamp=clamp, eps=eps,
                                            scale=(1.0 / math.sqrt(d0) if scale is None else scale), seg_edges=seg_edges)
        return (dq[..., :d0].contiguous(), dk[..., :d0].contiguous(), dv[..., :d0].contiguous(),
                dgate[..., :d0].contiguous() if dgate is not None else None, dbias)
    if not _supported(q, gate, bias):
        f = lambda t: t.float() if t is not None else None          # noqa: E731
        return _bt.attn_bwd(f(q), f(k), f(v), blk, f(gate), f(bias), f(o), f(l), f(m), f(do), score=score, norm=norm, clamp=clamp,
                            eps=eps, scale=scale)
    dd = (do.float() * o.float()).sum(-1)
    l = l.float()
    inv = 1.0 / torch.where(l > 0, l, torch.ones_like(l)) if norm == "softmax" else 1.0 / (l + eps)
    stat = _pack_stat(m, -dd, inv)
    return _bwd(q, k, v, blk, gate, bias, do.reshape(q.shape), stat, score, norm, clamp, scale, seg_edges)


class _MaskedSparseAttentionCuda(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, gate, bias, blk, cfg):
        score, norm, clamp, eps, scale = cfg
        acc, l, m = attn_fwd_partial(q, k, v, blk, gate, bias, score=score, norm=norm, clamp=clamp, scale=scale)
        o = normalize(acc, l, norm, eps).to(q.dtype)
        ctx.blk, ctx.cfg = blk, cfg
        ctx.save_for_backward(q, k, v, gate, bias, o, l, m)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, gate, bias, o, l, m = ctx.saved_tensors
        score, norm, clamp, eps, scale = ctx.cfg
        dq, dk, dv, dgate, dbias = attn_bwd(q, k, v, ctx.blk, gate, bias, o, l, m, do.contiguous(), score=score, norm=norm,
                                            clamp=clamp, eps=eps, scale=scale)
        return (dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype), dgate.to(gate.dtype) if dgate is not None else None,
                dbias.to(bias.dtype) if dbias is not None else None, None, None)


def masked_sparse_attention_cuda(q, k, v, blk: BlockCSR, *, gate=None, bias=None, score="dot", norm="softmax",
                                 clamp=(-5.0, 5.0), eps=1e-6, scale=None):
    """Differentiable normalised attention over ``blk`` on the native kernels."""
    if score in ("gated", "biased") and blk.etype is None:
        raise ValueError(f"score={score!r} needs edge types in the block")
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else float(scale)
    cfg = (score, norm, (float(clamp[0]), float(clamp[1])), float(eps), scale)
    return _MaskedSparseAttentionCuda.apply(q, k, v, gate, bias, blk.to(q.device), cfg)

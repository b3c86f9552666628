"""Algebraic specification of structure-masked sparse multi-head attention on an explicit edge list.

Every kernel and every distributed layer of the package is tested against this function (normally in fp64).
It is written for clarity: it materialises per-edge tensors ``[E, H]`` and ``[E, H, d]``.

Conventions (same contract as the reference's ``gt3d/gt3d/attention/ref.py:49-108``)
-----------------------------------------------------------------------------------
* ``q, k, v``: ``[N, H, d]``.
* ``edge_index``: ``[2, E]``; row 0 is the source ``j`` (key / value side), row 1 the destination ``i`` (query
  side).  Attention is normalised over the in-edges of every destination.
* ``edge_type``: optional ``[E]`` integer tensor selecting a row of ``gate`` (``[T, H, d]``) or ``bias`` (``[T, H]``).

Score modes
    ``dot``     s_ij = scale <q_i, k_j>
    ``gated``   s_ij = scale sum_f q_if k_jf gate[t_ij, f]          (Exphormer)
    ``biased``  s_ij = scale <q_i, k_j> + bias[t_ij]                (Graphormer spatial bias)
Normalisations
    ``softmax``   exact softmax over the in-edges; rows without in-edges give 0
    ``clampexp``  p_ij = exp(clamp(s_ij, lo, hi)), o_i = sum_j p_ij v_j / (sum_j p_ij + eps)
"""
import math

import torch

SCORES = ("dot", "gated", "biased")
NORMS = ("softmax", "clampexp")


def segment_sum(src: torch.Tensor, index: torch.Tensor, num_segments: int) -> torch.Tensor:
    """``out[s] = sum_{e: index[e] == s} src[e]`` (trailing dimensions kept)."""
    out = torch.zeros((num_segments,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    return out.index_add_(0, index, src)


def segment_max(src: torch.Tensor, index: torch.Tensor, num_segments: int) -> torch.Tensor:
    """``out[s] = max_{e: index[e] == s} src[e]``; ``-inf`` for empty segments."""
    out = torch.full((num_segments,) + tuple(src.shape[1:]), float("-inf"), dtype=src.dtype, device=src.device)
    idx = index.reshape((-1,) + (1,) * (src.dim() - 1)).expand_as(src)
    return out.scatter_reduce(0, idx, src, reduce="amax", include_self=True)


def edge_scores(q, k, src, dst, edge_type, gate, bias, score, scale):
    """Per-edge scores ``[E, H]`` of the three score modes."""
    qk = q[dst] * k[src]
    if score == "dot":
        return qk.sum(-1) * scale
    if score == "gated":
        if gate is None or edge_type is None:
            raise ValueError("score='gated' needs gate and edge_type")
        return (qk * gate[edge_type]).sum(-1) * scale
    if score == "biased":
        if bias is None or edge_type is None:
            raise ValueError("score='biased' needs bias and edge_type")
        return qk.sum(-1) * scale + bias[edge_type]
    raise ValueError(f"unknown score mode {score!r}")


def edge_weights(s, dst, n, norm, clamp, eps):
    """Unnormalised attention weight of every edge, ``(p [E, H], m, floor)``: for ``softmax`` ``p = exp(s - m[dst])`` with
    the row maximum ``m`` (0 for rows without in-edges) and nothing added to the normaliser; for ``clampexp``
    ``p = exp(clamp(s))``, no maximum, and ``eps`` added to the normaliser."""
    if norm == "softmax":
        m = segment_max(s, dst, n)
        m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))
        return torch.exp(s - m[dst]), m, 0.0
    if norm == "clampexp":
        return torch.exp(s.clamp(clamp[0], clamp[1])), None, eps
    raise ValueError(f"unknown norm mode {norm!r}")


def masked_sparse_attention_ref(q, k, v, edge_index, *, edge_type=None, gate=None, bias=None, score="dot",
                                norm="softmax", clamp=(-5.0, 5.0), eps=1e-6, scale=None, return_stats=False):
    """Masked sparse attention on an edge list; returns ``o [N, H, d]``.

    With ``return_stats=True`` also returns ``(z, m)``: the per-row normaliser ``[N, H]`` and, for softmax, the row
    maximum (0 for empty rows); ``m`` is ``None`` for clamp-exp.
    """
    if not (q.dim() == 3 and k.dim() == 3 and v.shape == k.shape and q.shape[1:] == k.shape[1:]):
        raise ValueError("q [Nq,H,d], k/v [Nk,H,d] expected")
    n = q.shape[0]
    src, dst = edge_index[0].long(), edge_index[1].long()
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    et = edge_type.long() if edge_type is not None else None
    s = edge_scores(q, k, src, dst, et, gate, bias, score, scale)
    p, m, floor = edge_weights(s, dst, n, norm, clamp, eps)
    z = segment_sum(p, dst, n)
    o = segment_sum(p.unsqueeze(-1) * v[src], dst, n) / (z + floor).clamp_min(torch.finfo(z.dtype).tiny).unsqueeze(-1)
    return (o, (z, m)) if return_stats else o

"""Ring attention with rotating K/V (Ring Attention as published), uni- and bidirectional, attention only.

(P, 1) grid; rank ``r`` owns chunk ``r`` and projects its K, V once.  The packed ``[K | V]`` chunk (``[2, chunk, H d]``
in the wire dtype) hops around the ring; at step ``s`` the rank runs the block kernel on the sub-block of its rows whose
sources live in the visiting chunk.  The clamp-exp partials add up; ``o = acc / (l + eps)`` is formed by the module so
the backward receives ``(dacc, dl)``.  In backward K/V travel again and a ``[dK | dV]`` accumulator travels with every
chunk.  ``bidir=True`` splits every chunk in two halves that travel in opposite directions (both directions of every
NVLink are used in each hop) and runs one kernel per step on the two visiting halves.
Algorithm of ``gt3d/gt3d/dist/ring_kv.py:54-386``.
"""
import torch
import torch.distributed as dist

from .attention import AttentionBlock, split_block_by_source_chunk
from .grid import group_size
from .ring import RingComm, rotate_backward, rotate_forward


def split_block_bidir(edge_index_local, p, chunk, rank, h_a, etype=None):
    """Step sub-blocks of the bidirectional ring of ``rank``: an edge whose source is row ``loc`` of chunk ``c`` belongs
    to step ``(rank - c) mod p`` if ``loc < h_a`` (half A, clockwise) else ``(c - rank) mod p`` (half B); sources are
    renumbered to ``loc``, the row's position in the step's concatenated buffer."""
    src, dst = edge_index_local[0], edge_index_local[1]
    c, loc = src // chunk, src % chunk
    step_of = torch.where(loc < h_a, (rank - c) % p, (c - rank) % p)
    return [(torch.stack([loc[step_of == s], dst[step_of == s]]), etype[step_of == s] if etype is not None else None)
            for s in range(p)]


class _RingAttnKV(torch.autograd.Function):
    @staticmethod
    def _payloads(k, v, mod, wire):
        n = k.shape[0]
        kv = torch.stack([k.reshape(n, -1), v.reshape(n, -1)]).to(wire)
        if not mod.bidir:
            return [kv.contiguous()], [+1]
        return [kv[:, :mod.h_a].contiguous(), kv[:, mod.h_a:].contiguous()], [+1, -1]

    @staticmethod
    def _visiting(bufs, mod, kdt):
        kv = bufs[0] if len(bufs) == 1 else torch.cat(bufs, dim=1)
        return kv if kv.dtype == kdt else kv.to(kdt)

    @staticmethod
    def forward(ctx, q, k, v, gate, mod):
        from ..attention import get_backend
        be = get_backend(mod.backend)
        ring, h, d = mod.ring, mod.h, mod.d
        n = q.shape[0]
        wire = mod.comm_dtype or q.dtype
        kdt = q.dtype if mod.backend == "torch" else wire
        pdt = torch.float64 if q.dtype == torch.float64 else torch.float32
        gate_c = gate.to(q.dtype if mod.backend == "torch" else torch.float32) if gate is not None else None
        with torch.no_grad():
            acc = torch.zeros(n, h, d, dtype=pdt, device=q.device)
            l = torch.zeros(n, h, dtype=pdt, device=q.device)
            payloads, dirs = _RingAttnKV._payloads(k, v, mod, wire)

            def step(s, bufs):
                blk = mod.attns[s if mod.bidir else (ring.rank - s) % ring.size].csr
                if not blk.num_edges:
                    return
                kv = _RingAttnKV._visiting(bufs, mod, kdt)
                a, ll, _ = be.attn_fwd_partial(q, kv[0].view(n, h, d), kv[1].view(n, h, d), blk, gate_c, None, score=mod.score,
                                               norm=mod.norm, clamp=mod.clamp, scale=mod.scale)
                acc.add_(a.to(pdt))
                l.add_(ll.to(pdt))

            rotate_forward(ring, payloads, dirs, step, mod.no_comm, "ring_kv fwd")
        ctx.mod, ctx.pdt = mod, pdt
        ctx.gate_dtype = gate.dtype if gate is not None else None
        ctx.save_for_backward(q, k, v, gate_c)
        return acc, l

    @staticmethod
    def backward(ctx, dacc, dl):
        from ..attention import get_backend
        q, k, v, gate_c = ctx.saved_tensors
        mod, pdt = ctx.mod, ctx.pdt
        be = get_backend(mod.backend)
        ring, h, d = mod.ring, mod.h, mod.d
        n, hd = q.shape[0], h * d
        wire = mod.comm_dtype or q.dtype
        kdt = q.dtype if mod.backend == "torch" else wire
        with torch.no_grad():
            dacc, dl = dacc.contiguous().to(pdt), dl.contiguous().to(pdt)
            m0 = torch.zeros_like(dl)
            dq = torch.zeros(n, h, d, dtype=pdt, device=q.device)
            state = {"dgate": None}
            payloads, dirs = _RingAttnKV._payloads(k, v, mod, wire)
            sizes = [p.shape[1] for p in payloads]

            def step(s, bufs):
                blk = mod.attns[s if mod.bidir else (ring.rank - s) % ring.size].csr
                if not blk.num_edges:
                    return [torch.zeros(2, sz, hd, dtype=pdt, device=q.device) for sz in sizes]
                kv = _RingAttnKV._visiting(bufs, mod, kdt)
                dq_s, dk_s, dv_s, dg_s, _ = be.attn_bwd_partial(q, kv[0].view(n, h, d), kv[1].view(n, h, d), blk, gate_c, None,
                                                                m0, dacc, dl, score=mod.score, norm=mod.norm, clamp=mod.clamp,
                                                                scale=mod.scale)
                dq.add_(dq_s.to(pdt))
                if dg_s is not None:
                    state["dgate"] = dg_s if state["dgate"] is None else state["dgate"] + dg_s
                dkv = torch.stack([dk_s.reshape(n, hd), dv_s.reshape(n, hd)]).to(pdt)
                return [dkv] if len(sizes) == 1 else [dkv[:, :sizes[0]].contiguous(), dkv[:, sizes[0]:].contiguous()]

            tot = rotate_backward(ring, payloads, dirs, step, wire, mod.no_comm, "ring_kv bwd")
            dkv = tot[0] if len(tot) == 1 else torch.cat(tot, dim=1)
        dgate = state["dgate"]
        return (dq.to(q.dtype), dkv[0].reshape(n, h, d).to(k.dtype), dkv[1].reshape(n, h, d).to(v.dtype),
                dgate.to(ctx.gate_dtype) if dgate is not None and ctx.gate_dtype is not None else None, None)


class DistRingAttentionKV(torch.nn.Module):
    """``q, k, v``: owned chunk with all heads ``[chunk, H, d]``; returns the owned chunk of ``o``.  ``blocks``: the
    ``P`` sub-blocks of the local block (per source chunk, or per step for ``bidir``); ``from_block`` splits a whole
    local block.  ``no_comm`` skips the hops (compute-only timing, wrong result)."""

    def __init__(self, grid, blocks, num_heads, head_dim, backend="cuda", score="gated", norm="clampexp",
                 clamp=(-5.0, 5.0), eps=1e-6, comm_dtype=None, no_comm=False, bidir=False):
        super().__init__()
        if grid.p_cols != 1:
            raise ValueError("ring attention is a 1D row partition: use a (P, 1) grid")
        if norm != "clampexp":
            raise ValueError("sub-block partials add without rescaling only for clamp-exp")
        self.grid, self.h, self.d = grid, num_heads, head_dim
        self.backend, self.score, self.norm, self.clamp, self.eps = backend, score, norm, tuple(clamp), eps
        self.scale = 1.0 / (head_dim ** 0.5)
        self.comm_dtype, self.no_comm, self.bidir = comm_dtype, no_comm, bidir
        self.h_a = grid.chunk // 2
        self.ring = RingComm(grid.col_group)
        self.attns = [b if isinstance(b, AttentionBlock) else AttentionBlock(grid, b[0], b[1], n_cols=grid.chunk) for b in blocks]
        if len(self.attns) != self.ring.size:
            raise ValueError("one sub-block per ring step is required")

    @classmethod
    def from_block(cls, grid, block_edge_index, block_edge_type, num_heads, head_dim, bidir=False, **kw):
        if bidir:
            rank = dist.get_rank(grid.col_group) if group_size(grid.col_group) > 1 else 0
            parts = split_block_bidir(block_edge_index, grid.p_rows, grid.chunk, rank, grid.chunk // 2, block_edge_type)
            return cls(grid, parts, num_heads, head_dim, bidir=True, **kw)
        parts = split_block_by_source_chunk(block_edge_index, grid.p_rows, grid.chunk, block_edge_type)
        return cls(grid, [(ei, et) for ei, et, _ in parts], num_heads, head_dim, **kw)

    def to(self, device):
        for a in self.attns:
            a.to(device)
        return super().to(device)

    def forward(self, q_loc, k_loc, v_loc, gate=None):
        acc, l = _RingAttnKV.apply(q_loc.contiguous(), k_loc.contiguous(), v_loc.contiguous(), gate, self)
        return (acc / (l + self.eps).unsqueeze(-1)).to(q_loc.dtype)

"""Ring attention baselines on a (P, 1) grid (pure row partition): payload chunks rotate around the ring of ranks
with NCCL point-to-point transfers that overlap the per-step kernels.

``RingComm``            neighbours of a group and batched ``isend`` / ``irecv`` hops
``rotate_forward``      the forward schedule: at step ``s`` the rank holds the payload of chunk ``(rank -/+ s) mod P``
``rotate_backward``     the backward schedule: payloads rotate again and, with them, one gradient accumulator per
                        payload to which every rank adds its contribution; after ``P`` hops it is back at the owner
``DistExphormerLayerRing``  Exphormer layer where the *layer input* x rotates; K, V and the GCN message of the visiting
                        chunk are re-projected at every hop and recomputed in backward (memory ``O(N / P)``)

The schedules serve both this x-rotating layer and the K/V-rotating operator of :mod:`gt_b200.parallel.ring_kv`
(uni- and bidirectional).  Only clamp-exp attention is valid here: its partials add without rescaling.  The
algorithms are those of ``gt3d/gt3d/dist/ring.py:41-265``; per the build target these baselines stay on NCCL P2P.
"""
import torch
import torch.distributed as dist

from ..ops import functional as K
from ..ops.sparse import spmm_raw
from ..utils.timers import timers
from .grid import group_size


class RingComm:
    """Ring over the ranks of ``group`` in group-rank order."""

    def __init__(self, group):
        self.group = group
        self.size = group_size(group)
        self.rank = dist.get_rank(group) if self.size > 1 else 0
        if self.size > 1:
            self.next = dist.get_global_rank(group, (self.rank + 1) % self.size) if group is not None else (self.rank + 1) % self.size
            self.prev = dist.get_global_rank(group, (self.rank - 1) % self.size) if group is not None else (self.rank - 1) % self.size
        else:
            self.next = self.prev = 0

    def hop(self, moves):
        """``moves``: list of ``(send_buf, recv_buf, direction)``, direction +1 = to next / from prev, -1 = the reverse.
        All transfers of a step are posted as one batch (same order on every rank).  Returns the work handles."""
        ops = []
        for send, recv, direction in moves:
            to, frm = (self.next, self.prev) if direction > 0 else (self.prev, self.next)
            ops.append(dist.P2POp(dist.isend, send, to, group=self.group))
            ops.append(dist.P2POp(dist.irecv, recv, frm, group=self.group))
        return dist.batch_isend_irecv(ops)

    @staticmethod
    def wait(works):
        for w in works:
            w.wait()


def rotate_forward(ring, payloads, directions, step, no_comm=False, tag="ring fwd"):
    """Run ``step(s, bufs)`` for ``s = 0..P-1`` where ``bufs[i]`` is payload ``i`` after ``s`` hops in direction
    ``directions[i]``.  The hop to step ``s + 1`` is posted before ``step(s)`` and awaited after it."""
    p = ring.size
    bufs = [b.clone(memory_format=torch.contiguous_format) for b in payloads]      # hops overwrite the buffers
    spare = [torch.empty_like(b) for b in bufs] if p > 1 else None
    t = timers()
    for s in range(p):
        works = None
        if s < p - 1 and not no_comm:
            works = ring.hop([(b, n, d) for b, n, d in zip(bufs, spare, directions)])
        t.start(f"{tag}: compute")
        step(s, bufs)
        t.stop(f"{tag}: compute")
        if works is not None:
            t.start(f"{tag}: wait")
            ring.wait(works)
            t.stop(f"{tag}: wait")
            bufs, spare = spare, bufs


def rotate_backward(ring, payloads, directions, step, wire_dtype, no_comm=False, tag="ring bwd"):
    """Backward schedule.  ``step(s, bufs)`` returns one contribution per payload (gradient w.r.t. the visiting chunk's
    payload, any float dtype).  Every contribution is added to the accumulator that arrived with the chunk and sent on;
    after the last step the accumulators of the rank's own payloads are returned (in ``wire_dtype``)."""
    p = ring.size
    bufs = [b.clone(memory_format=torch.contiguous_format) for b in payloads]      # hops overwrite the buffers
    spare = [torch.empty_like(b) for b in bufs] if p > 1 else None
    acc_in, works_acc, totals = None, None, None
    t = timers()
    for s in range(p):
        works = None
        if s < p - 1 and not no_comm:
            works = ring.hop([(b, n, d) for b, n, d in zip(bufs, spare, directions)])
        t.start(f"{tag}: compute")
        contrib = step(s, bufs)
        t.stop(f"{tag}: compute")
        if p == 1 or no_comm:
            totals = contrib if totals is None else [a + b for a, b in zip(totals, contrib)]
            continue
        if s > 0:
            t.start(f"{tag}: wait grad")
            ring.wait(works_acc)
            t.stop(f"{tag}: wait grad")
            contrib = [c + a.to(c.dtype) for c, a in zip(contrib, acc_in)]
        send = [c.to(wire_dtype).contiguous() for c in contrib]
        acc_in = [torch.empty_like(x) for x in send]
        works_acc = ring.hop([(x, y, d) for x, y, d in zip(send, acc_in, directions)])
        if works is not None:
            t.start(f"{tag}: wait")
            ring.wait(works)
            t.stop(f"{tag}: wait")
            bufs, spare = spare, bufs
    if p > 1 and not no_comm:
        ring.wait(works_acc)
        return acc_in
    return [x.to(wire_dtype) for x in totals]


class _RingAttnGCN(torch.autograd.Function):
    """Owned rows of the payload ``[acc | l | gcn partial]`` summed over the ``P`` ring steps; saves the owned input."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv, wg, gate, layer):
        from ..attention import get_backend
        L, ring = layer, layer.ring
        be = get_backend(L.backend)
        h, d = L.num_heads, L.d_head
        hd = h * d
        wire = L.comm_dtype or x.dtype
        gate_c = gate.to(x.dtype if L.backend == "torch" else torch.float32)
        with_gcn = L.with_gcn and wg is not None
        pdt = torch.float64 if x.dtype == torch.float64 else torch.float32
        with torch.no_grad():
            n, dim = x.shape
            q = K.linear_nograd(x, wq).view(n, h, d)
            packed = torch.zeros(n, hd + h + (dim if with_gcn else 0), dtype=pdt, device=x.device)

            def step(s, bufs):
                c = (ring.rank - s) % ring.size
                xs = bufs[0].to(x.dtype)
                blk = L.attns[c].block.csr
                if with_gcn and L.gcn_blocks[c].csr64.num_edges:
                    msg = K.linear_nograd(xs, wg)
                    packed[:, hd + h:] += spmm_raw(L.gcn_blocks[c].matrix(msg.dtype, msg.device), msg).to(pdt)
                if blk.num_edges:
                    ks, vs = K.linear_nograd(xs, wk).view(-1, h, d), K.linear_nograd(xs, wv).view(-1, h, d)
                    acc_s, l_s, _ = be.attn_fwd_partial(q, ks, vs, blk, gate_c, None, score="gated", norm="clampexp",
                                                        clamp=L.attn_clamp, scale=L.attn_scale)
                    packed[:, :hd] += acc_s.reshape(n, hd).to(pdt)
                    packed[:, hd:hd + h] += l_s.to(pdt)

            rotate_forward(ring, [x.detach().to(wire)], [+1], step, L.no_comm, "ring fwd")
        ctx.save_for_backward(x, wq, wk, wv, wg if with_gcn else None, gate)
        ctx.layer, ctx.with_gcn, ctx.gate_c_dtype, ctx.pdt = L, with_gcn, gate_c.dtype, pdt
        return packed

    @staticmethod
    def backward(ctx, dpo):
        from ..attention import get_backend
        x, wq, wk, wv, wg, gate = ctx.saved_tensors
        L, ring = ctx.layer, ctx.layer.ring
        be = get_backend(L.backend)
        h, d = L.num_heads, L.d_head
        hd = h * d
        wire = L.comm_dtype or x.dtype
        pdt, with_gcn = ctx.pdt, ctx.with_gcn
        gate_c = gate.to(ctx.gate_c_dtype)
        with torch.no_grad():
            n, dim = x.shape
            dpo = dpo.contiguous()
            dacc = dpo[:, :hd].contiguous().to(pdt).view(n, h, d)
            dl = dpo[:, hd:hd + h].contiguous().to(pdt)
            dagg = dpo[:, hd + h:].contiguous().to(x.dtype) if with_gcn else None
            q = K.linear_nograd(x, wq).view(n, h, d)
            m0 = torch.zeros_like(dl)
            dq = torch.zeros(n, h, d, dtype=pdt, device=x.device)
            dwk, dwv = torch.zeros_like(wk), torch.zeros_like(wv)
            dwg = torch.zeros_like(wg) if with_gcn else None
            state = {"dgate": None}

            def step(s, bufs):
                c = (ring.rank - s) % ring.size
                xs = bufs[0].to(x.dtype)
                blk = L.attns[c].block.csr
                dxs = torch.zeros(xs.shape[0], dim, dtype=x.dtype, device=x.device)
                if with_gcn and L.gcn_blocks[c].csr64.num_edges:
                    dp_s = spmm_raw(L.gcn_blocks[c].matrix(dagg.dtype, dagg.device), dagg, transpose=True)
                    dwg.add_(K.matmul_tn(dp_s, xs).to(dwg.dtype))
                    dxs += K.matmul_nn(dp_s, wg)
                if blk.num_edges:
                    ks, vs = K.linear_nograd(xs, wk).view(-1, h, d), K.linear_nograd(xs, wv).view(-1, h, d)
                    dq_s, dks, dvs, dgate_s, _ = be.attn_bwd_partial(q, ks, vs, blk, gate_c, None, m0, dacc, dl, score="gated",
                                                                     norm="clampexp", clamp=L.attn_clamp, scale=L.attn_scale)
                    dq.add_(dq_s.to(pdt))
                    if dgate_s is not None:
                        state["dgate"] = dgate_s if state["dgate"] is None else state["dgate"] + dgate_s
                    dks, dvs = dks.to(x.dtype).view(-1, hd), dvs.to(x.dtype).view(-1, hd)
                    dwk.add_(K.matmul_tn(dks, xs).to(dwk.dtype))
                    dwv.add_(K.matmul_tn(dvs, xs).to(dwv.dtype))
                    dxs += K.matmul_nn(dks, wk)
                    dxs += K.matmul_nn(dvs, wv)
                return [dxs]

            dx = rotate_backward(ring, [x.detach().to(wire)], [+1], step, wire, L.no_comm, "ring bwd")[0].to(x.dtype)
            dq2 = dq.view(n, hd).to(x.dtype)
            dwq = K.matmul_tn(dq2, x).to(wq.dtype)
            dx = dx + K.matmul_nn(dq2, wq)
        dgate = state["dgate"]
        return dx, dwq, dwk, dwv, dwg, (dgate.to(gate.dtype) if dgate is not None else None), None


def _streamed_base():
    from ..models.exphormer_dist import DistExphormerLayerStreamed
    return DistExphormerLayerStreamed


class DistExphormerLayerRing(torch.nn.Module):
    """Exphormer layer on a (P, 1) grid with x-rotating ring attention.  Parameters and the owned-row tail are those of
    the streamed layer (the class is assembled lazily to avoid an import cycle with the models package)."""

    def __new__(cls, *args, **kwargs):
        return _make_ring_layer(*args, **kwargs)


_RING_CLASS = []


def _make_ring_layer(grid, gcn_blocks, attn_blocks, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                     comm_dtype=None, tail_checkpoint=False, with_gcn=True, norm="bn"):
    if not _RING_CLASS:
        base = _streamed_base()

        class _DistExphormerLayerRing(base):
            self_checkpointing = True

            def __init__(self, grid, gcn_blocks, attn_blocks, *a, **kw):
                if grid.p_cols != 1:
                    raise ValueError("ring attention is a 1D row partition: use a (P, 1) grid")
                super().__init__(grid, gcn_blocks, attn_blocks, *a, **kw)
                self.ring = RingComm(grid.col_group)
                self.no_comm = False
                if not (self.ring.size == grid.p_rows == len(attn_blocks)):
                    raise ValueError("one sub-block per ring step is required")

            def forward(self, x, edge_type_emb):
                gate = self.gate(edge_type_emb)
                wg = self.gcn.lin.weight if self.with_gcn else None
                packed_o = _RingAttnGCN.apply(x, self.q.weight, self.k.weight, self.v.weight, wg, gate, self)
                if self.tail_checkpoint and self.training:
                    return torch.utils.checkpoint.checkpoint(self._tail, x, packed_o, use_reentrant=False)
                return self._tail(x, packed_o)

        _DistExphormerLayerRing.__name__ = "DistExphormerLayerRing"
        _RING_CLASS.append(_DistExphormerLayerRing)
    return _RING_CLASS[0](grid, gcn_blocks, attn_blocks, dim_h, num_heads, dropout, bn_eps, bn_momentum, backend,
                          comm_dtype=comm_dtype, rs_dtype=None, tail_checkpoint=tail_checkpoint, with_gcn=with_gcn, norm=norm)

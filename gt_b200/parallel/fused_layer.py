"""The attention + aggregation branch of the fused 2D layer as ONE explicit-backward operator on the native kernels.

``fused_branch(layer, x, gate)`` maps the owned rows ``x [O, d]`` (bf16) to the owned rows of the reduce-scattered
payload ``(acc [O, H d_h] fp32, l [O, H] fp32, agg [O, d] bf16)`` -- what the reference's fused layer obtains with two
all-gathers of x, three projections, the attention kernel, the SpMM and one reduce-scatter of ``[acc | l | gcn_agg]``
(``gt3d/gt3d/models/exphormer_dist.py:433-453``, backward mirror ``gt3d/gt3d/dist/grid2d.py:247-268``).  Differences in
mechanism:

* K | V | message | Q are column slices of one GEMM output (the kernels take row strides), their gradients are column slices
  of one buffer that feeds ONE weight-gradient GEMM and ONE input-gradient GEMM: no split / concatenate / cast copies, and the
  weight gradients are added into the training engine's flat gradient buffer by the GEMM itself.
* On a multi-rank grid every collective is part of a compute kernel, ordered by epoch channels instead of barriers
  (``signal`` after the producer, bounded wait inside the consumer):

  ==========================  ==============================================================================================
  all-gather x -> projections  the GEMM's TMA producer reads the owners' rows from peer memory (``gemm_nt_gather``), waiting
                               per peer for that peer's "x published" epoch
  reduce-scatter of partials   the attention forward and the SpMM store every finished ``[acc | l]`` / ``agg`` row as bf16
                               straight into the slot the row's OWNER keeps for this rank; the owner sums its slots
                               (``sum_payload``) after the row group has signalled
  all-gather of (dacc,dl,dagg) owners publish one packed bf16 gradient row block; ``pull_unpack`` reads the row block from the
                               owners' memory and writes the row vector / statistics / dagg the backward kernels consume
  reduce-scatter of dx         ``gemm_nt_scatter`` stores finished tiles into the owner's slots; ``sum_slots_wait`` adds them
  ==========================  ==============================================================================================

  Buffers alternate between two copies per kind (``GroupContext.staging``): every use is "all members signal, all members wait",
  so when a copy comes up again two uses later every reader has passed the wait of the use in between, which it can only do
  after finishing with that copy (single stream per rank).

Falls back (returns None from ``fused_branch``) for CPU tensors, fp32 activations, the NCCL transport on multi-rank grids,
sparse-communication plans and shapes outside the kernels' limits; the caller then runs the op-by-op path.
"""
import torch

from ..attention.backend_cuda import SEG_EDGES, _plan_list
from ..ops import native
from .collectives import _HEAP
from .grid import group_size


class Channel:
    """Epoch channel of a group: ``flags int32[8]`` at the same heap offset on every member plus a device-resident counter."""

    def __init__(self, heap, ctx):
        self.ctx = ctx
        self.off = heap.alloc(32, 256)
        self.flags = heap.view(self.off, (8,), torch.int32)
        self.counter = torch.zeros(1, dtype=torch.int32, device=heap.device)
        self.ptrs = [heap.peer_base[r] + self.off for r in ctx.ranks]

    def signal(self):
        native.ext().channel_signal(self.ptrs, self.ctx.me, self.counter)


def _round8(n):
    return -(-n // 8) * 8


def branch_supported(layer, x):
    g = layer.grid
    h, dh, d = layer.num_heads, layer.d_head, layer.dim_h
    on_device = x.is_cuda or (_HEAP[0] is not None and _HEAP[0].host)      # host: the emulated transport between CPU ranks (tests)
    if not (on_device and x.dtype == torch.bfloat16 and layer.kernel_dtype in (None, torch.bfloat16)):
        return False
    if getattr(layer, "sp_row", None) is not None or getattr(layer, "sp_col", None) is not None or layer.gather_proj:
        return False
    if getattr(g, "p_heads", 1) > 1 or h * dh != d or d % 8 or d > 512 or (h * dh // 8) > 32:
        return False
    if not native.ext().attn_shape_supported(h, dh, 3):
        return False
    multi = group_size(g.row_group) > 1 or group_size(g.col_group) > 1
    if multi and (_HEAP[0] is None or group_size(g.row_group) > 8 or group_size(g.col_group) > 8
                  or not (_HEAP[0].group_is_local(g.row_group) and _HEAP[0].group_is_local(g.col_group))):
        return False
    if x.shape[0] % 8:
        return False
    return True


def _stack(layer):
    """``(W [rows, d] bf16, grad [rows, d] fp32 or None)``: rows K | V | (message) | Q.  With the training engine these are views
    of its flat buffers; otherwise the stack is built with a concatenation."""
    st = getattr(layer, "_w_stack", None)
    if st is not None:
        return st
    ws = [layer.k.weight, layer.v.weight] + ([layer.gcn.lin.weight] if layer.with_gcn else []) + [layer.q.weight]
    return torch.cat([w.detach() for w in ws], dim=0).to(torch.bfloat16).contiguous(), None


class _Comm:
    """Channels of one layer (created once, in the same order on every rank)."""

    def __init__(self, layer):
        heap, g = _HEAP[0], layer.grid
        self.heap = heap
        self.row, self.col = heap.ctx(g.row_group), heap.ctx(g.col_group)
        self.p_o, self.p_d = self.row.size, self.col.size
        mk = lambda c: Channel(heap, c)                    # noqa: E731
        self.x_col, self.x_row = mk(self.col), mk(self.row)
        self.pay, self.dpay = mk(self.row), mk(self.row)
        self.dx_col, self.dx_row = mk(self.col), mk(self.row)


def _comm(layer):
    g = layer.grid
    if group_size(g.row_group) == 1 and group_size(g.col_group) == 1:
        return None
    c = getattr(layer, "_fb_comm", None)
    if c is None:
        c = layer._fb_comm = _Comm(layer)
    return c


def _attn_cfg(layer):
    a = layer.attn
    return 1, 1, float(a.scale), float(a.clamp[0]), float(a.clamp[1])          # gated scores, clamp-exp


class _FusedBranch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, wq, wk, wv, wg, layer):
        e = native.ext()
        dev = x.device
        g = layer.grid
        h, dh, d = layer.num_heads, layer.d_head, layer.dim_h
        hd = h * dh
        hp = _round8(h)
        with_gcn = layer.with_gcn
        n_kvg = (3 if with_gcn else 2) * d
        w_stack, _ = _stack(layer)
        status = native.status(dev)
        comm = _comm(layer)
        o = x.shape[0]
        x = x.contiguous()
        blk = layer.attn.block.csr
        plan = blk.row_plan(SEG_EDGES)
        sc, nm, scale, lo, hi = _attn_cfg(layer)
        gate_c = gate.detach().float().contiguous().view(gate.shape[0], -1)
        from .symm import wait_spins
        MAX_SPINS = wait_spins()
        if comm is None:
            # ---- one rank: one GEMM for K | V | message | Q, kernels read its column slices ----
            qkvg = native.gemm_nt(x, w_stack)
            ld = qkvg.shape[1]
            k_v, v_v, q_v = qkvg[:, :d], qkvg[:, d:2 * d], qkvg[:, n_kvg:]
            msg_v = qkvg[:, 2 * d:3 * d] if with_gcn else None
            xg_col = xg_row = x
            kvg, q, ldk, ldq = qkvg, q_v, ld, ld
        else:
            heap = comm.heap
            xoff = comm.col.staging(o * d * 2, "fb_x")
            heap.view(xoff, (o, d), torch.bfloat16).copy_(x)
            if comm.p_d > 1:
                comm.x_col.signal()
            if comm.p_o > 1:
                comm.x_row.signal()
            w_kvg, w_q = w_stack[:n_kvg], w_stack[n_kvg:]
            if comm.p_d > 1:
                kvg = torch.empty(comm.p_d * o, n_kvg, dtype=torch.bfloat16, device=dev)
                xg_col = torch.empty(comm.p_d * o, d, dtype=torch.bfloat16, device=dev)
                e.gemm_nt_gather([heap.peer_base[r] + xoff for r in comm.col.ranks], o, d, d, w_kvg, kvg, None, 0, 0.0, None, 0, xg_col,
                                 status, comm.x_col.flags, comm.x_col.counter, MAX_SPINS, comm.col.me)
            else:
                kvg, xg_col = native.gemm_nt(x, w_kvg), x
            if comm.p_o > 1:
                q = torch.empty(comm.p_o * o, d, dtype=torch.bfloat16, device=dev)
                xg_row = torch.empty(comm.p_o * o, d, dtype=torch.bfloat16, device=dev)
                e.gemm_nt_gather([heap.peer_base[r] + xoff for r in comm.row.ranks], o, d, d, w_q, q, None, 0, 0.0, None, 0, xg_row,
                                 status, comm.x_row.flags, comm.x_row.counter, MAX_SPINS, comm.row.me)
            else:
                q, xg_row = native.gemm_nt(x, w_q), x
            ldk, ldq = n_kvg, d
            k_v, v_v, q_v = kvg[:, :d], kvg[:, d:2 * d], q
            msg_v = kvg[:, 2 * d:3 * d] if with_gcn else None
        rows = q_v.shape[0]
        scratch = torch.empty(plan.num_slots, (hd + 2 * h + 3) // 4 * 4, dtype=torch.float32, device=dev) if plan.num_slots else None
        push = comm is not None and comm.p_o > 1
        gm = layer.gcn_block.matrix(torch.bfloat16, dev) if with_gcn else None
        if with_gcn:
            gplan = gm.row_plan(native.SPMM_SEG)
            gscratch = torch.empty(gplan.num_slots, d, dtype=torch.float32, device=dev) if gplan.num_slots else None
        if not push:
            acc = torch.empty(rows, hd, dtype=torch.float32, device=dev)
            l = torch.empty(rows, h, dtype=torch.float32, device=dev)
            e.attn_fwd(q_v, k_v, v_v, blk.col, blk.etype, gate_c, None, _plan_list(plan), None, acc, l, None, scratch, h, dh, sc, nm, scale,
                       lo, hi, hd, h, False, None, None, 0, ldq, ldk, [], 0, 0, 0)
            agg = None
            if with_gcn:
                agg = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)
                e.spmm(gm.crow, gm.col, gm.weight, msg_v, agg, False, _plan_list(gplan), gscratch, [], 0, 0, 0)
        else:
            width = hd + hp + (d if with_gcn else 0)
            slot_bytes = o * width * 2
            poff = comm.row.staging(comm.p_o * slot_bytes, "fb_pay")
            mine = [comm.heap.peer_base[r] + poff + comm.row.me * slot_bytes for r in comm.row.ranks]
            dummy = native.status(dev)                      # acc / l are unused when the rows are pushed
            e.attn_fwd(q_v, k_v, v_v, blk.col, blk.etype, gate_c, None, _plan_list(plan), None, dummy, dummy, None, scratch, h, dh, sc, nm,
                       scale, lo, hi, hd, h, False, None, None, 0, ldq, ldk, mine, o, width, hd)
            if with_gcn:
                e.spmm(gm.crow, gm.col, gm.weight, msg_v, dummy, False, _plan_list(gplan), gscratch, [p + (hd + hp) * 2 for p in mine], o, width,
                       rows)
            comm.pay.signal()
            acc = torch.empty(o, hd, dtype=torch.float32, device=dev)
            l = torch.empty(o, h, dtype=torch.float32, device=dev)
            agg = torch.empty(o, d, dtype=torch.bfloat16, device=dev) if with_gcn else None
            e.sum_payload(comm.heap.view(poff, (comm.p_o, o, width), torch.bfloat16), acc, l, agg, hd, hd + hp, comm.pay.flags, comm.pay.counter,
                          MAX_SPINS, status)
        ctx.layer = layer
        ctx.gate_dtype = gate.dtype
        ctx.dims = (ldq, ldk, n_kvg, rows, o)
        ctx.save_for_backward(q if comm is not None else kvg, kvg, xg_col, xg_row, gate_c)
        if agg is None:
            agg = x.new_zeros(0)
        return acc, l, agg

    @staticmethod
    def backward(ctx, dacc, dl, dagg):
        e = native.ext()
        layer = ctx.layer
        qbuf, kvg, xg_col, xg_row, gate_c = ctx.saved_tensors
        ldq, ldk, n_kvg, rows, o = ctx.dims
        dev = kvg.device
        h, dh, d = layer.num_heads, layer.d_head, layer.dim_h
        hd, hp = h * dh, _round8(h)
        with_gcn = layer.with_gcn
        comm = _comm(layer)
        status = native.status(dev)
        from .symm import wait_spins
        MAX_SPINS = wait_spins()
        w_stack, g_stack = _stack(layer)
        blk = layer.attn.block.csr
        sc, nm, scale, lo, hi = _attn_cfg(layer)
        dacc = dacc.contiguous()
        dl = dl.contiguous()
        cols = kvg.shape[0]
        row_vec = torch.empty(rows, hd, dtype=torch.bfloat16, device=dev)
        stat = torch.empty(rows, h, 4, dtype=torch.float32, device=dev)
        push = comm is not None and comm.p_o > 1
        if not push:
            e.attn_bwd_prep(dacc, dl, row_vec, stat)
            dagg_blk = dagg.contiguous() if with_gcn else None
        else:
            width = hd + hp + (d if with_gcn else 0)
            doff = comm.row.staging(o * width * 2, "fb_dpay")
            parts = [dacc, dl if hp == h else torch.nn.functional.pad(dl, (0, hp - h))] + ([dagg.contiguous()] if with_gcn else [])
            e.pack_cols(parts, comm.heap.view(doff, (o, width), torch.bfloat16), True)
            comm.dpay.signal()
            dagg_blk = torch.empty(rows, d, dtype=torch.bfloat16, device=dev) if with_gcn else None
            e.pull_unpack([comm.heap.peer_base[r] + doff for r in comm.row.ranks], o, width, row_vec, stat, dagg_blk, hd, hd + hp,
                          comm.dpay.flags, comm.dpay.counter, MAX_SPINS, status)
        # gradient buffers: one matrix per operand group, the passes write its column slices
        if comm is None:
            dall = torch.empty(rows, n_kvg + d, dtype=torch.bfloat16, device=dev)
            dkvg, dq, ldo_kv, ldo_q = dall, dall[:, n_kvg:], n_kvg + d, n_kvg + d
            q_v = kvg[:, n_kvg:]
        else:
            dkvg = torch.empty(cols, n_kvg, dtype=torch.bfloat16, device=dev)
            dq = torch.empty(rows, d, dtype=torch.bfloat16, device=dev)
            ldo_kv, ldo_q = n_kvg, d
            q_v = qbuf
        k_v, v_v = kvg[:, :d], kvg[:, d:2 * d]
        # column pass first: dk | dv into the first two column groups of dkvg, and the score gradient of every edge for the row pass
        from ..attention.backend_cuda import ds_buffer
        ds = ds_buffer(blk, h, torch.bfloat16, dev)
        _, rowidx, et_t, pos, _ = blk.csc()
        cplan = blk.col_plan(SEG_EDGES)
        cscratch = torch.empty(cplan.num_slots, 2 * hd, dtype=torch.float32, device=dev) if cplan.num_slots else None
        e.attn_bwd_col(q_v, k_v, v_v, row_vec, stat, rowidx, et_t, gate_c, None, _plan_list(cplan), dkvg, dkvg[:, d:2 * d], cscratch,
                       h, dh, sc, nm, scale, lo, hi, ldq, ldk, 0, ldo_kv, ds, pos if ds is not None else None)
        # row pass: dq and the gate gradient (K-only when the score gradients were handed over)
        plan = blk.row_plan(SEG_EDGES)
        nb = e.attn_bwd_row_blocks(plan.num_segments)
        t = gate_c.shape[0]
        dgp = torch.empty(nb, t * hd, dtype=torch.float32, device=dev)
        scratch = torch.empty(plan.num_slots, hd, dtype=torch.float32, device=dev) if plan.num_slots else None
        e.attn_bwd_row(q_v, k_v, v_v, row_vec, stat, blk.col, blk.etype, gate_c, None, _plan_list(plan), None, dq, False, dgp, None, nb, scratch,
                       h, dh, sc, nm, scale, lo, hi, ldq, ldk, 0, ldo_q, ds)
        dgate = torch.empty(t * hd, dtype=torch.float32, device=dev)
        e.reduce_partials(dgp, dgate, False)
        if with_gcn:
            gm = layer.gcn_block.matrix(torch.bfloat16, dev)
            ptr, idx, _, _, w_t = gm.csc()
            tplan = gm.col_plan(native.SPMM_SEG)
            tscratch = torch.empty(tplan.num_slots, d, dtype=torch.float32, device=dev) if tplan.num_slots else None
            e.spmm(ptr, idx, w_t if w_t.dtype == torch.float32 else w_t.float(), dagg_blk, dkvg[:, 2 * d:3 * d], False, _plan_list(tplan), tscratch,
                   [], 0, 0, 0)
        # weight gradients: K | V | message | Q rows of the stacked matrix
        grads = [None, None, None, None]
        if g_stack is not None:
            if comm is None:
                native.gemm_tn(dkvg, xg_col, out=g_stack, accumulate=True)
            else:
                native.gemm_tn(dkvg, xg_col, out=g_stack[:n_kvg], accumulate=True)
                native.gemm_tn(dq, xg_row, out=g_stack[n_kvg:], accumulate=True)
        else:
            if comm is None:
                dw = native.gemm_tn(dkvg, xg_col)
            else:
                dw = torch.cat([native.gemm_tn(dkvg, xg_col), native.gemm_tn(dq, xg_row)], dim=0)
            dwk, dwv = dw[:d], dw[d:2 * d]
            dwg = dw[2 * d:3 * d] if with_gcn else None
            grads = [dw[n_kvg:], dwk, dwv, dwg]
        # input gradient
        if comm is None:
            dx = native.gemm_nt(dkvg, w_stack.t().contiguous())
        else:
            heap = comm.heap
            w_kvg_t, w_q_t = w_stack[:n_kvg].t().contiguous(), w_stack[n_kvg:].t().contiguous()
            dx = torch.empty(o, d, dtype=torch.bfloat16, device=dev)
            first = True
            if comm.p_d > 1:
                soff = comm.col.staging(comm.p_d * o * d * 2, "fb_dxc")
                e.gemm_nt_scatter(dkvg, w_kvg_t, [heap.peer_base[r] + soff + comm.col.me * o * d * 2 for r in comm.col.ranks], o, d, status)
                comm.dx_col.signal()
            if comm.p_o > 1:
                roff = comm.row.staging(comm.p_o * o * d * 2, "fb_dxr")
                e.gemm_nt_scatter(dq, w_q_t, [heap.peer_base[r] + roff + comm.row.me * o * d * 2 for r in comm.row.ranks], o, d, status)
                comm.dx_row.signal()
            if comm.p_d > 1:
                e.sum_slots_wait(heap.view(soff, (comm.p_d, o, d), torch.bfloat16), dx, False, comm.dx_col.flags, comm.dx_col.counter, MAX_SPINS,
                                 status)
                first = False
            else:
                native.gemm_nt(dkvg, w_kvg_t, out=dx)
                first = False
            if comm.p_o > 1:
                e.sum_slots_wait(heap.view(roff, (comm.p_o, o, d), torch.bfloat16), dx, not first, comm.dx_row.flags, comm.dx_row.counter,
                                 MAX_SPINS, status)
            else:
                dx = dx + native.gemm_nt(dq, w_q_t)
        dgate = dgate.view(t, h, dh).to(ctx.gate_dtype)
        return dx, dgate, grads[0], grads[1], grads[2], grads[3], None


def fused_branch(layer, x, gate):
    """``(acc_owned, l_owned, agg_owned or None)`` or ``None`` when the configuration is outside this operator."""
    if not branch_supported(layer, x):
        return None
    wg = layer.gcn.lin.weight if layer.with_gcn else None
    acc, l, agg = _FusedBranch.apply(x, gate, layer.q.weight, layer.k.weight, layer.v.weight, wg, layer)
    return acc, l, (agg if layer.with_gcn else None)

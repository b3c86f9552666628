"""The native entry points that the fused 2D layer calls (``parallel/fused_layer.py``), restated in plain torch for the host
emulation of the peer-memory transport (:mod:`gt_b200.parallel.symm_host`).

Each method takes the arguments of the binding of the same name (``csrc/binding.cpp``) and does what the kernel does to its
outputs, with fp32 arithmetic on CPU tensors: the GEMMs with the all-gather in their operand loads or the reduce-scatter in their
epilogue, the gather attention passes in partial (unnormalised) form with gated scores and clamp-exp weights, the aggregation, the
payload packing, and the owner-side sums behind a bounded channel wait.  What is emulated is the DATA FLOW between ranks (which
slice goes into which peer's slot at which offset, which flag is waited for before which read); the arithmetic inside a kernel is
whatever torch does.  ``row_vec`` / ``stat`` carry ``dacc`` / ``dl`` from ``attn_bwd_prep`` or ``pull_unpack`` to the two backward
passes; the layout inside ``stat`` is private to this emulation.

Used by the tests that run the fused operator on 2 x 2, 4 x 2 and 2 x 4 grids of CPU processes against the fp64 reference model.
"""
import time

import torch


def _edge_rows(plan, n_edges):
    """Major index (row of a CSR pass, column of a CSC pass) of every entry, from the segment list of a plan."""
    seg_row, seg_beg, seg_end = plan[0].long(), plan[1].long(), plan[2].long()
    out = torch.full((n_edges,), -1, dtype=torch.long)
    lens = seg_end - seg_beg
    if int(lens.sum()) != n_edges:
        raise ValueError("the segments of the plan do not cover every entry exactly once")
    owner = torch.repeat_interleave(seg_row, lens)
    start = torch.repeat_interleave(seg_beg - torch.cumsum(lens, 0) + lens, lens)
    out[start + torch.arange(n_edges)] = owner
    if int(out.min()) < 0:
        raise ValueError("the segments of the plan overlap")
    return out


class FusedKernelsHost:
    """Mixin of :class:`gt_b200.parallel.symm_host.HostExt` (which provides ``_typed`` and ``_wait``)."""

    @staticmethod
    def attn_shape_supported(h, d, t):
        return True

    @staticmethod
    def attn_bwd_row_blocks(n_seg):
        return 1

    # ---- dense products ---------------------------------------------------------------------------------------------------
    @staticmethod
    def _epilogue(y, bias, act, p):
        if p:
            raise NotImplementedError("dropout inside the emulated GEMM epilogue")
        if bias is not None:
            y = y + bias.float()
        return torch.relu(y) if act == 1 else (torch.nn.functional.gelu(y) if act == 2 else y)

    def gemm_nt(self, a, b, c, bias, act, p, seed, site, accumulate, status):
        y = self._epilogue(a.float() @ b.float().t(), bias, act, p)
        c.copy_(c.float() + y if accumulate else y)

    def gemm_tn(self, a, b, c, accumulate, status):
        y = a.float().t() @ b.float()
        c.copy_(c + y if accumulate else y)

    def gemm_nt_gather(self, peer_ptrs, chunk, k, lda, b, c, bias, act, p, seed, site, gathered, status, flags, counter, max_spins, me):
        if lda != k:
            raise NotImplementedError("strided peer operand")
        want = int(counter) if counter is not None else 0
        for i, ptr in enumerate(peer_ptrs):
            if flags is not None and i != me:
                self._wait_one(flags, i, want, status)
            a = self._typed(ptr, chunk * k, torch.bfloat16, "read").view(chunk, k)
            if gathered is not None:
                gathered[i * chunk:(i + 1) * chunk] = a
            c[i * chunk:(i + 1) * chunk] = self._epilogue(a.float() @ b.float().t(), bias, act, p)

    def gemm_nt_scatter(self, a, b, slot_ptrs, chunk, ldc, status):
        n = b.shape[0]
        if ldc != n:
            raise NotImplementedError("strided slots")
        for i, ptr in enumerate(slot_ptrs):
            y = a[i * chunk:(i + 1) * chunk].float() @ b.float().t()
            self._typed(ptr, chunk * n, torch.bfloat16, "write").view(chunk, n).copy_(y)

    # ---- attention, gated scores and clamp-exp weights, partial form --------------------------------------------------------------
    @staticmethod
    def _partial(q, k, v, rows, cols, et, gate, h, d, scale, lo, hi):
        qe = q.reshape(-1, h, d)[rows] * gate.reshape(-1, h, d)[et]
        s = (qe * k.reshape(-1, h, d)[cols]).sum(-1) * scale
        p = torch.exp(s.clamp(lo, hi))
        acc = torch.zeros(q.shape[0], h, d).index_add_(0, rows, p.unsqueeze(-1) * v.reshape(-1, h, d)[cols])
        l = torch.zeros(q.shape[0], h).index_add_(0, rows, p)
        return acc, l

    @staticmethod
    def _check_mode(score, norm, gate, etype):
        if score != 1 or norm != 1 or gate is None or etype is None:
            raise NotImplementedError("the emulation covers gated scores with clamp-exp weights (the fused Exphormer layer)")

    def attn_fwd(self, q, k, v, idx, etype, gate, bias, plan, row_map, acc, l, m, scratch, h, d, score, norm, scale, lo, hi, acc_stride, l_stride,
                 accumulate, k_peers, v_peers, rows_per_peer, ldq, ldk, push_ptrs, push_rows, push_ld, push_l_off):
        self._check_mode(score, norm, gate, etype)
        if k_peers is not None or v_peers is not None or row_map is not None:
            raise NotImplementedError("the emulation covers the forward of the fused layer (local K / V, every row of the block)")
        rows = _edge_rows(plan, idx.numel())
        a, s = self._partial(q.float(), k.float(), v.float(), rows, idx.long(), etype.long(), gate.float(), h, d, scale, lo, hi)
        a = a.reshape(q.shape[0], h * d)
        if not push_ptrs:
            acc.copy_(acc + a if accumulate else a)
            l.copy_(l + s if accumulate else s)
            return
        for i, ptr in enumerate(push_ptrs):                  # rows of owner i go into MY slot of owner i's payload buffer
            slot = self._typed(ptr, push_rows * push_ld, torch.bfloat16, "write").view(push_rows, push_ld)
            lo_r = i * push_rows
            slot[:, :h * d] = a[lo_r:lo_r + push_rows]
            slot[:, push_l_off:push_l_off + h] = s[lo_r:lo_r + push_rows]
            pad = -(-h // 8) * 8
            if pad > h:
                slot[:, push_l_off + h:push_l_off + pad] = 0

    def _grads(self, q, k, v, rows, cols, et, gate, row_vec, stat, h, d, scale, lo, hi):
        with torch.enable_grad():                            # called from inside an autograd backward, where recording is off
            q32, k32, v32, g32 = (t.float().detach().clone().requires_grad_(True) for t in (q, k, v, gate))
            acc, l = self._partial(q32, k32, v32, rows, cols, et, g32, h, d, scale, lo, hi)
            dacc = row_vec.float().reshape(-1, h, d)
            dl = stat[:, :, 0]
            return torch.autograd.grad((acc, l), (q32, k32, v32, g32), (dacc, dl))

    @staticmethod
    def attn_bwd_prep(dacc, dl, row_vec, stat):
        row_vec.copy_(dacc)
        stat.zero_()
        stat[:, :, 0] = dl

    def attn_bwd_col(self, q, k, v, row_vec, stat, rowidx, etype_t, gate, bias, plan, dk, dv, scratch, h, d, score, norm, scale, lo, hi, ldq, ldk,
                     ldr, ldo, ds_out, pos):
        self._check_mode(score, norm, gate, etype_t)
        cols = _edge_rows(plan, rowidx.numel())              # the plan of this pass walks the columns
        _, gk, gv, _ = self._grads(q, k, v, rowidx.long(), cols, etype_t.long(), gate, row_vec, stat, h, d, scale, lo, hi)
        dk[:, :h * d] = gk.reshape(-1, h * d)
        dv[:, :h * d] = gv.reshape(-1, h * d)

    def attn_bwd_row(self, q, k, v, row_vec, stat, idx, etype, gate, bias, plan, row_map, dq, accumulate_dq, dgate_part, dbias_part, n_blocks,
                     scratch, h, d, score, norm, scale, lo, hi, ldq, ldk, ldr, ldo, ds_in):
        self._check_mode(score, norm, gate, etype)
        rows = _edge_rows(plan, idx.numel())
        gq, _, _, gg = self._grads(q, k, v, rows, idx.long(), etype.long(), gate, row_vec, stat, h, d, scale, lo, hi)
        gq = gq.reshape(-1, h * d)
        dq[:, :h * d] = dq[:, :h * d].float() + gq if accumulate_dq else gq
        if dgate_part is not None:
            dgate_part.zero_()
            dgate_part[0] = gg.reshape(-1)

    @staticmethod
    def reduce_partials(part, out, accumulate):
        s = part.sum(0)
        out.copy_(out + s if accumulate else s)

    # ---- aggregation ------------------------------------------------------------------------------------------------------
    def spmm(self, ptr, idx, w, x, out, accumulate, plan, scratch, push_ptrs, push_rows, push_ld, n_out):
        n_rows = ptr.numel() - 1
        rows = torch.repeat_interleave(torch.arange(n_rows), (ptr[1:] - ptr[:-1]).long())
        vals = x.float()[idx.long()]
        if w is not None:
            vals = vals * w.float().unsqueeze(1)
        y = torch.zeros(n_rows, x.shape[1]).index_add_(0, rows, vals)
        if not push_ptrs:
            out.copy_(out.float() + y if accumulate else y)
            return
        for i, p in enumerate(push_ptrs):                    # the pointer already addresses the aggregation columns of my slot
            width = x.shape[1]
            flat = self._typed(p, (push_rows - 1) * push_ld + width, torch.bfloat16, "write")
            torch.as_strided(flat, (push_rows, width), (push_ld, 1)).copy_(y[i * push_rows:(i + 1) * push_rows])

    # ---- payload packing and the owner-side sums -----------------------------------------------------------------------------------
    def pack_cols(self, parts, packed, to_packed):
        c = 0
        self._access("write" if to_packed else "read", packed)
        for t in parts:
            w = t.shape[1]
            if to_packed:
                packed[:, c:c + w] = t
            else:
                t.copy_(packed[:, c:c + w])
            c += w

    def _wait_one(self, flags, p, want, status):
        if self.log is not None:
            self._note("wait", self._place(flags)[1], p)
        deadline = time.monotonic() + self.wait_seconds
        while int(flags[p]) < want:
            if time.monotonic() > deadline:
                status.fill_(100 + p)
                return
            time.sleep(0)

    def sum_payload(self, slots, acc, l, agg, l_off, agg_off, flags, counter, max_spins, status):
        if flags is not None:
            self._wait(flags, slots.shape[0], int(counter), status)
        self._access("read", slots)
        s = slots.float().sum(0)
        acc.copy_(s[:, :acc.shape[1]])
        l.copy_(s[:, l_off:l_off + l.shape[1]])
        if agg is not None:
            agg.copy_(s[:, agg_off:agg_off + agg.shape[1]])

    def pull_unpack(self, src_ptrs, rows_per_peer, width, row_vec, stat, dagg, l_off, agg_off, flags, counter, max_spins, status):
        if flags is not None:
            self._wait(flags, len(src_ptrs), int(counter), status)
        hd, h = row_vec.shape[1], stat.shape[1]
        stat.zero_()
        for i, ptr in enumerate(src_ptrs):
            pay = self._typed(ptr, rows_per_peer * width, torch.bfloat16, "read").view(rows_per_peer, width)
            r = slice(i * rows_per_peer, (i + 1) * rows_per_peer)
            row_vec[r] = pay[:, :hd]
            stat[r, :, 0] = pay[:, l_off:l_off + h].float()
            if dagg is not None:
                dagg[r] = pay[:, agg_off:agg_off + dagg.shape[1]]

    def sum_slots_wait(self, slots, out, accumulate, flags, counter, max_spins, status):
        if flags is not None:
            self._wait(flags, slots.shape[0], int(counter), status)
        self._access("read", slots)
        s = slots.float().sum(0).view(out.shape)
        out.copy_(out.float() + s if accumulate else s)

    def sum_slots(self, slots, out, accumulate):
        self.sum_slots_wait(slots, out, accumulate, None, None, 0, None)

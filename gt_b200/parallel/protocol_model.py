"""Symbolic programs of the peer-memory protocols, for the happens-before checker of :mod:`gt_b200.utils.hb_check`.

``fused_step_trace`` restates, operation by operation, what one training step of the fused 2D layer does to memory that other
ranks can see: which staging copy every use takes (``GroupContext.staging``: two copies per kind, alternating; the alternation
restarts in ``SymmetricHeap.begin_step``), who writes and reads it, and which channel is signalled or waited on in between
(``parallel/fused_layer.py``: ``_FusedBranch.forward`` / ``backward``; ``train/engine.py``: ``_body``;
``SymmetricHeap.all_reduce_two_shot``).  Local work (the attention passes, GEMMs on local operands, LayerNorm, the optimizer) is
left out: it touches no shared buffer.  ``barrier_collective_trace`` is the "write my staging copy, group barrier, read the
members' copies" pattern of ``SymmetricHeap.all_gather`` / ``reduce_scatter`` / ``all_to_all`` that the other layer kinds use.

The checker then proves for a grid and a depth what the docstrings argue in words (two copies per kind are enough however deep
the model; no buffer is rewritten while a peer may still read it; every read finds the version it expects), shows that the
argument does NOT hold with one copy (the negative control of the tests), and shows what a lost signal or a stopped rank leads
to: expired waits that name the silent peer, never a rank that blocks.

    python -m gt_b200.parallel.protocol_model --grid 2 2 --layers 3 --steps 2
    python -m gt_b200.parallel.protocol_model --grid 4 2 --layers 4 --copies 1          # reports the hazards of single buffering
    python -m gt_b200.parallel.protocol_model --grid 2 2 --drop 1 pay0 2                # rank 1 loses its 2nd signal on channel pay0
"""
import argparse

from ..utils.hb_check import ProtocolTrace, check


class _Ctx:
    """A rank's view of one group: the members' global ranks, its index among them and the per-kind use counts."""

    def __init__(self, name, members, rank):
        self.name, self.members, self.me, self.size = name, tuple(members), tuple(members).index(rank), len(members)
        self.kind_count = {}

    def staging(self, kind, copies):
        n = self.kind_count.get(kind, 0)
        self.kind_count[kind] = n + 1
        return (self.name, kind, n % copies)


def grid_groups(p_d, p_o):
    """``rank -> (row members, column members)`` for rank ``d * p_o + o`` of a ``p_d x p_o`` grid: the row group shares the row block
    ``d`` (``p_o`` members), the column group shares the column block ``o`` (``p_d`` members)."""
    out = {}
    for d in range(p_d):
        for o in range(p_o):
            out[d * p_o + o] = ([d * p_o + j for j in range(p_o)], [i * p_o + o for i in range(p_d)])
    return out


def fused_step_trace(p_d, p_o, layers, steps=2, copies=2, begin_barriers=True, eval_after=False, recompute=False, grad_allreduce=True):
    """Programs of all ranks for ``steps`` training steps of ``layers`` fused layers on a ``p_d x p_o`` grid.

    ``copies``: staging copies per kind (the package uses 2).  ``begin_barriers``: the group barriers of ``begin_step``.
    ``eval_after``: a forward-only pass after every step (an evaluation; it does not call ``begin_step``).  ``recompute``: layer
    checkpointing, every layer's forward runs again right before its backward."""
    world = p_d * p_o
    tr = ProtocolTrace(world)
    groups = grid_groups(p_d, p_o)
    everyone = tuple(range(world))
    for r in range(world):
        # buffer names carry the kind of group only: the heap is symmetric, a staging copy sits at the same offset on every rank
        row = _Ctx("row", groups[r][0], r)
        col = _Ctx("col", groups[r][1], r)
        wld = _Ctx("world", everyone, r)

        def forward(step, l, phase):
            tag = (phase, step, l)
            # x -> my staging copy, published to the column and the row group; the projection GEMMs read the members' copies
            xb = col.staging("fb_x", copies)
            tr.write(r, r, xb, ("x",) + tag, "x to staging")
            if p_d > 1:
                tr.signal(r, "x_col%d" % l, col.members)
            if p_o > 1:
                tr.signal(r, "x_row%d" % l, row.members)
            if p_d > 1:
                for p in col.members:
                    if p != r:
                        tr.wait(r, "x_col%d" % l, col.members, p, "gemm_nt_gather (K|V|message)")
                    tr.read(r, p, xb, ("x",) + tag, "gemm_nt_gather (K|V|message)")
            if p_o > 1:
                for p in row.members:
                    if p != r:
                        tr.wait(r, "x_row%d" % l, row.members, p, "gemm_nt_gather (Q)")
                    tr.read(r, p, xb, ("x",) + tag, "gemm_nt_gather (Q)")
            # partial rows pushed into the owners' slots by the attention / aggregation epilogues; the owner sums its slots
            if p_o > 1:
                pb = row.staging("fb_pay", copies)
                for p in row.members:
                    tr.write(r, p, pb + (row.me,), ("pay",) + tag, "attention / SpMM epilogue push")
                tr.signal(r, "pay%d" % l, row.members)
                for p in row.members:
                    tr.wait(r, "pay%d" % l, row.members, p, "sum_payload")
                for s in range(row.size):
                    tr.read(r, r, pb + (s,), ("pay",) + tag, "sum_payload")

        def backward(step, l):
            tag = ("bwd", step, l)
            if p_o > 1:                                     # owners publish (dacc | dl | dagg); the row block is pulled from them
                db = row.staging("fb_dpay", copies)
                tr.write(r, r, db, ("dpay",) + tag, "pack_cols")
                tr.signal(r, "dpay%d" % l, row.members)
                for p in row.members:
                    tr.wait(r, "dpay%d" % l, row.members, p, "pull_unpack")
                for p in row.members:
                    tr.read(r, p, db, ("dpay",) + tag, "pull_unpack")
            if p_d > 1:                                     # dx tiles stored into the owners' slots, summed by the owner
                cb = col.staging("fb_dxc", copies)
                for p in col.members:
                    tr.write(r, p, cb + (col.me,), ("dxc",) + tag, "gemm_nt_scatter (column group)")
                tr.signal(r, "dx_col%d" % l, col.members)
            if p_o > 1:
                rb = row.staging("fb_dxr", copies)
                for p in row.members:
                    tr.write(r, p, rb + (row.me,), ("dxr",) + tag, "gemm_nt_scatter (row group)")
                tr.signal(r, "dx_row%d" % l, row.members)
            if p_d > 1:
                for p in col.members:
                    tr.wait(r, "dx_col%d" % l, col.members, p, "sum_slots_wait (column group)")
                for s in range(col.size):
                    tr.read(r, r, cb + (s,), ("dxc",) + tag, "sum_slots_wait (column group)")
            if p_o > 1:
                for p in row.members:
                    tr.wait(r, "dx_row%d" % l, row.members, p, "sum_slots_wait (row group)")
                for s in range(row.size):
                    tr.read(r, r, rb + (s,), ("dxr",) + tag, "sum_slots_wait (row group)")

        for step in range(steps):
            for c in (row, col, wld):                       # begin_step: the alternation restarts, the groups synchronise
                c.kind_count.clear()
                if begin_barriers and c.size > 1:
                    tr.barrier(r, "barrier_" + c.name, c.members, "begin_step")
            tr.write(r, r, ("grads",), ("zero", step), "gradient buffer zero-fill")
            for l in range(layers):
                forward(step, l, "fwd")
            for l in reversed(range(layers)):
                if recompute:
                    forward(step, l, "recompute")
                backward(step, l)
            tr.write(r, r, ("grads",), ("g", step), "weight-gradient GEMMs")
            if grad_allreduce and world > 1:                # two-shot all-reduce: reduce my slice from everyone, store it to everyone
                tr.signal(r, "grad_ready", everyone)
                for p in everyone:
                    tr.wait(r, "grad_ready", everyone, p, "allreduce_two_shot")
                for p in everyone:
                    tr.read(r, p, ("grads",), ("g", step), "allreduce_two_shot")
                for p in everyone:
                    tr.write(r, p, ("grads_sum", r), ("sum", step), "allreduce_two_shot")
                tr.signal(r, "grad_done", everyone)
                for p in everyone:
                    tr.wait(r, "grad_done", everyone, p, "channel_wait")
                for s in everyone:
                    tr.read(r, r, ("grads_sum", s), ("sum", step), "optimizer")
            if eval_after:
                for l in range(layers):
                    forward(step, l, "eval")
    return tr


def barrier_collective_trace(size, uses, copies=2):
    """``uses`` collectives of one kind on a group of ``size`` ranks: write my staging copy, group barrier, read every member's copy."""
    tr = ProtocolTrace(size)
    members = tuple(range(size))
    for r in range(size):
        c = _Ctx("g", members, r)
        for u in range(uses):
            b = c.staging("ag", copies)
            tr.write(r, r, b, ("ag", u), "staging copy")
            tr.barrier(r, "barrier_g", members, "group barrier")
            for p in members:
                tr.read(r, p, b, ("ag", u), "pull kernel")
    return tr


def describe(rep, limit=12):
    lines = [f"operations {rep.n_ops}, violations {len(rep.violations)}, expired waits {len(rep.expired)}, "
             f"all ranks reached the end: {rep.completed}, status words {rep.status}"]
    for v in rep.violations[:limit]:
        lines.append(f"  {v.kind}: rank {v.rank} op {v.op}, buffer {v.buf} of rank {v.owner}: {v.detail}")
    for r, op, chan, peer in rep.expired[:limit]:
        lines.append(f"  expired: rank {r} op {op} waited on channel {chan} for rank {peer}")
    return "\n".join(lines)


def main(argv=None):
    ap = argparse.ArgumentParser(description="happens-before check of the fused layer's peer-memory protocol")
    ap.add_argument("--grid", type=int, nargs=2, default=[2, 2], metavar=("P_d", "P_o"))
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--copies", type=int, default=2, help="staging copies per kind (the package uses 2)")
    ap.add_argument("--no_begin_barriers", action="store_true")
    ap.add_argument("--eval_after", action="store_true")
    ap.add_argument("--recompute", action="store_true")
    ap.add_argument("--drop", nargs=3, action="append", default=[], metavar=("RANK", "CHANNEL", "K"),
                    help="the K-th signal of RANK on CHANNEL (x_col<l>, x_row<l>, pay<l>, dpay<l>, dx_col<l>, dx_row<l>, grad_ready, grad_done, "
                         "barrier_<group>) is lost")
    ap.add_argument("--die", nargs=2, action="append", default=[], metavar=("RANK", "OP"), help="RANK stops before its operation number OP")
    args = ap.parse_args(argv)
    tr = fused_step_trace(args.grid[0], args.grid[1], args.layers, args.steps, args.copies, not args.no_begin_barriers, args.eval_after,
                          args.recompute)
    rep = check(tr, drop={(int(r), c, int(k)) for r, c, k in args.drop}, die={int(r): int(o) for r, o in args.die})
    print(describe(rep))
    return 0 if not rep.violations and not rep.expired else 1


if __name__ == "__main__":
    raise SystemExit(main())

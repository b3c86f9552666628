"""Per-epoch census of the collectives a training step issues: calls, payload bytes and (on GPUs) device time per kind
and group size.  The counterpart of the reference trainer's ``--coll_stats`` (``gt3d/gt3d/train/train_dist.py:120-190``),
which patches ``torch.distributed``; here the methods of the peer-memory transport (``gt_b200.parallel.symm.SymmetricHeap``)
are patched the same way and reported under ``p2p_*`` kinds (the collectives fused into GEMMs included), so ``--comm nccl``
and ``--comm p2p`` runs both give a complete table.

Device time is taken with one CUDA-event pair per call (recorded on the launching stream, read after the epoch), so the
census itself adds no host synchronisation inside the step; it is not usable under CUDA-graph capture.
"""
import collections
import contextlib

import torch
import torch.distributed as dist

_KINDS = {
    "all_gather_into_tensor": ("all_gather", lambda a, kw: a[0]),
    "reduce_scatter_tensor": ("reduce_scatter", lambda a, kw: a[1] if len(a) > 1 else kw["input"]),
    "all_reduce": ("all_reduce", lambda a, kw: a[0]),
    "all_to_all_single": ("all_to_all", lambda a, kw: a[1] if len(a) > 1 else kw["input"]),
    "broadcast": ("broadcast", lambda a, kw: a[0]),
}


# methods of the symmetric heap (peer-memory transport): name -> (kind, where the group is: argument index or "plan")
_HEAP_KINDS = {
    "all_gather": ("p2p_all_gather", 1),
    "reduce_scatter": ("p2p_reduce_scatter", 1),
    "all_reduce": ("p2p_all_reduce", 3),
    "rows_to_heads": ("p2p_all_to_all", 1),
    "heads_to_rows": ("p2p_all_to_all", 1),
    "linear_gather": ("p2p_gather+gemm", 2),
    "linear_scatter": ("p2p_gemm+scatter", 2),
    "pull_gather": ("p2p_sparse_gather", "plan"),
    "pull_reduce": ("p2p_sparse_reduce", "plan"),
}


def _group_size(kw):
    g = kw.get("group")
    return dist.get_world_size(g) if g is not None else dist.get_world_size()


class CollectiveStats:
    """``begin_epoch()`` / ``end_epoch(keep)`` bracket a step; ``report()`` prints the per-epoch mean on rank 0."""

    def __init__(self):
        self.rows = collections.defaultdict(lambda: [0, 0, 0.0])        # (kind, group size) -> calls, bytes, ms
        self.epochs = 0
        self._pending = []
        self._orig = {}
        self._orig_heap = {}
        self._cur = None

    # ---- patching ------------------------------------------------------------------------------------------------------
    def _wrap(self, name, fn, kind, pick):
        def wrapped(*a, **kw):
            t = pick(a, kw)
            key = (kind, _group_size(kw))
            nbytes = t.numel() * t.element_size()
            ev = None
            if t.is_cuda and not torch.cuda.is_current_stream_capturing():
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
            out = fn(*a, **kw)
            if ev is not None:
                if kw.get("async_op") and out is not None:
                    out.wait()
                ev[1].record()
            self._cur.append((key, nbytes, ev))
            return out
        return wrapped

    def _wrap_heap(self, name, fn, kind, where):
        def wrapped(heap, *a, **kw):
            t = a[0]
            if where == "plan":
                group = a[1].group
            else:
                group = kw.get("group", a[where] if len(a) > where else None)
            key = (kind, heap.ctx(group).size)
            ev = None
            if t.is_cuda and not torch.cuda.is_current_stream_capturing():
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
            out = fn(heap, *a, **kw)
            if ev is not None:
                ev[1].record()
            if self._cur is not None:
                self._cur.append((key, t.numel() * t.element_size(), ev))
            return out
        return wrapped

    def record(self, kind, group_size, nbytes, events=None):
        """Entry point for transports that do not go through ``torch.distributed`` (the symmetric-heap kernels)."""
        if self._cur is not None:
            self._cur.append(((kind, group_size), nbytes, events))

    def begin_epoch(self):
        self._cur = []
        for name, (kind, pick) in _KINDS.items():
            self._orig[name] = getattr(dist, name)
            setattr(dist, name, self._wrap(name, self._orig[name], kind, pick))
        from ..parallel.symm import SymmetricHeap
        for name, (kind, where) in _HEAP_KINDS.items():
            if hasattr(SymmetricHeap, name):
                self._orig_heap[name] = getattr(SymmetricHeap, name)
                setattr(SymmetricHeap, name, self._wrap_heap(name, self._orig_heap[name], kind, where))
        global ACTIVE
        ACTIVE = self

    def end_epoch(self, keep=True):
        global ACTIVE
        ACTIVE = None
        for name, fn in self._orig.items():
            setattr(dist, name, fn)
        self._orig = {}
        if self._orig_heap:
            from ..parallel.symm import SymmetricHeap
            for name, fn in self._orig_heap.items():
                setattr(SymmetricHeap, name, fn)
            self._orig_heap = {}
        cur, self._cur = self._cur, None
        if not keep:
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for key, nbytes, ev in cur:
            r = self.rows[key]
            r[0] += 1
            r[1] += nbytes
            if ev is not None:
                r[2] += ev[0].elapsed_time(ev[1])
        self.epochs += 1

    def table(self):
        n = max(self.epochs, 1)
        return {k: dict(calls=v[0] / n, mbytes=v[1] / n / 2 ** 20, ms=v[2] / n) for k, v in sorted(self.rows.items())}

    def report(self, file=None):
        if dist.is_initialized() and dist.get_rank() != 0:
            return
        print(f"[coll_stats] per epoch, rank 0, mean of {self.epochs} epochs (payload = the larger side of the call)", file=file)
        print(f"[coll_stats] {'kind':16s} {'group':>5s} {'calls':>8s} {'MiB':>10s} {'device ms':>10s}", file=file)
        tot = [0.0, 0.0, 0.0]
        for (kind, g), r in self.table().items():
            print(f"[coll_stats] {kind:16s} {g:5d} {r['calls']:8.1f} {r['mbytes']:10.2f} {r['ms']:10.3f}", file=file)
            tot = [tot[0] + r["calls"], tot[1] + r["mbytes"], tot[2] + r["ms"]]
        print(f"[coll_stats] {'total':16s} {'':5s} {tot[0]:8.1f} {tot[1]:10.2f} {tot[2]:10.3f}", file=file, flush=True)


ACTIVE = None


@contextlib.contextmanager
def collective_stats():
    cs = CollectiveStats()
    cs.begin_epoch()
    try:
        yield cs
    finally:
        cs.end_epoch()

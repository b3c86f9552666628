"""Per-kernel device time of the sparse gather against the sparse reduce-scatter of the same rows.

    torchrun --nproc-per-node 4 -m gt_b200.bench.profile_sparse_comm --rows 612352 --width 256 --share 0.25 --transport a2a

Builds a :class:`SparseRowPlan` over the world group in which every rank needs a random ``--share`` of the block's rows, times
``gather`` and ``reduce_scatter`` (device time, max over ranks), and prints the profiler's kernel table of each on rank 0, so
that the kernels that make one direction slower than the other (index_select, the all-to-all, the segmented sum, the pull
kernels) can be read off.  Counterpart of the reference's ``gt3d/bench/profile_sparse_comm.py``.  On CPU ranks (gloo) it runs
the same plan and prints wall-clock times only.  Returns ``{"gather_ms", "reduce_ms", "share"}``.
"""
import argparse
import io
import json
import time

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=612352, help="rows of the gathered block (all ranks together)")
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--share", type=float, default=0.25)
    ap.add_argument("--transport", default="a2a", choices=["a2a", "pull"])
    ap.add_argument("--heap_mb", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    from ..parallel.sparse_comm import SparseRowPlan
    from ..train.train_dist import init_dist
    from ..utils.profiling import kernel_profile
    init_dist()
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    dt = torch.bfloat16 if cuda else torch.float32
    per = -(-args.rows // world // 8) * 8
    g = torch.Generator().manual_seed(100 + rank)
    need = torch.randperm(per * world, generator=g)[:max(1, int(args.share * per * world))].sort().values.to(dev)
    heap = None
    if cuda and world > 1 and args.transport == "pull":
        from ..parallel.symm import SymmetricHeap
        heap = SymmetricHeap(dev, args.heap_mb << 20)
    plan = SparseRowPlan(dist.group.WORLD, per, need, name="profile", transport=args.transport if heap is not None else "a2a", heap=heap)
    torch.manual_seed(rank)
    x = torch.randn(per, args.width, device=dev).to(dt)
    y = torch.randn(plan.n_need, args.width, device=dev).to(dt)

    def step(fn):
        if heap is not None:
            heap.begin_step()
        return fn()

    def timed(fn):
        if cuda:
            from ._timing import time_ms
            return time_ms(lambda: step(fn), args.iters, 3, max_over_ranks=True)
        step(fn)
        t0 = time.perf_counter()
        for _ in range(args.iters):
            step(fn)
        return (time.perf_counter() - t0) / args.iters * 1e3

    res = dict(world=world, rows=per * world, width=args.width, share=round(plan.share, 4), transport=plan.transport)
    for name, fn in (("gather", lambda: plan.gather(x)), ("reduce", lambda: plan.reduce_scatter(y))):
        res[f"{name}_ms"] = round(timed(fn), 4)
        if cuda:
            buf = io.StringIO()
            with kernel_profile(rank=rank, world=world, top=12, file=buf):
                for _ in range(args.iters):
                    step(fn)
            if rank == 0:
                print(f"--- {name}: {args.iters} calls ---\n" + buf.getvalue(), flush=True)
    if rank == 0:
        print("SPARSE_COMM " + json.dumps(res), flush=True)
    if heap is not None:
        heap.close()
    return res


if __name__ == "__main__":
    main()

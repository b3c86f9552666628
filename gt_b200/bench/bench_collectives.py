"""Row-collective benchmark: the ways this package can move the rows of a gathered block, at one payload shape.

    torchrun --nproc-per-node 8 -m gt_b200.bench.bench_collectives --rows 169344 --width 256 --share 0.25

Measures, over the world group, device time (max over ranks) of
  * dense all-gather / reduce-scatter by NCCL and by the peer-memory kernels (symmetric heap),
  * the sparse gather / reduce of a random ``--share`` of the block's rows by all-to-all-v (NCCL) and by the
    receiver-driven pull kernels, with a correctness check of both against an index of the dense result,
  * one ring hop of the chunk with one or two buffers in flight.
Counterpart of the reference's ``bench_sparse_comm.py``, ``bench_pull_nvshmem.py``, ``bench_pull_sparse.py`` and
``ring_p2p.py``; prints ``COLL`` lines and one ``A2A_OVER_AG`` line (the constant of the sparse-communication rule).
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ._timing import time_ms


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=169344, help="rows of the gathered block (all ranks together)")
    ap.add_argument("--width", type=int, default=256)
    ap.add_argument("--share", type=float, default=0.25)
    ap.add_argument("--heap_mb", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    args = ap.parse_args(argv)
    from ..train.train_dist import init_dist
    init_dist()
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    from ..parallel.collectives import raw_all_gather_rows, raw_reduce_scatter_rows
    from ..parallel.ring import RingComm
    from ..parallel.sparse_comm import SparseRowPlan
    dt = torch.bfloat16 if cuda else torch.float32
    per = -(-args.rows // world // 8) * 8
    torch.manual_seed(rank)
    x = torch.randn(per, args.width, device=dev).to(dt)
    full = torch.randn(per * world, args.width, device=dev).to(dt)
    heap = None
    if cuda and world > 1:
        from ..parallel.symm import SymmetricHeap
        heap = SymmetricHeap(dev, args.heap_mb << 20)

    def t(fn):
        if cuda:
            return time_ms(fn, args.iters, 3, max_over_ranks=True)
        import time
        fn()
        t0 = time.perf_counter()
        for _ in range(args.iters):
            fn()
        return (time.perf_counter() - t0) / args.iters * 1e3

    res = {}
    moved = per * (world - 1) * args.width * x.element_size()
    res["ag_nccl"] = t(lambda: raw_all_gather_rows(x, None))
    res["rs_nccl"] = t(lambda: raw_reduce_scatter_rows(full, None))
    if heap is not None:
        def ag_heap():
            heap.begin_step()
            return heap.all_gather(x, None)

        def rs_heap():
            heap.begin_step()
            return heap.reduce_scatter(full, None)
        res["ag_heap"], res["rs_heap"] = t(ag_heap), t(rs_heap)
        assert torch.equal(ag_heap(), raw_all_gather_rows(x, None)), "heap all-gather differs from NCCL"
    # projection with its collective: NCCL all-gather + GEMM vs the GEMM that gathers through TMA loads from peer memory,
    # and GEMM + NCCL reduce-scatter vs the GEMM whose epilogue stores into the owners' memory
    if heap is not None and cuda and args.width <= 512:
        from ..ops import native
        n_out = 3 * args.width
        w = (torch.randn(n_out, args.width, device=dev) * args.width ** -0.5).bfloat16()
        wt = w.t().contiguous()
        dy = torch.randn(per * world, n_out, device=dev).bfloat16()
        res["ag_then_gemm_nccl"] = t(lambda: native.gemm_nt(raw_all_gather_rows(x, None), w))
        res["gemm_then_rs_nccl"] = t(lambda: raw_reduce_scatter_rows(native.gemm_nt(dy, wt), None))

        def fused_ag():
            heap.begin_step()
            return heap.linear_gather(x, w, None, want_gathered=True)

        def fused_rs():
            heap.begin_step()
            return heap.linear_scatter(dy, wt, None)
        res["ag_gemm_fused"], res["gemm_rs_fused"] = t(fused_ag), t(fused_rs)
        res["gemm_only"] = t(lambda: native.gemm_nt(full, w))
    # sparse: a random share of the block
    g = torch.Generator().manual_seed(100 + rank)
    need = torch.randperm(per * world, generator=g)[:max(int(args.share * per * world), 1)].sort().values.to(dev)
    dense = raw_all_gather_rows(x, None)
    plans = {"a2a": SparseRowPlan(None, per, need, "bench", "a2a")}
    if heap is not None:
        plans["pull"] = SparseRowPlan(None, per, need, "bench", "pull", heap)
    for name, plan in plans.items():
        def gat(plan=plan):
            if heap is not None:
                heap.begin_step()
            return plan.gather(x)

        def red(plan=plan, y=dense[need].contiguous()):
            if heap is not None:
                heap.begin_step()
            return plan.reduce_scatter(y)
        out = gat()
        assert torch.equal(out[:need.numel()], dense[need]), f"{name} gather differs from the dense result"
        res[f"sparse_gather_{name}"], res[f"sparse_reduce_{name}"] = t(gat), t(red)
    # one ring hop
    if world > 1:
        ring = RingComm(None)
        a, b = torch.empty_like(x), torch.empty_like(x)
        res["ring_hop_1buf"] = t(lambda: RingComm.wait(ring.hop([(x, a, +1)])))
        res["ring_hop_2buf"] = t(lambda: RingComm.wait(ring.hop([(x, a, +1), (x, b, -1)])))
    if rank == 0:
        for k, ms in res.items():
            nb = moved * (args.share if k.startswith("sparse") else 1.0) if not k.startswith("ring") else per * args.width * x.element_size()
            print("COLL " + json.dumps(dict(kind=k, world=world, rows=per * world, width=args.width, ms=ms, gbs_per_rank=nb / ms / 1e6 if ms else None)), flush=True)
        if res.get("sparse_gather_a2a") and res.get("ag_nccl"):
            print("A2A_OVER_AG " + json.dumps(dict(world=world, value=res["sparse_gather_a2a"] / args.share / res["ag_nccl"])), flush=True)
    return res


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        if dist.get_world_size() > 1:
            dist.barrier()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            os._exit(0)

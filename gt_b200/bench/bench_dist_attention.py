"""Attention-only operator benchmark across the distribution strategies, forward + backward of one layer's attention
(projections included), device time, max over ranks (counterpart of the reference's ``gt3d/bench/bench_dist_attention.py``).

    torchrun --nproc-per-node 4 -m gt_b200.bench.bench_dist_attention --grid 2 2 --strategy gather
    torchrun --nproc-per-node 8 -m gt_b200.bench.bench_dist_attention --grid 8 1 --strategy ring_kv2
    torchrun --nproc-per-node 8 -m gt_b200.bench.bench_dist_attention --grid 2 2 2 --strategy head

Strategies: ``gather`` (gather x over both groups, project on the gathered blocks, partial kernel, reduce-scatter — the
fused layer's operator), ``gather_proj`` (project on the owner, gather Q / K / V), ``ring_kv`` / ``ring_kv2`` (K | V
rotate around a (P, 1) ring, one or both directions), ``head`` (3D grid: all-to-all to head slices, head-slice gathers).
``--comm p2p`` moves the dense collectives to the peer-memory kernels; ``--sparse_comm`` moves only the rows the tile
references; ``--coll_timers`` prints the collective census of one iteration.  Prints one ``ATTN`` JSON line plus the
model's prediction for the same shape (``MODEL`` line).
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ._timing import time_ms


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--grid", type=int, nargs="+", default=None)
    ap.add_argument("--strategy", default="gather", choices=["gather", "gather_proj", "ring_kv", "ring_kv2", "head"])
    ap.add_argument("--graph", default="exphormer_arxiv")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--exp_deg", type=int, default=4)
    ap.add_argument("--comm", default="nccl", choices=["nccl", "p2p"])
    ap.add_argument("--heap_mb", type=int, default=2048)
    ap.add_argument("--sparse_comm", action="store_true")
    ap.add_argument("--coll_timers", action="store_true")
    ap.add_argument("--no_comm", action="store_true", help="(head, ring_kv*) skip the transfers: compute-only time, wrong values")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    from ..train.train_dist import init_dist
    init_dist()
    rank, world = dist.get_rank(), dist.get_world_size()
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    from ..data.expander import keyed_expander_edges
    from ..data.synthetic import workload_graph
    from ..models.exphormer_ref import ExphormerRef
    from ..ops import functional as K
    from ..parallel import attention as pa
    from ..parallel.collectives import all_gather_rows, set_transport
    from ..parallel.grid import make_grid
    from ..parallel.ring_kv import DistRingAttentionKV
    from ..parallel.sparse_comm import build_sparse_comm, sparse_all_gather
    from ..train.workloads import DEFAULT_GRIDS, pad_to
    shape = tuple(args.grid or DEFAULT_GRIDS[world])
    heap = None
    if args.comm == "p2p" and cuda and world > 1:
        from ..parallel.symm import SymmetricHeap
        heap = SymmetricHeap(dev, args.heap_mb << 20)
        set_transport(heap)
    wl = workload_graph(args.graph, seed=0, scale_down=args.scale_down)
    n = wl["n"]
    ei, et = ExphormerRef.build_attention_edges(wl["edge_index"], keyed_expander_edges(n, args.exp_deg, seed=0), None)
    grid = make_grid(shape, n, n_pad=pad_to(n, 8 * world)).to(dev)
    b_ei, b_et = grid.local_block(ei, et)
    b_ei, b_et = b_ei.to(dev), b_et.to(dev)
    d, h = args.hidden, args.heads
    dh = d // h
    dt = torch.bfloat16 if cuda else torch.float32
    backend = "cuda" if cuda else "torch"
    torch.manual_seed(0)
    x = torch.randn(grid.chunk, d, device=dev).to(dt).requires_grad_()
    wq, wk, wv = (torch.randn(d, d, device=dev).mul_(d ** -0.5).requires_grad_() for _ in range(3))
    gate = torch.randn(2, h, dh, device=dev).requires_grad_()
    wire = torch.bfloat16 if cuda else None
    sp = None
    block = pa.AttentionBlock(grid, b_ei, b_et)
    if args.sparse_comm and args.strategy in ("gather", "gather_proj"):
        sp, info = build_sparse_comm(grid, block, None, None, transport="pull" if heap is not None else "a2a", heap=heap)
        if rank == 0:
            print(f"[sparse_comm] row share {info['row_share']:.3f} col share {info['col_share']:.3f} -> "
                  f"{'sparse' if sp is not None else 'dense'}", flush=True)
        if sp is not None:
            block = sp["attn"]

    def gather(t, group, plan):
        return sparse_all_gather(t, plan, wire) if plan is not None else all_gather_rows(t, group, wire)

    if args.strategy in ("gather", "gather_proj"):
        op = pa.DistAttentionPartial(grid, block, h, dh, backend=backend)
        p_row, p_col = (sp["row"], sp["col"]) if sp is not None else (None, None)

        def fwd():
            if args.strategy == "gather":
                x_col, x_row = gather(x, grid.col_group, p_col), gather(x, grid.row_group, p_row)
                kv = K.linear(x_col, torch.cat([wk, wv], dim=0))
                q = K.linear(x_row, wq).view(-1, h, dh)
            else:
                q = gather(K.linear(x, wq), grid.row_group, p_row).view(-1, h, dh)
                kv = gather(K.linear(x, torch.cat([wk, wv], dim=0)), grid.col_group, p_col)
            k, v = kv[:, :d].contiguous().view(-1, h, dh), kv[:, d:].contiguous().view(-1, h, dh)
            acc, l, m = op(q, k, v, gate)
            o, _ = pa.combine_partials(acc, l, m, grid, "clampexp", 1e-6, rs_dtype=wire, plan=p_row)
            return o
    elif args.strategy == "head":
        op = pa.DistHeadSparseAttention(grid, block, h, dh, backend=backend, comm_dtype=wire, no_comm=args.no_comm)

        def fwd():
            q, k, v = (K.linear(x, w).view(-1, h, dh) for w in (wq, wk, wv))
            return op(q, k, v, gate)
    else:
        op = DistRingAttentionKV.from_block(grid, b_ei, b_et, h, dh, backend=backend, bidir=args.strategy == "ring_kv2", comm_dtype=wire,
                                            no_comm=args.no_comm)

        def fwd():
            q, k, v = (K.linear(x, w).view(-1, h, dh) for w in (wq, wk, wv))
            return op(q, k, v, gate)

    leaves = [x, wq, wk, wv, gate]

    def step():
        if heap is not None:
            heap.begin_step()
        o = fwd()
        go = torch.ones_like(o)
        torch.autograd.backward(o, go)
        for t in leaves:
            t.grad = None

    if cuda:
        ms = time_ms(step, args.iters, args.warmup, max_over_ranks=True)
    else:
        import time
        step()
        t0 = time.perf_counter()
        for _ in range(args.iters):
            step()
        ms = (time.perf_counter() - t0) / args.iters * 1e3
    if args.coll_timers:
        from ..utils.collstats import CollectiveStats
        cs = CollectiveStats()
        cs.begin_epoch(); step(); cs.end_epoch()
        cs.report()
    if rank == 0:
        from ..perf import grid_select as gs
        g = gs.Graph(n, int(ei.shape[1]), 0, d, exp_deg=args.exp_deg)
        m = gs.Model(d, h, 1, with_gcn=False, sparse_comm=args.sparse_comm, transport=args.comm)
        pd, po, pi = (shape + (1,))[:3]
        if args.strategy in ("gather", "gather_proj"):
            pred = gs.attn_operator_ms(pd, po, 1, g, m, "fused")
        elif args.strategy == "head":
            pred = gs.attn_operator_ms(pd, po, pi, g, m, "head")
        else:
            f, b = gs.ring_layer_ms(world, g, m)
            pred = f + b
        print("ATTN " + json.dumps(dict(strategy=args.strategy, grid=shape, world=world, nodes=n, edges=int(ei.shape[1]), hidden=d, heads=h,
                                        comm=args.comm, sparse_comm=bool(sp), ms_fwd_bwd=ms, timing="device_max_over_ranks")), flush=True)
        print("MODEL " + json.dumps(dict(predicted_ms=pred, ratio=ms / pred if pred else None)), flush=True)
    return ms


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        if dist.get_world_size() > 1:
            dist.barrier()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
            os._exit(0)

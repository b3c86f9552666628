"""Same model, same batch as TorchGT: time one training iteration (forward + backward + optimizer step) of the node-level
Graphormer (TorchGT's slim configuration: 4 layers, hidden 64, FFN 64, 8 heads) on TorchGT's batch construction:
``seq_len`` randomly drawn training nodes, the edges of the graph induced on them, and a global token (node 0) connected
to every node in both directions.  Counterpart of the reference's ``gt3d/bench/torchgt_batch_bench.py``; the graph is a
named synthetic workload (no dataset download).

    python -m gt_b200.bench.torchgt_batch_bench --graph exphormer_arxiv --seq_len 64000
    torchrun --nproc-per-node 4 -m gt_b200.bench.torchgt_batch_bench --graph unimp_products --seq_len 870000 --grid 2 2 --fused

Prints one ``RESULT`` JSON line: device time per iteration (CUDA events, maximum over ranks) and peak memory.
"""
import argparse
import json
import os
import time

import torch
import torch.distributed as dist


def torchgt_batch(x, y, edge_index, train_idx, seq_len, seed=0):
    """First batch of an epoch: shuffled training ids, induced sub-graph relabelled to ``1..n``, global token = node 0.
    Returns ``(x_batch, y_batch, edge_index over n + 1 nodes, n + 1)``."""
    g = torch.Generator().manual_seed(seed)
    idx = train_idx[torch.randperm(train_idx.numel(), generator=g)][:seq_len]
    n = idx.numel()
    new_id = torch.full((x.shape[0],), -1, dtype=torch.long)
    new_id[idx] = torch.arange(n)
    s, d = new_id[edge_index[0]], new_id[edge_index[1]]
    keep = (s >= 0) & (d >= 0)
    sub = torch.stack([s[keep], d[keep]]) + 1
    nodes, zero = torch.arange(1, n + 1), torch.zeros(n, dtype=torch.long)
    token = torch.cat([torch.stack([nodes, zero]), torch.stack([zero, nodes])], 1)
    return x[idx], y[idx], torch.cat([sub, token], 1), n + 1


def _parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--graph", default="exphormer_arxiv")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--seq_len", type=int, default=64000)
    ap.add_argument("--hidden", type=int, default=64)
    ap.add_argument("--ffn", type=int, default=64)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--grid", type=int, nargs=2, default=None)
    ap.add_argument("--fused", action="store_true", help="fused-communication blocks (gather LN(x) once, one reduce-scatter)")
    ap.add_argument("--comm_bf16", action="store_true")
    ap.add_argument("--rs_bf16", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    return ap


def _one_device_step(args, batch, num_classes, dev, backend):
    """Training iteration of the single-device model on the whole batch."""
    from ..models.graphormer_node import GraphormerNode
    xb, yb, eb, n = batch
    net = GraphormerNode(xb.shape[1], args.hidden, args.ffn, args.heads, args.layers, num_classes, eb, n, backend=backend).to(dev)
    feats, labels = xb.to(dev), yb.to(dev)
    optim = torch.optim.AdamW(net.parameters(), lr=1e-3)

    def iteration():
        torch.nn.functional.cross_entropy(net(feats).float(), labels).backward()
        optim.step()
        optim.zero_grad(set_to_none=True)
    return net, iteration


def _grid_step(args, batch, num_classes, dev, backend):
    """Training iteration of the 2D-distributed model: this rank's chunk of the batch (node 0 = the global token)."""
    from ..models.graphormer_node import DistGraphormerNode
    from ..parallel.grid import Grid2D
    from ..parallel.layers import allreduce_grads, dist_cross_entropy
    xb, yb, eb, n = batch
    grid = Grid2D(args.grid[0], args.grid[1], n).to(dev)
    tile_edges, _ = grid.local_block(eb)
    wire = torch.bfloat16 if args.comm_bf16 else None
    net = DistGraphormerNode(grid, (tile_edges.to(dev), None), xb.shape[1], args.hidden, args.ffn, args.heads, args.layers, num_classes,
                             backend=backend, comm_dtype=wire, fused=args.fused, rs_dtype=torch.bfloat16 if args.rs_bf16 else None).to(dev)
    weights = list(net.parameters())
    for w in weights:
        dist.broadcast(w.data, 0)
    token_row = torch.zeros(1, xb.shape[1])
    feats = grid.take_owned(torch.cat([token_row, xb])).to(dev)
    labels = grid.take_owned(torch.cat([torch.zeros(1, dtype=torch.long), yb])).to(dev)
    labelled = grid.valid_mask.clone()
    if grid.owned_range()[0] == 0:
        labelled[0] = False                                                   # the global token carries no label
    optim = torch.optim.AdamW(weights, lr=1e-3)

    def iteration():
        dist_cross_entropy(net(feats), labels, labelled, n - 1).backward()
        allreduce_grads(weights)
        optim.step()
        optim.zero_grad(set_to_none=True)
    return net, iteration


def _time_iterations(iteration, iters, dev):
    """``(ms per iteration, peak GB)``: CUDA events on a GPU, the host clock on the CPU; maximum over ranks."""
    if dev.type == "cuda":
        torch.cuda.synchronize(dev)
        torch.cuda.reset_peak_memory_stats(dev)
        if dist.is_initialized():
            dist.barrier()
        first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        first.record()
        for _ in range(iters):
            iteration()
        last.record()
        torch.cuda.synchronize(dev)
        ms, peak = first.elapsed_time(last) / iters, torch.cuda.max_memory_allocated(dev) / 2 ** 30
    else:
        began = time.perf_counter()
        for _ in range(iters):
            iteration()
        ms, peak = (time.perf_counter() - began) / iters * 1e3, 0.0
    if dist.is_initialized() and dist.get_world_size() > 1:
        both = torch.tensor([ms, peak], dtype=torch.float64, device=dev)
        dist.all_reduce(both, op=dist.ReduceOp.MAX)
        ms, peak = float(both[0]), float(both[1])
    return ms, peak


def main(argv=None):
    args = _parser().parse_args(argv)
    from ..data.synthetic import workload_graph
    on_gpu = args.device == "cuda"
    if args.grid is not None and not dist.is_initialized():
        dist.init_process_group("nccl" if on_gpu else "gloo")
    rank = dist.get_rank() if dist.is_initialized() else 0
    if on_gpu:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank % max(torch.cuda.device_count(), 1))))
        torch.cuda.set_device(dev)
    else:
        dev = torch.device("cpu")
    wl = workload_graph(args.graph, seed=0, scale_down=args.scale_down)
    batch = torchgt_batch(wl["x"], wl["y"], wl["edge_index"], wl["masks"]["train"].nonzero().view(-1), args.seq_len)
    torch.manual_seed(0)
    build = _one_device_step if args.grid is None else _grid_step
    net, iteration = build(args, batch, wl["num_classes"], dev, "cuda" if on_gpu else "torch")
    net.train()
    for _ in range(args.warmup):
        iteration()
    ms, peak = _time_iterations(iteration, args.iters, dev)
    n = batch[3]
    res = dict(graph=args.graph, batch_nodes=n - 1, edges=int(batch[2].shape[1]), token_edges=2 * (n - 1), layers=args.layers,
               hidden=args.hidden, ffn=args.ffn, heads=args.heads, grid=args.grid or [1, 1], fused=args.fused, iteration_ms=ms,
               epoch_s=2 * ms / 1e3, peak_gb=peak)
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    return res


if __name__ == "__main__":
    main()

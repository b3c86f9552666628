"""Baseline: the two distribution strategies of DAC'26 (Lin, Madduri, Kandemir, "Scalable and Adaptive Parallel Training
of Graph Transformer on Large Graphs") written with stock PyTorch operators only - no kernel of this package - so that
the package's 2D / 3D grids can be compared with the published 1D schemes on the same machine.  Counterpart of the
reference's ``baseline/dac26/dac26_sga.py`` (which uses DGL's sparse SDDMM / SpMM; DGL is not available here, the same
three steps are written as gather / segment-softmax / index_add on the edge list).

Sparse Graph Attention, paper Eq. 3-5:  Q, K, V = X W_Q, X W_K, X W_V;  Z = (Q K^T) . A (SDDMM);  U = row-softmax(Z /
sqrt(d'));  Y = U V (SpMM);  X' = X W_o + Y.

Strategies (contiguous row ranges per rank):
  single  one process, no communication.
  gp_ag   paper Alg. 1: project the N/p owned rows; all-gather K and V (2 gathers forward, 2 reduce-scatters backward);
          attention over the local N/p x N block of A for all heads.
  gp_a2a  paper Alg. 2: all-to-all of Q, K, V from node to head partitioning ([N/p, h, d'] -> [N, h/p, d']); attention
          over the whole graph for h/p heads; all-to-all back (4 forward, 4 backward); needs p | h.
Weights are replicated; one flat gradient all-reduce per iteration.

    python baseline/dac26/dac26_sga.py --graph cpu_small --strategy single
    torchrun --nproc-per-node 4 baseline/dac26/dac26_sga.py --graph exphormer_arxiv --strategy gp_a2a
    python baseline/dac26/dac26_sga.py --graph exphormer_arxiv --micro        (MM / SpMM / SDDMM on one device)

Prints one RESULT line per run (device-timed on GPUs, max over ranks).
"""
import argparse
import json
import math
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


# ---- collectives with autograd ----------------------------------------------------------------------------------------------
class AllGatherRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        p = dist.get_world_size()
        out = x.new_empty((p * x.shape[0],) + tuple(x.shape[1:]))
        dist.all_gather_into_tensor(out, x.contiguous())
        return out

    @staticmethod
    def backward(ctx, g):
        p = dist.get_world_size()
        out = g.new_empty((g.shape[0] // p,) + tuple(g.shape[1:]))
        if dist.get_backend() == "gloo":
            full = g.contiguous().clone()
            dist.all_reduce(full)
            out.copy_(full[dist.get_rank() * out.shape[0]:(dist.get_rank() + 1) * out.shape[0]])
        else:
            dist.reduce_scatter_tensor(out, g.contiguous())
        return out


def _a2a(x):
    out = torch.empty_like(x)
    dist.all_to_all_single(out, x.contiguous())
    return out


class RowsToHeads(torch.autograd.Function):
    """[n, h, d] (my rows, all heads) -> [p n, h / p, d] (all rows, my heads)."""

    @staticmethod
    def forward(ctx, x):
        p = dist.get_world_size()
        n, h, d = x.shape
        send = x.view(n, p, h // p, d).permute(1, 0, 2, 3).contiguous()          # [p, n, h/p, d]: block j goes to rank j
        return _a2a(send).view(p * n, h // p, d)

    @staticmethod
    def backward(ctx, g):
        p = dist.get_world_size()
        pn, hp, d = g.shape
        back = _a2a(g.contiguous().view(p, pn // p, hp, d))                       # block j: my rows' gradient for rank j's heads
        return back.permute(1, 0, 2, 3).reshape(pn // p, p * hp, d)


class HeadsToRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y):
        p = dist.get_world_size()
        pn, hp, d = y.shape
        back = _a2a(y.contiguous().view(p, pn // p, hp, d))
        return back.permute(1, 0, 2, 3).reshape(pn // p, p * hp, d)

    @staticmethod
    def backward(ctx, g):
        p = dist.get_world_size()
        n, h, d = g.shape
        send = g.view(n, p, h // p, d).permute(1, 0, 2, 3).contiguous()
        return _a2a(send).view(p * n, h // p, d)


# ---- the operator with library ops ------------------------------------------------------------------------------------------
def sga(q, k, v, src, dst, n_rows):
    """Row-softmax attention over the edges (src -> dst): SDDMM, segment softmax, SpMM with stock PyTorch ops."""
    d = q.shape[-1]
    z = (q[dst] * k[src]).sum(-1) / math.sqrt(d)                                   # SDDMM  [E, h]
    zmax = torch.full((n_rows, z.shape[1]), float("-inf"), dtype=z.dtype, device=z.device)
    zmax = zmax.scatter_reduce(0, dst.unsqueeze(-1).expand_as(z), z, reduce="amax")
    e = torch.exp(z - zmax[dst])
    den = torch.zeros_like(zmax).index_add_(0, dst, e)
    u = e / den[dst]
    return torch.zeros(n_rows, q.shape[1], d, dtype=q.dtype, device=q.device).index_add_(0, dst, u.unsqueeze(-1) * v[src])   # SpMM


class SGALayer(torch.nn.Module):
    def __init__(self, d, h, strategy):
        super().__init__()
        self.h, self.strategy = h, strategy
        self.wq, self.wk, self.wv, self.wo = (torch.nn.Linear(d, d, bias=False) for _ in range(4))

    def forward(self, graph, x):
        n, h = x.shape[0], self.h
        q, k, v = (w(x).view(n, h, -1) for w in (self.wq, self.wk, self.wv))
        src, dst, n_rows = graph
        if self.strategy == "gp_ag":
            y = sga(q, AllGatherRows.apply(k), AllGatherRows.apply(v), src, dst, n)
        elif self.strategy == "gp_a2a":
            y = HeadsToRows.apply(sga(RowsToHeads.apply(q), RowsToHeads.apply(k), RowsToHeads.apply(v), src, dst, n_rows))
        else:
            y = sga(q, k, v, src, dst, n)
        return self.wo(x) + y.reshape(n, -1)


class SGAModel(torch.nn.Module):
    def __init__(self, f_in, d, h, layers, classes, strategy):
        super().__init__()
        self.inp = torch.nn.Linear(f_in, d)
        self.layers = torch.nn.ModuleList([SGALayer(d, h, strategy) for _ in range(layers)])
        self.out = torch.nn.Linear(d, classes)

    def forward(self, graph, x):
        x = self.inp(x)
        for layer in self.layers:
            x = F.relu(layer(graph, x))
        return self.out(x)


def local_graph(n_pad, ei, strategy, rank, p, dev):
    """Edge list of the rank's block: gp_ag keeps the edges into its rows (dst made local); the others keep everything."""
    src, dst = ei[0], ei[1]
    if strategy == "gp_ag":
        per = n_pad // p
        keep = (dst >= rank * per) & (dst < (rank + 1) * per)
        return src[keep].to(dev), (dst[keep] - rank * per).to(dev), per
    return src.to(dev), dst.to(dev), n_pad


def timed(fn, iters, warmup, dev):
    for _ in range(warmup):
        fn()
    if dev.type == "cuda":
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        b.synchronize()
        ms = a.elapsed_time(b) / iters
    else:
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        ms = (time.perf_counter() - t0) / iters * 1e3
    if dist.is_initialized() and dist.get_world_size() > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--graph", default="cpu_small", help="synthetic workload name (gt_b200.data.synthetic.WORKLOADS)")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--graph_file", default=None, help="graph written by prepare_graphs.py (random features and labels)")
    ap.add_argument("--strategy", default="single", choices=["single", "gp_ag", "gp_a2a"])
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--micro", action="store_true", help="MM / SpMM / SDDMM on one device")
    ap.add_argument("--kernel", action="store_true", help="one attention forward + backward on the whole graph, one device")
    args = ap.parse_args(argv)
    from gt_b200.data.synthetic import add_self_loops, workload_graph
    cuda = torch.cuda.is_available()
    multi = "RANK" in os.environ or dist.is_initialized()
    if multi and not dist.is_initialized():
        if cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if cuda else "gloo")
    rank, p = (dist.get_rank(), dist.get_world_size()) if multi else (0, 1)
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    if args.strategy == "single" and p > 1:
        raise SystemExit("--strategy single runs as one process")
    if args.strategy == "gp_a2a" and args.heads % p:
        raise SystemExit("gp_a2a needs the number of ranks to divide the number of heads")
    if args.graph_file:
        from gt_b200.data.synthetic import node_data
        g = torch.load(args.graph_file, weights_only=True)
        x_, y_, masks_ = node_data(g["num_nodes"], 128, 40, seed=args.seed + 17)
        wl = dict(n=g["num_nodes"], edge_index=g["edge_index"], x=x_, y=y_, masks=masks_, cfg=dict(features=128, classes=40))
        args.graph = os.path.basename(args.graph_file)
    else:
        wl = workload_graph(args.graph, seed=args.seed, scale_down=args.scale_down)
    n, ei = wl["n"], add_self_loops(wl["edge_index"], wl["n"])
    n_pad = -(-n // p) * p
    per = n_pad // p
    graph = local_graph(n_pad, ei, args.strategy, rank, p, dev)
    torch.manual_seed(args.seed)
    d, h = args.hidden, args.heads
    res = dict(graph=args.graph, nodes=n, edges=int(ei.shape[1]), strategy=args.strategy, world=p, hidden=d, heads=h)
    if args.micro or args.kernel:
        q, k, v = (torch.randn(n, h, d // h, device=dev, requires_grad=True) for _ in range(3))
        src, dst = ei[0].to(dev), ei[1].to(dev)
        if args.micro:
            x, w = torch.randn(n, d, device=dev), torch.randn(d, d, device=dev)
            res["mm_ms"] = timed(lambda: x @ w, args.iters, args.warmup, dev)
            res["sddmm_ms"] = timed(lambda: (q[dst] * k[src]).sum(-1), args.iters, args.warmup, dev)
            u = torch.rand(ei.shape[1], h, device=dev)
            res["spmm_ms"] = timed(lambda: torch.zeros(n, h, d // h, device=dev).index_add_(0, dst, u.unsqueeze(-1) * v[src]),
                                   args.iters, args.warmup, dev)
        else:
            def fb():
                y = sga(q, k, v, src, dst, n)
                y.backward(torch.ones_like(y))
                q.grad = k.grad = v.grad = None
            res["fwd_ms"] = timed(lambda: sga(q, k, v, src, dst, n), args.iters, args.warmup, dev)
            res["fwd_bwd_ms"] = timed(fb, args.iters, args.warmup, dev)
    else:
        cfg = wl["cfg"]
        model = SGAModel(cfg["features"], d, h, args.layers, cfg["classes"], args.strategy).to(dev)
        if p > 1:
            for prm in model.parameters():
                dist.broadcast(prm.data, src=0)
        x = torch.zeros(n_pad, cfg["features"]); x[:n] = wl["x"]
        y = torch.zeros(n_pad, dtype=torch.long); y[:n] = wl["y"]
        m = torch.zeros(n_pad, dtype=torch.bool); m[:n] = wl["masks"]["train"]
        sl = slice(rank * per, (rank + 1) * per)
        x_loc, y_loc, m_loc = x[sl].to(dev), y[sl].to(dev), m[sl].to(dev)
        n_train = int(m.sum())
        opt = torch.optim.Adam(model.parameters(), lr=1e-3)
        losses = []

        def step():
            opt.zero_grad(set_to_none=True)
            logits = model(graph, x_loc)
            loss = F.cross_entropy(logits[m_loc], y_loc[m_loc], reduction="sum") / n_train
            loss.backward()
            if p > 1:
                flat = torch.cat([prm.grad.reshape(-1) for prm in model.parameters()])
                dist.all_reduce(flat)
                off = 0
                for prm in model.parameters():
                    prm.grad.copy_(flat[off:off + prm.numel()].view_as(prm))
                    off += prm.numel()
            opt.step()
            losses.append(loss.detach())
        res["iter_ms"] = timed(step, args.iters, args.warmup, dev)
        tot = torch.stack(losses[-1:]).sum()
        if p > 1:
            dist.all_reduce(tot)
        res["loss"] = float(tot)
        first = losses[0].clone()
        if p > 1:
            dist.all_reduce(first)
        res["first_loss"] = float(first)
    if rank == 0:
        print("RESULT " + json.dumps(res), flush=True)
    return res


if __name__ == "__main__":
    main()

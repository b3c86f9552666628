"""Single-process full-graph Exphormer training with a selectable attention back-end (``ref`` / ``torch`` / ``cuda``).

The recipe is the GraphGPS Exphormer one the reference reproduces (``gt3d/gt3d/train/train_single_gpu.py:1-10,59-115``):
reverse edges + self loops, degree-3 expander (type-1 edges), GCN + Exphormer x 4, hidden 80, 2 heads, dropout 0.3,
BatchNorm, AdamW lr 1e-3 wd 1e-3, cosine schedule with 5 warm-up epochs, gradient-norm clip 1.0, cross-entropy on the
train split, test accuracy reported at the best validation epoch.

    python -m gt_b200.train.train_single_gpu --backend cuda --epochs 600 --graph arxiv.pt
    python -m gt_b200.train.train_single_gpu --synthetic exphormer_arxiv --epochs 20

``--graph FILE`` is a ``torch.save``d dict ``{x [N,F], y [N], edge_index [2,E] (one direction), train_idx, valid_idx,
test_idx}`` (what ``ogb``'s ``PygNodePropPredDataset`` yields; no dataset download happens here).  This path uses stock
``torch.optim.AdamW`` and the module-level ops, so it doubles as the plain-PyTorch baseline of the distributed engine.
"""
import argparse
import time

import torch
import torch.nn.functional as F

from ..data.expander import random_regular_expander_edges
from ..data.synthetic import add_self_loops, symmetrize, workload_graph
from ..models.exphormer import AttentionGraph, Exphormer
from .engine import cosine_with_warmup


def load_graph_file(path, device, self_loops=True):
    blob = torch.load(path, map_location="cpu", weights_only=False)
    n = blob["x"].shape[0]
    ei = symmetrize(blob["edge_index"].long(), n)
    if self_loops:
        ei = add_self_loops(ei, n)
    split = {k: blob[f"{k}_idx"].long().to(device) for k in ("train", "valid", "test")}
    y = blob["y"].view(-1).long()
    return n, blob["x"].float().to(device), y.to(device), ei.to(device), split, int(y.max()) + 1


def load_synthetic(name, device, seed=0, scale_down=1, self_loops=True):
    wl = workload_graph(name, seed=seed, scale_down=scale_down)
    n, ei = wl["n"], wl["edge_index"]
    if self_loops:
        ei = add_self_loops(ei, n)
    split = {k: wl["masks"][k].nonzero().view(-1).to(device) for k in ("train", "valid", "test")}
    return n, wl["x"].to(device), wl["y"].to(device), ei.to(device), split, wl["cfg"]["classes"]


@torch.no_grad()
def evaluate(model, x, graph, y, split):
    model.eval()
    pred = model(x, graph).argmax(-1)
    return {k: (pred[idx] == y[idx]).float().mean().item() for k, idx in split.items()}


def build_parser():
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    a = ap.add_argument
    a("--backend", default=None, choices=["ref", "torch", "cuda", "triton"], help="'triton' is an alias of 'cuda'")
    a("--graph", default=None)
    a("--synthetic", default="cpu_small")
    a("--scale_down", type=int, default=1)
    a("--no_self_loops", action="store_true")
    a("--exp_deg", type=int, default=3)
    a("--seed", type=int, default=0)
    for flag, kind, value in (("--hidden", int, 80), ("--heads", int, 2), ("--layers", int, 4), ("--dropout", float, 0.3),
                              ("--epochs", int, 600), ("--warmup", int, 5), ("--lr", float, 1e-3), ("--weight_decay", float, 1e-3),
                              ("--eval_every", int, 1)):
        a(flag, type=kind, default=value)
    a("--norm", default="bn", choices=["bn", "ln", "rms"])
    return ap


class _Stopwatch:
    """Accumulates seconds per phase; synchronises the device at both ends of a phase so that the host clock brackets the
    device work of exactly that phase."""

    def __init__(self, cuda):
        self.cuda, self.total = cuda, {}

    def run(self, phase, fn):
        if self.cuda:
            torch.cuda.synchronize()
        began = time.perf_counter()
        out = fn()
        if self.cuda:
            torch.cuda.synchronize()
        self.total[phase] = self.total.get(phase, 0.0) + time.perf_counter() - began
        return out


def train_epoch(model, opt, sched, x, graph, y, train_idx, clip=1.0):
    """One full-graph step: loss on the train split, clipped gradients, AdamW and schedule step.  Returns the loss tensor."""
    model.train()
    opt.zero_grad(set_to_none=True)
    loss = F.cross_entropy(model(x, graph)[train_idx], y[train_idx])
    loss.backward()
    torch.nn.utils.clip_grad_norm_(model.parameters(), clip)
    opt.step()
    sched.step()
    return loss


def main(argv=None):
    args = build_parser().parse_args(argv)
    torch.manual_seed(args.seed)
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda" if cuda else "cpu")
    backend = args.backend or ("cuda" if cuda else "torch")
    backend = "cuda" if backend == "triton" else backend
    loops = not args.no_self_loops
    data = load_graph_file(args.graph, dev, loops) if args.graph else load_synthetic(args.synthetic, dev, args.seed, args.scale_down, loops)
    n, x, y, ei, split, classes = data
    graph = AttentionGraph(ei, random_regular_expander_edges(n, args.exp_deg, seed=args.seed, device=dev), n).to(dev)
    print(f"graph: N={n} E_gcn={ei.shape[1]} E_attn={graph.edge_index.shape[1]} classes={classes} backend={backend}", flush=True)
    model = Exphormer(x.shape[1], args.hidden, classes, args.layers, args.heads, dropout=args.dropout, gnn_dropout=args.dropout,
                      backend=backend, norm=args.norm).to(dev)
    print(f"params: {sum(p.numel() for p in model.parameters())}", flush=True)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=args.weight_decay)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: cosine_with_warmup(s, args.warmup, args.epochs))
    watch = _Stopwatch(cuda)
    best = dict(val=-1.0, test=0.0, epoch=-1)
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    last = args.epochs - 1
    for epoch in range(args.epochs):
        loss = watch.run("train", lambda: train_epoch(model, opt, sched, x, graph, y, split["train"]))
        if epoch % args.eval_every and epoch != last:
            continue
        acc = watch.run("eval", lambda: evaluate(model, x, graph, y, split))
        if acc["valid"] > best["val"]:
            best = dict(val=acc["valid"], test=acc["test"], epoch=epoch)
        if epoch % 10 == 0 or epoch == last:
            print(f"epoch {epoch:4d} loss {loss.item():.4f} train {acc['train']:.4f} val {acc['valid']:.4f} test {acc['test']:.4f} "
                  f"| best val {best['val']:.4f} test {best['test']:.4f} @ {best['epoch']} | "
                  f"{watch.total['train'] / (epoch + 1) * 1e3:.1f} ms/epoch train, lr {sched.get_last_lr()[0]:.2e}", flush=True)
    t_train, t_eval = watch.total.get("train", 0.0), watch.total.get("eval", 0.0)
    peak = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0
    print(f"FINAL backend={backend} best_val={best['val']:.4f} test@best_val={best['test']:.4f} epoch={best['epoch']} "
          f"train_time={t_train:.1f}s ({t_train / max(args.epochs, 1) * 1e3:.1f} ms/epoch) eval_time={t_eval:.1f}s peak_mem={peak:.2f}GB", flush=True)
    return best


if __name__ == "__main__":
    main()

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


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--backend", default=None, choices=["ref", "torch", "cuda", "triton"], help="'triton' is an alias of 'cuda'")
    ap.add_argument("--graph", default=None)
    ap.add_argument("--synthetic", default="cpu_small")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--epochs", type=int, default=600)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--hidden", type=int, default=80)
    ap.add_argument("--heads", type=int, default=2)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--dropout", type=float, default=0.3)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--weight_decay", type=float, default=1e-3)
    ap.add_argument("--exp_deg", type=int, default=3)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--eval_every", type=int, default=1)
    ap.add_argument("--norm", default="bn", choices=["bn", "ln", "rms"])
    ap.add_argument("--no_self_loops", action="store_true")
    args = ap.parse_args(argv)
    torch.manual_seed(args.seed)
    cuda = torch.cuda.is_available()
    dev = torch.device("cuda" if cuda else "cpu")
    backend = {"triton": "cuda", None: "cuda" if cuda else "torch"}.get(args.backend, args.backend)
    if args.graph:
        n, x, y, ei, split, classes = load_graph_file(args.graph, dev, not args.no_self_loops)
    else:
        n, x, y, ei, split, classes = load_synthetic(args.synthetic, dev, args.seed, args.scale_down, not args.no_self_loops)
    exp = random_regular_expander_edges(n, args.exp_deg, seed=args.seed, device=dev)
    graph = AttentionGraph(ei, exp, n).to(dev)
    print(f"graph: N={n} E_gcn={ei.shape[1]} E_attn={graph.edge_index.shape[1]} classes={classes} backend={backend}", flush=True)
    model = Exphormer(x.shape[1], args.hidden, classes, args.layers, args.heads, dropout=args.dropout, gnn_dropout=args.dropout,
                      backend=backend, norm=args.norm).to(dev)
    print(f"params: {sum(p.numel() for p in model.parameters())}", flush=True)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=args.weight_decay)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: cosine_with_warmup(s, args.warmup, args.epochs))

    def sync():
        if cuda:
            torch.cuda.synchronize()
    best = dict(val=-1.0, test=0.0, epoch=-1)
    t_train = t_eval = 0.0
    if cuda:
        torch.cuda.reset_peak_memory_stats()
    for epoch in range(args.epochs):
        sync(); t0 = time.perf_counter()
        model.train()
        opt.zero_grad(set_to_none=True)
        loss = F.cross_entropy(model(x, graph)[split["train"]], y[split["train"]])
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        sched.step()
        sync(); t1 = time.perf_counter(); t_train += t1 - t0
        if epoch % args.eval_every == 0 or epoch == args.epochs - 1:
            acc = evaluate(model, x, graph, y, split)
            sync(); t_eval += time.perf_counter() - t1
            if acc["valid"] > best["val"]:
                best = dict(val=acc["valid"], test=acc["test"], epoch=epoch)
            if epoch % 10 == 0 or epoch == args.epochs - 1:
                print(f"epoch {epoch:4d} loss {loss.item():.4f} train {acc['train']:.4f} val {acc['valid']:.4f} test {acc['test']:.4f} "
                      f"| best val {best['val']:.4f} test {best['test']:.4f} @ {best['epoch']} | {t_train / (epoch + 1) * 1e3:.1f} ms/epoch train, "
                      f"lr {sched.get_last_lr()[0]:.2e}", flush=True)
    peak = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0
    print(f"FINAL backend={backend} best_val={best['val']:.4f} test@best_val={best['test']:.4f} epoch={best['epoch']} "
          f"train_time={t_train:.1f}s ({t_train / max(args.epochs, 1) * 1e3:.1f} ms/epoch) eval_time={t_eval:.1f}s peak_mem={peak:.2f}GB", flush=True)
    return best


if __name__ == "__main__":
    main()

"""Locality factor of a graph for the performance model: time of the attention and SpMM kernels on the graph's real block
over their time on a uniformly random block of the same shape (rows, columns, edges).  Power-law graphs with hubs and a global
token gather less uniformly than a random block, which the model's linear constants (fitted on random blocks by
``kernel_constants``) do not see; the ratio is the ``skew`` field of ``gt_b200.perf.grid_select.Graph``.  Counterpart of the
reference's ``gt3d/bench/graph_constants.py:115-149``.

    python -m gt_b200.bench.graph_constants --graph exphormer_arxiv --out graph_constants_exphormer_arxiv.json
"""
import argparse
import json

import torch

from ._timing import time_ms


def measure(blk, n_rows, n_cols, h, d, dev, iters):
    from ..attention import backend_cuda as bc
    from ..ops import native
    q = torch.randn(n_rows, h, d, device=dev).bfloat16()
    k, v = (torch.randn(n_cols, h, d, device=dev).bfloat16() for _ in range(2))
    gate = torch.randn(3, h, d, device=dev)
    kw = dict(score="gated", norm="clampexp")
    acc, l, m = bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw)
    dacc, dl = torch.randn_like(acc), torch.randn_like(l)
    f = time_ms(lambda: bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw), iters, 3)
    b = time_ms(lambda: bc.attn_bwd_partial(q, k, v, blk, gate, None, m, dacc, dl, **kw), iters, 3)
    return f, b


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--graph", default="exphormer_arxiv")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--exp_deg", type=int, default=4)
    ap.add_argument("--no_token", action="store_true")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from ..attention import BlockCSR
    from ..data.expander import keyed_expander_edges
    from ..data.synthetic import virtual_node_edges, workload_graph
    from ..models.exphormer_ref import ExphormerRef
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    wl = workload_graph(args.graph, seed=0, scale_down=args.scale_down)
    n = wl["n"]
    tok = None if args.no_token else virtual_node_edges(n)[0]
    ei, et = ExphormerRef.build_attention_edges(wl["edge_index"], keyed_expander_edges(n, args.exp_deg, seed=0), tok)
    n_tot = n + (0 if args.no_token else 1)
    real = BlockCSR.from_edges(ei, n_tot, n_tot, et).to(dev)
    g = torch.Generator().manual_seed(1)
    e = int(ei.shape[1])
    rnd = BlockCSR.from_edges(torch.randint(0, n_tot, (2, e), generator=g), n_tot, n_tot, torch.randint(0, 3, (e,), generator=g)).to(dev)
    f_real, b_real = measure(real, n_tot, n_tot, args.heads, args.head_dim, dev, args.iters)
    f_rnd, b_rnd = measure(rnd, n_tot, n_tot, args.heads, args.head_dim, dev, args.iters)
    out = dict(graph=args.graph, nodes=n_tot, edges=e, heads=args.heads, head_dim=args.head_dim, fwd_ms=f_real, bwd_ms=b_real,
               fwd_ms_random=f_rnd, bwd_ms_random=b_rnd, skew_fwd=f_real / f_rnd, skew_bwd=b_real / b_rnd,
               skew=(f_real + b_real) / (f_rnd + b_rnd))
    print("GRAPH " + json.dumps(out), flush=True)
    if args.out:
        with open(args.out, "w") as fh:
            json.dump(out, fh, indent=1)
    return out


if __name__ == "__main__":
    main()

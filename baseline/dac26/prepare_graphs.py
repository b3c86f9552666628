"""Write the three graphs of the DAC'26 evaluation as plain tensor files ``{"num_nodes": int, "edge_index": int64 [2, E]}``
for ``dac26_sga.py --graph_file`` (counterpart of the reference's ``baseline/dac26/prepare_graphs.py``, which extracts
ogbn-proteins, ogbn-products and Reddit from dataset copies).  No dataset can be downloaded here, so each graph is either

  * converted from an edge list the user supplies (``--edges FILE``: a ``.pt`` tensor / dict or a ``.npy`` array ``[2, E]``), or
  * a seeded Chung-Lu stand-in with the node and (directed) edge counts of the paper's Table 2:
    proteins 132,534 / 79.1M, products 2,449,029 / 123.7M, Reddit 232,965 / 114.6M  (``--scale_down`` divides both).

    python baseline/dac26/prepare_graphs.py --out graphs --scale_down 16
    python baseline/dac26/prepare_graphs.py --out graphs --name mygraph --edges my_edge_index.pt
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

SHAPES = {"proteins": (132_534, 79_122_504), "products": (2_449_029, 123_718_280), "reddit": (232_965, 114_615_892)}


def stand_in(name, scale_down=1, seed=0):
    from gt_b200.data.synthetic import chung_lu, symmetrize
    n, e = SHAPES[name]
    n, e = max(n // scale_down, 64), max(e // scale_down, 128)
    return n, symmetrize(chung_lu(n, e // 2, 2.1, seed), n)


def from_file(path):
    if path.endswith(".npy"):
        import numpy as np
        ei = torch.from_numpy(np.load(path)).long()
        return int(ei.max()) + 1, ei
    obj = torch.load(path, weights_only=True)
    if isinstance(obj, dict):
        return int(obj.get("num_nodes", int(obj["edge_index"].max()) + 1)), obj["edge_index"].long()
    return int(obj.max()) + 1, obj.long()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", default="graphs")
    ap.add_argument("--graphs", nargs="+", default=sorted(SHAPES), choices=sorted(SHAPES))
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--name", default=None, help="with --edges: name of the output file")
    ap.add_argument("--edges", default=None)
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    jobs = [(args.name or "graph", lambda: from_file(args.edges))] if args.edges else \
        [(g, lambda g=g: stand_in(g, args.scale_down)) for g in args.graphs]
    written = []
    for name, make in jobs:
        n, ei = make()
        if ei.dim() != 2 or ei.shape[0] != 2 or int(ei.min()) < 0 or int(ei.max()) >= n:
            raise SystemExit(f"{name}: edge_index must be [2, E] with ids in [0, {n})")
        path = os.path.join(args.out, f"{name}.pt")
        torch.save({"num_nodes": n, "edge_index": ei.contiguous()}, path)
        print(f"{name}: {n} nodes, {ei.shape[1]} directed edges -> {path}", flush=True)
        written.append(path)
    return written


if __name__ == "__main__":
    main()

"""How much of an attention mask lies in dense 128 x 128 tiles, under several node orders (CPU study, no process group).

The tensor-core tile kernel (``csrc/attn_tile.cu``) pays where a tile of the mask holds more than about a tenth of its entries;
everything else stays on the gather kernels.  This tool counts, for a named workload, the edges per tile of the attention mask
(graph edges + self loops, optionally expander edges, a global token, the sampled 2-hop mask) and reports per node order

  * the share of edges in tiles with at least ``--min_edges`` entries and the number of such tiles (what the density dispatch
    of ``gt_b200.attention.tiles`` would hand to the tile kernel),
  * the number of non-empty tiles and the mean edges per non-empty tile.

Node orders: ``native`` (generator ids), ``random``, ``bfs`` (reverse Cuthill-McKee) and ``degree`` (descending degree: hubs first).

    python -m gt_b200.bench.tile_density --graph exphormer_arxiv
    python -m gt_b200.bench.tile_density --graph graphormer_rmat --scale_down 8 --khop --exp_degree 0 --no_token

Prints one ``TILE_DENSITY`` JSON line per order and returns the list of result dicts.
"""
import argparse
import json

import torch

from .comm_sparsity import attention_edges, reorder

TILE = 128


def degree_order(edge_index, n):
    """Relabel nodes by descending in-degree + out-degree (ties by old id)."""
    deg = torch.bincount(edge_index[0], minlength=n) + torch.bincount(edge_index[1], minlength=n)
    old = torch.argsort(deg, descending=True, stable=True)          # position -> old id
    perm = torch.empty(n, dtype=torch.long)
    perm[old] = torch.arange(n)
    return perm[edge_index]


def tile_stats(edge_index, n, min_edges):
    """Edges per (destination tile, source tile) of an ``n x n`` mask."""
    n_t = -(-n // TILE)
    key = (edge_index[1] // TILE) * n_t + edge_index[0] // TILE
    cnt = torch.unique(key, return_counts=True)[1]
    dense = cnt >= min_edges
    e = int(edge_index.shape[1])
    return dict(edges=e, tiles_nonempty=int(cnt.numel()), tiles_total=n_t * n_t, mean_edges_per_nonempty_tile=round(e / max(int(cnt.numel()), 1), 2),
                max_edges_in_a_tile=int(cnt.max()) if cnt.numel() else 0, dense_tiles=int(dense.sum()),
                dense_edge_share=round(float(cnt[dense].sum()) / max(e, 1), 5))


def survey(wl_edges, n, orders=("native", "random", "bfs", "degree"), exp_degree=4, token=True, khop=False, max_two_hop=64, min_edges=1638, seed=0):
    if khop:
        from ..models.gt_variants import khop_typed_edges
        att, _ = khop_typed_edges(wl_edges, n, max_two_hop=max_two_hop, seed=seed)
        n_tot = n
    else:
        att, n_tot = attention_edges(wl_edges, n, exp_degree, token, seed)
    out = []
    for order in orders:
        ei = degree_order(att, n_tot) if order == "degree" else reorder(att, n_tot, order, seed)
        out.append(dict(order=order, nodes=n_tot, min_edges=min_edges, **tile_stats(ei, n_tot, min_edges)))
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--graph", default="exphormer_arxiv")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--orders", nargs="+", default=["native", "random", "bfs", "degree"])
    ap.add_argument("--exp_degree", type=int, default=4)
    ap.add_argument("--no_token", action="store_true")
    ap.add_argument("--khop", action="store_true", help="the sampled 2-hop mask of the Graphormer workload instead of graph + expander edges")
    ap.add_argument("--max_two_hop", type=int, default=64)
    ap.add_argument("--min_edges", type=int, default=1638, help="entries a tile must hold to count as dense (default: 10 %% of 128 x 128)")
    args = ap.parse_args(argv)
    from ..data.synthetic import workload_graph
    wl = workload_graph(args.graph, seed=0, scale_down=args.scale_down)
    res = survey(wl["edge_index"], wl["n"], args.orders, args.exp_degree, not args.no_token, args.khop, args.max_two_hop, args.min_edges)
    for r in res:
        print("TILE_DENSITY " + json.dumps(dict(graph=args.graph, scale_down=args.scale_down, **r)), flush=True)
    return res


if __name__ == "__main__":
    main()

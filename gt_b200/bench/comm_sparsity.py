"""Communication sparsity of the gather layouts, counted on the CPU: which rows of a gathered block does a rank's tile
actually reference?  (Counterpart of the reference's ``gt3d/bench/comm_sparsity.py``; the numbers decide where the
sparse collectives of ``gt_b200.parallel.sparse_comm`` can pay.)

Rank ``(r, c)`` of a ``P_d x P_o`` grid computes the tile ``A[row block r, column block c]``.  A source row of the column
block that no edge of the tile touches need not be received (K / V-side gather) and receives no gradient (dx
reduce-scatter); a destination row with no edge in the tile need not be received (Q-side gather) and its partial
``(acc, l)`` is zero.  Reported per grid, over the part of each block the rank does not own itself:

  ``col_need`` / ``row_need``  mean and maximum over tiles of the referenced share of the non-owned rows,
  ``ring_need``                for the ``(P, 1)`` ring: share of a chunk that some OTHER rank references (what a hop carries),
  ``balance``                  edges of the fullest tile over the mean tile (what a locality-preserving order costs).

Three node orders: ``native`` (the generator's ids), ``random`` (a permutation: a partition without locality) and
``bfs`` (reverse Cuthill-McKee on the graph edges: a locality-preserving order).  Expander edges are generated after the
reordering (they are keyed on the final ids, as in training); the virtual node keeps the last id.

    python -m gt_b200.bench.comm_sparsity --graph exphormer_arxiv --grids 2x1 2x2 2x4 8x1 --out comm_sparsity_arxiv.json
"""
import argparse
import json

import torch


def attention_edges(wl_edges, n, exp_degree, token, seed=0):
    """Graph edges + self loops + expander edges (+ both directions to a virtual node ``n``) as one ``[2, E]`` tensor."""
    from ..data.expander import keyed_expander_edges
    from ..data.synthetic import add_self_loops, unique_edges, virtual_node_edges
    parts = [add_self_loops(wl_edges, n)]
    if exp_degree > 0:
        parts.append(keyed_expander_edges(n, exp_degree, seed=seed))
    n_tot = n
    if token:
        parts.append(virtual_node_edges(n)[0])
        n_tot = n + 1
    return unique_edges(torch.cat(parts, 1), n_tot), n_tot


def reorder(edge_index, n, order, seed=0):
    """Relabel node ids ``[0, n)``: ``native`` (identity), ``random`` or ``bfs`` (reverse Cuthill-McKee)."""
    if order == "native":
        return edge_index
    if order == "random":
        perm = torch.randperm(n, generator=torch.Generator().manual_seed(seed))
    elif order == "bfs":
        import numpy as np
        from scipy.sparse import coo_matrix
        from scipy.sparse.csgraph import reverse_cuthill_mckee
        s, d = edge_index[0].numpy(), edge_index[1].numpy()
        a = coo_matrix((np.ones(len(s), dtype=np.int8), (d, s)), shape=(n, n)).tocsr()
        rank = reverse_cuthill_mckee(a, symmetric_mode=True)               # position -> old id
        perm = torch.empty(n, dtype=torch.long)
        perm[torch.from_numpy(rank.astype("int64"))] = torch.arange(n)      # old id -> new id
    else:
        raise ValueError(order)
    return perm[edge_index]


def _distinct_per_key(key, num_keys, span):
    """Number of distinct values of ``key`` inside each of the ``num_keys`` intervals of length ``span``."""
    u = torch.unique(key)
    return torch.bincount(u // span, minlength=num_keys)[:num_keys]


def grid_sparsity(edge_index, n, p_d, p_o):
    """Need shares of one grid (ownership rule of ``gt_b200.parallel.grid.BlockGrid``: rank ``(r, c)`` owns chunk
    ``c * P_d + r``)."""
    p = p_d * p_o
    chunk = -(-n // p)
    n_pad = chunk * p
    src, dst = edge_index[0], edge_index[1]
    ks, kd = src // chunk, dst // chunk
    r_src, c_src, r_dst, c_dst = ks % p_d, ks // p_d, kd % p_d, kd // p_d
    out = dict(grid=[p_d, p_o], chunk=chunk)
    tile = r_dst * p_o + c_src
    per_tile = torch.bincount(tile, minlength=p).double()
    out["balance"] = float(per_tile.max() / per_tile.mean().clamp_min(1e-9))
    # K / V side: distinct (row block of the destination, source id) pairs whose source the tile's rank does not own
    if p_d > 1:
        far = r_src != r_dst
        cnt = _distinct_per_key((r_dst[far] * p_o + c_src[far]) * n_pad + src[far], p, n_pad).double()
        share = cnt / ((p_d - 1) * chunk)
        out["col_need"] = dict(mean=float(share.mean()), max=float(share.max()))
    # Q side: distinct (column block of the source, destination id) pairs whose destination the rank does not own
    if p_o > 1:
        far = c_dst != c_src
        cnt = _distinct_per_key((r_dst[far] * p_o + c_src[far]) * n_pad + dst[far], p, n_pad).double()
        share = cnt / ((p_o - 1) * chunk)
        out["row_need"] = dict(mean=float(share.mean()), max=float(share.max()))
    return out


def ring_sparsity(edge_index, n, p):
    """``(P, 1)`` ring: share of a chunk's rows referenced by an edge whose destination lives on another rank."""
    chunk = -(-n // p)
    src, dst = edge_index[0], edge_index[1]
    far = (src // chunk) != (dst // chunk)
    cnt = torch.bincount(torch.unique(src[far]) // chunk, minlength=p).double()
    share = cnt / chunk
    return dict(ranks=p, ring_need=dict(mean=float(share.mean()), max=float(share.max())))


def survey(wl_edges, n, grids, orders=("native", "random", "bfs"), exp_degree=4, token=True, seed=0):
    res = {}
    for order in orders:
        ei = reorder(wl_edges, n, order, seed)
        att, n_tot = attention_edges(ei, n, exp_degree, token, seed)
        rows = []
        for p_d, p_o in grids:
            row = grid_sparsity(att, n_tot, p_d, p_o)
            if p_o == 1 and p_d > 1:
                row.update(ring_sparsity(att, n_tot, p_d))
            rows.append(row)
        res[order] = rows
    return dict(nodes=n, attention_edges=int(att.shape[1]), exp_degree=exp_degree, token=bool(token), orders=res)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--graph", default="exphormer_arxiv", help="name of a synthetic workload graph")
    ap.add_argument("--scale_down", type=int, default=1)
    ap.add_argument("--grids", nargs="+", default=["2x1", "2x2", "2x4", "4x2", "8x1"])
    ap.add_argument("--orders", nargs="+", default=["native", "random", "bfs"])
    ap.add_argument("--exp_degree", type=int, default=4)
    ap.add_argument("--no_token", action="store_true")
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from ..data.synthetic import workload_graph
    wl = workload_graph(args.graph, seed=0, scale_down=args.scale_down)
    grids = [tuple(int(v) for v in g.split("x")) for g in args.grids]
    res = survey(wl["edge_index"], wl["n"], grids, args.orders, args.exp_degree, not args.no_token)
    res["graph"] = args.graph
    for order, rows in res["orders"].items():
        for row in rows:
            print("SPARSITY " + json.dumps(dict(order=order, **row)), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)
    return res


if __name__ == "__main__":
    main()

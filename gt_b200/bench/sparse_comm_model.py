"""Where do the sparsity-aware collectives pay?  The analytic table behind the selection rule of
``gt_b200.parallel.sparse_comm.SparseRowPlan.worthwhile`` (counterpart of the reference's
``gt3d/bench/sparse_comm_model.py``).

Under an id order without locality a source row of the column block is referenced by the tile of rank ``(r, c)`` when one
of its edges ends in row block ``r``.  With ``d`` attention edges per node (self loop included, expander excluded) that
happens with probability ``1 - exp(-d / P_d)``; the ``2 d_e`` expander endpoints of a node add the order-independent floor
``1 - (1 - 1 / P_d) ** (2 d_e)``; a virtual node adds nothing per row (its own row is one row).  The Q side has the same
share with ``P_o``.  A sparse collective moves ``share`` of the dense bytes at ``A2A_OVER_AG`` times the dense rate
(1.0 on an NVSwitch node: every peer at full bandwidth), so it is chosen when ``share / A2A_OVER_AG < MARGIN``.
``gt_b200.bench.comm_sparsity`` counts the same shares on a real edge set.

    python -m gt_b200.bench.sparse_comm_model --gpus 8 64 --po 1 2 4 --degree 13.8 --exp_degree 4
"""
import argparse
import json
import math


def need_share(degree, exp_degree, parts):
    """Expected referenced share of the non-owned rows of a block gathered over ``parts`` owners."""
    if parts <= 1:
        return 1.0
    miss_graph = math.exp(-degree / parts)
    miss_exp = (1.0 - 1.0 / parts) ** (2 * exp_degree)
    return 1.0 - miss_graph * miss_exp


def table(gpus, pos, degree, exp_degree):
    from ..parallel.sparse_comm import A2A_OVER_AG, MARGIN
    rows = []
    for p in gpus:
        for p_o in pos:
            if p % p_o:
                continue
            p_d = p // p_o
            col, row = need_share(degree, exp_degree, p_d), need_share(degree, exp_degree, p_o)
            rows.append(dict(gpus=p, grid=[p_d, p_o], col_share=col, row_share=row,
                             col_time_ratio=col / A2A_OVER_AG, row_time_ratio=row / A2A_OVER_AG,
                             use_col=p_d > 1 and col / A2A_OVER_AG < MARGIN, use_row=p_o > 1 and row / A2A_OVER_AG < MARGIN))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, nargs="+", default=[2, 4, 8, 64])
    ap.add_argument("--po", type=int, nargs="+", default=[1, 2, 4])
    ap.add_argument("--degree", type=float, default=13.8, help="attention edges per node without the expander (arxiv-like: 13.8)")
    ap.add_argument("--exp_degree", type=int, default=4)
    args = ap.parse_args(argv)
    rows = table(args.gpus, args.po, args.degree, args.exp_degree)
    for r in rows:
        print("SPARSE_MODEL " + json.dumps(r), flush=True)
    return rows


if __name__ == "__main__":
    main()

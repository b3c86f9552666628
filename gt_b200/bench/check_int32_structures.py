"""Do the sparse structures of a workload fit the 32-bit indices of the kernels?  (Counterpart of the reference's
``gt3d/bench/check_int32_structures.py``, which checks the same question for its cuSPARSE / Triton structures.)

The kernels of this package keep every index array of a tile as ``int32`` (row / column pointers, source and destination
ids, segment plans, permutations to the transposed order, need-set maps) and form byte offsets of feature rows in 64 bits
(``row * width`` is widened before the multiply).  So a tile is valid while

  * its edge count (the largest pointer value) and its segment and slot counts stay below 2^31,
  * its row and column counts stay below 2^31,
  * packed payload rows times payload width is only ever formed in 64 bits (nothing to check).

``limits`` evaluates this per rank for a graph size and a grid without building the graph (edges per tile = E / P times a
skew factor); ``--build`` also builds the named synthetic workload's tile structures on the CPU for one grid and reports the
true maxima and the dtypes found.

    python -m gt_b200.bench.check_int32_structures --nodes 111059956 --edges 3339184668 --grids 8x8 16x8 --skew 1.5
    python -m gt_b200.bench.check_int32_structures --build cpu_small --grids 2x2
"""
import argparse
import json

INT32_MAX = 2 ** 31 - 1


def limits(nodes, edges, p_d, p_o, skew=1.3, seg_edges=256, stream_sub=1):
    """Largest index values a rank of a ``p_d x p_o`` grid sees; ``ok`` is False when one exceeds int32."""
    p = p_d * p_o
    chunk = -(-nodes // p)
    rows, cols = chunk * p_o, chunk * p_d
    tile_edges = int(edges / p * skew)
    sub_edges = tile_edges // max(stream_sub, 1)
    segments = rows + sub_edges // max(seg_edges, 1)
    vals = dict(rows=rows, cols=cols, tile_edges=tile_edges, edges_per_kernel=sub_edges, segments=segments)
    return dict(grid=[p_d, p_o], stream_sub=stream_sub, **vals, ok=all(v <= INT32_MAX for v in vals.values()),
                headroom=INT32_MAX / max(vals.values()))


def built(name, p_d, p_o, scale_down=1):
    """Build rank tiles of a synthetic workload on the CPU and report the dtypes and maxima of their index arrays."""
    import torch
    from ..attention import BlockCSR
    from ..data.synthetic import add_self_loops, workload_graph
    from ..parallel.grid import BlockGrid
    from ..utils.checks import validate_block
    wl = workload_graph(name, seed=0, scale_down=scale_down)
    ei = add_self_loops(wl["edge_index"], wl["n"])
    worst = dict(edges=0, max_ptr=0, max_col=0)
    dtypes = set()
    for rank in range(p_d * p_o):
        grid = BlockGrid.virtual(p_d, p_o, wl["n"], rank)
        b_ei, _ = grid.local_block(ei)
        blk = BlockCSR.from_edges(b_ei, grid.n_row_block, grid.n_col_block)
        validate_block(blk)
        worst["edges"] = max(worst["edges"], blk.num_edges)
        worst["max_ptr"] = max(worst["max_ptr"], int(blk.crow.max()))
        worst["max_col"] = max(worst["max_col"], int(blk.col.max()) if blk.num_edges else 0)
        dtypes |= {str(blk.crow.dtype), str(blk.col.dtype)}
    return dict(graph=name, grid=[p_d, p_o], nodes=wl["n"], dtypes=sorted(dtypes), **worst,
                ok=dtypes == {"torch.int32"} and worst["max_ptr"] <= INT32_MAX)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--nodes", type=int, default=111_059_956)
    ap.add_argument("--edges", type=int, default=3_339_184_668, help="attention edges, both directions, self loops and expander included")
    ap.add_argument("--grids", nargs="+", default=["2x4", "8x8", "16x8"])
    ap.add_argument("--skew", type=float, default=1.3)
    ap.add_argument("--stream_sub", type=int, default=1)
    ap.add_argument("--build", default=None, help="name of a synthetic workload to build on the CPU")
    ap.add_argument("--scale_down", type=int, default=1)
    args = ap.parse_args(argv)
    out = []
    for g in args.grids:
        p_d, p_o = (int(v) for v in g.split("x"))
        row = built(args.build, p_d, p_o, args.scale_down) if args.build else limits(args.nodes, args.edges, p_d, p_o, args.skew,
                                                                                    stream_sub=args.stream_sub)
        out.append(row)
        print("INT32 " + json.dumps(row), flush=True)
    return out


if __name__ == "__main__":
    main()

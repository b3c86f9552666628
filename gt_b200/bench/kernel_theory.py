"""Microbenchmarks behind the analytic model of the attention kernels, on one GPU (counterpart of the reference's
``gt3d/bench/kernel_theory.py``).

The gather kernels move a known number of bytes per edge, per destination row and per source row, so the time of a pass
is the larger of (a) those bytes over the memory bandwidth and (b) the latency of a warp's chain of dependent loads.
Measured here:

  * ``hbm_read_gbs``   a 1 GiB streaming read (sum reduction), the bandwidth side of the model;
  * ``call_floor_us``  forward and backward (row pass + column pass) on a block with rows but no edges (launches + row
                       bookkeeping);
  * ``sweep``          forward and backward on REGULAR blocks (each row and each column holds exactly ``d`` edges, ``d`` = 0 ... 128):
                       ns per row is flat while a row is latency bound and grows with the row's bytes afterwards; the
                       knee and the slope (ns per edge) are the two numbers the model takes;
  * ``kernels``        registers, local-memory bytes, shared memory and resident blocks per SM of the compiled instances.

Regular blocks are built from ``d`` random permutations, so the gathered rows have no locality.  The operands of the
default size (2 x 524,288 x 256 bf16 = 512 MB) are larger than L2.

    python -m gt_b200.bench.kernel_theory --out kernel_theory_b200.json
"""
import argparse
import json

import torch

from ._timing import time_ms


def regular_block(n, degree, types=3, seed=0):
    """``BlockCSR`` over ``n x n`` in which every row and every column holds exactly ``degree`` entries."""
    from ..attention import BlockCSR
    g = torch.Generator().manual_seed(seed)
    rows = torch.arange(n)
    if degree == 0:
        ei = torch.zeros(2, 0, dtype=torch.long)
    else:
        ei = torch.cat([torch.stack([torch.randperm(n, generator=g), rows]) for _ in range(degree)], 1)
    et = torch.randint(0, types, (ei.shape[1],), generator=g)
    return BlockCSR.from_edges(ei, n, n, et)


def passes(q, k, v, blk, gate, score, norm):
    """The three kernel passes on one block as callables: forward, backward row pass + column pass together."""
    from ..attention import backend_cuda as bc
    bias = None
    kw = dict(score=score, norm=norm)
    acc, l, m = bc.attn_fwd_partial(q, k, v, blk, gate, bias, **kw)
    dacc, dl = torch.randn_like(acc), torch.randn_like(l)
    return dict(fwd=lambda: bc.attn_fwd_partial(q, k, v, blk, gate, bias, **kw),
                bwd=lambda: bc.attn_bwd_partial(q, k, v, blk, gate, bias, m, dacc, dl, **kw))


def pass_bytes(n, degree, hd, es):
    """Bytes an ideal pass without cache reuse moves: per edge two gathered rows and an index, per row its operands."""
    e = n * degree
    return dict(fwd=e * (2 * hd * es + 8) + n * (hd * es + hd * 4 + 32),
                bwd=2 * e * (2 * hd * es + 8) + n * (6 * hd * es + 64))


def fit_knee(degrees, ns_per_row):
    """Least-squares line through the upper half of the sweep (bandwidth side) and the flat level of the lower end."""
    pts = [(d, t) for d, t in zip(degrees, ns_per_row) if d >= 16]
    if len(pts) < 2:
        return dict(ns_per_edge=None, floor_ns_per_row=ns_per_row[0] if ns_per_row else None, knee_degree=None)
    mx = sum(d for d, _ in pts) / len(pts)
    my = sum(t for _, t in pts) / len(pts)
    slope = sum((d - mx) * (t - my) for d, t in pts) / max(sum((d - mx) ** 2 for d, _ in pts), 1e-9)
    floor = min(t for d, t in zip(degrees, ns_per_row) if d <= 2) if any(d <= 2 for d in degrees) else ns_per_row[0]
    return dict(ns_per_edge=slope, floor_ns_per_row=floor, knee_degree=floor / slope if slope > 0 else None)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=1 << 19)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--degrees", type=int, nargs="+", default=[0, 1, 2, 4, 8, 16, 32, 64, 128])
    ap.add_argument("--score", default="gated")
    ap.add_argument("--norm", default="clampexp")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from ..ops import native
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, h, d = args.rows, args.heads, args.head_dim
    res = dict(rows=n, heads=h, head_dim=d, score=args.score, norm=args.norm, device=torch.cuda.get_device_name(dev))
    buf = torch.empty(1 << 28, dtype=torch.float32, device=dev)
    res["hbm_read_gbs"] = buf.numel() * 4 / time_ms(lambda: buf.sum(), iters=5, warmup=3) / 1e6
    del buf
    res["kernels"] = [dict(zip(("name", "regs", "local_bytes", "static_smem", "dyn_smem", "blocks_per_sm"), t))
                      for t in native.ext().attn_kernel_info()]
    torch.manual_seed(0)
    q, k, v = (torch.randn(n, h, d, device=dev).bfloat16() for _ in range(3))
    gate = torch.randn(3, h, d, device=dev) if args.score == "gated" else None
    sweep = []
    for deg in args.degrees:
        blk = regular_block(n, deg).to(dev)
        fns = passes(q, k, v, blk, gate, args.score, args.norm)
        by = pass_bytes(n, deg, h * d, 2)
        row = dict(degree=deg, edges=n * deg)
        for name, fn in fns.items():
            ms = time_ms(fn, iters=args.iters, warmup=3, flush=True, dev=dev)
            row[name + "_ms"] = ms
            row[name + "_ns_per_row"] = ms * 1e6 / n
            row[name + "_model_gbs"] = by[name] / ms / 1e6
        sweep.append(row)
        print("THEORY " + json.dumps(row), flush=True)
    res["sweep"] = sweep
    res["call_floor_us"] = {p: sweep[0][p + "_ms"] * 1e3 for p in ("fwd", "bwd")} if args.degrees and args.degrees[0] == 0 else None
    res["fit"] = {p: fit_knee([r["degree"] for r in sweep], [r[p + "_ns_per_row"] for r in sweep]) for p in ("fwd", "bwd")}
    print("THEORY_FIT " + json.dumps(dict(hbm_read_gbs=res["hbm_read_gbs"], fit=res["fit"], kernels=res["kernels"])), flush=True)
    if args.out:
        with open(args.out, "w") as f:
            json.dump(res, f, indent=1)
    return res


if __name__ == "__main__":
    main()

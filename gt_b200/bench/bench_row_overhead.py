"""Per-row overhead of the attention kernels on blocks with very few edges per row (counterpart of the reference's
``gt3d/bench/bench_row_overhead.py``).  A column sub-block of the streamed layer holds about ``E / (P n_sub)`` edges spread
over ``N / P_d`` rows, i.e. 1 to 3 edges per row, where the fixed cost per row (pointer reads, the q row, the result row)
outweighs the gathers.  Fixed number of rows, edges per row swept; reports ms per pass, ns per row and per edge for

  * the forward into fresh outputs over all rows (``fwd``),
  * the forward that ADDS into the packed payload and visits only rows that own an edge (``fwd_accum``, the streamed
    layer's kernel),
  * the backward (row pass + column pass, ``bwd``),
  * the row-sized bookkeeping the streamed layer does per sub-block when it cannot accumulate in place (zero-fill and add of
    the packed ``[rows, H d + H]`` fp32 buffer, ``bookkeeping``).

    python -m gt_b200.bench.bench_row_overhead --rows 612352 --cols 153088 --per_row 0.25 0.5 1 2 3 8
"""
import argparse
import json

import torch

from ._timing import time_ms


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=612352)
    ap.add_argument("--cols", type=int, default=153088)
    ap.add_argument("--per_row", type=float, nargs="+", default=[0.25, 0.5, 1, 2, 3, 8])
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args(argv)
    from ..attention import backend_cuda as bc
    from .bench_kernel_opts import random_block
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, c, h, d = args.rows, args.cols, args.heads, args.head_dim
    hd = h * d
    torch.manual_seed(0)
    q = torch.randn(n, h, d, device=dev).bfloat16()
    k, v = (torch.randn(c, h, d, device=dev).bfloat16() for _ in range(2))
    gate = torch.randn(3, h, d, device=dev)
    packed = torch.zeros(n, hd + h, device=dev)
    tmp = torch.zeros_like(packed)
    kw = dict(score="gated", norm="clampexp")
    out = []
    for per_row in args.per_row:
        e = int(n * per_row)
        blk = random_block(n, c, e).to(dev)
        acc, l, m = bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw)
        dacc, dl = torch.randn_like(acc), torch.randn_like(l)
        t = dict(
            fwd=time_ms(lambda: bc.attn_fwd_partial(q, k, v, blk, gate, None, **kw), iters=args.iters, warmup=3, flush=True, dev=dev),
            fwd_accum=time_ms(lambda: bc.attn_fwd_partial_accum(q, k, v, blk, gate, None, packed, hd, **kw), iters=args.iters, warmup=3,
                              flush=True, dev=dev),
            bwd=time_ms(lambda: bc.attn_bwd_partial(q, k, v, blk, gate, None, m, dacc, dl, **kw), iters=args.iters, warmup=3, flush=True,
                        dev=dev),
            bookkeeping=time_ms(lambda: packed.add_(tmp.zero_()), iters=args.iters, warmup=3, flush=True, dev=dev))
        row = dict(rows=n, cols=c, edges=e, per_row=per_row, nonempty_rows=int(blk.dcsr_rows().numel()))
        for name, ms in t.items():
            row[name + "_ms"] = ms
            row[name + "_ns_per_row"] = ms * 1e6 / n
        row["fwd_ns_per_edge"] = t["fwd"] * 1e6 / max(e, 1)
        out.append(row)
        print("ROWS " + json.dumps(row), flush=True)
    return out


if __name__ == "__main__":
    main()

"""Cost of a gather that is served from L2, relative to one served from HBM, for the attention passes (one GPU).

The forward and the backward row pass gather K / V rows of the column block; the backward column pass gathers q / dAcc rows of the
row block.  A block whose gathered side fits in L2 (``cols x 2 x H d`` bf16 well below 126 MB, no flush between launches) is timed
against a block with the same rows and edges whose gathered side is several times L2 (flushed before every launch);
``lambda = (time per edge, L2 resident) / (time per edge, HBM)`` per pass is the factor the performance model applies to blocks
that fit (counterpart of the reference's ``gt3d/bench/kernel_l2.py``; ``kernel_constants`` fits the same two regimes as slopes).

    python -m gt_b200.bench.kernel_l2 [--rows 262144] [--degree 16] [--out kernel_l2_b200.json]
"""
import argparse
import json

import torch

L2_BYTES = 126 << 20


def gathered_bytes(cols, h, d, es=2):
    """Bytes of the gathered operands (K and V, or q and dAcc) of a block with ``cols`` source rows."""
    return 2 * cols * h * d * es


def l2_factor(resident, hbm):
    """``{pass: lambda}`` from two measurements ``dict(edges=..., fwd_ms=..., bwd_ms=...)``: time per edge in L2 over time per edge from HBM."""
    out = {}
    for p in ("fwd", "bwd"):
        a, b = resident[p + "_ms"] / max(resident["edges"], 1), hbm[p + "_ms"] / max(hbm["edges"], 1)
        out[p] = a / b if b > 0 else None
    return out


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=262144)
    ap.add_argument("--degree", type=int, default=16, help="edges per destination row")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--resident_cols", type=int, default=32768, help="source rows of the L2-resident block (2 x cols x H d bf16 must fit)")
    ap.add_argument("--hbm_cols", type=int, default=1 << 20)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default=None)
    args = ap.parse_args(argv)
    from .kernel_constants import attention_points
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    h, d, e = args.heads, args.head_dim, args.rows * args.degree
    if gathered_bytes(args.resident_cols, h, d) > L2_BYTES // 2:
        raise SystemExit("--resident_cols: the gathered operands must stay below half of L2")
    res = dict(rows=args.rows, degree=args.degree, heads=h, head_dim=d, device=torch.cuda.get_device_name(dev))
    for name, cols, flush in (("resident", args.resident_cols, False), ("hbm", args.hbm_cols, True)):
        (_, _, _, f, b), = attention_points(dev, h, d, [(args.rows, cols, e)], flush, args.iters)
        res[name] = dict(cols=cols, edges=e, gathered_mb=gathered_bytes(cols, h, d) / 2 ** 20, fwd_ms=f, bwd_ms=b)
    res["lambda"] = l2_factor(res["resident"], res["hbm"])
    print("KERNEL_L2 " + json.dumps(res), flush=True)
    if args.out:
        with open(args.out, "w") as fobj:
            json.dump(res, fobj, indent=1)
    return res


if __name__ == "__main__":
    main()

"""Workload for Nsight Compute: the attention passes on the regular blocks of ``kernel_theory`` (every row and column
holds ``d`` edges), one call per (pass, degree) between ``cudaProfilerStart`` / ``cudaProfilerStop``, so that

    ncu --profile-from-start off --clock-control none -k regex:attn_ --metrics <few> --csv --page raw \\
        --log-file kernel_ncu.csv python -m gt_b200.bench.kernel_ncu --order kernel_ncu_order.json

captures exactly these launches (warm-up happens outside the profiled range).  The launch order is written as JSON;
``kernel_ncu_report`` joins it with the capture and sets the measured DRAM bytes against the bytes of the analytic model.
Counterpart of the reference's ``gt3d/bench/kernel_ncu.py``.

The default case is deliberately small (131,072 rows x 256 channels: 64 MB per operand, K and V together above L2;
under 1 GB on the device; 2 passes x 3 degrees = about 9 kernel launches), so that a capture ends by itself within a minute
or two.  Run the same command once without ``ncu`` first.
"""
import argparse
import json

import torch


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", type=int, default=1 << 17)
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--head_dim", type=int, default=32)
    ap.add_argument("--degrees", type=int, nargs="+", default=[1, 16, 64])
    ap.add_argument("--score", default="gated")
    ap.add_argument("--norm", default="clampexp")
    ap.add_argument("--order", default=None, help="write the launch order (JSON) here")
    args = ap.parse_args(argv)
    from .kernel_theory import pass_bytes, passes, regular_block
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    n, h, d = args.rows, args.heads, args.head_dim
    torch.manual_seed(0)
    q, k, v = (torch.randn(n, h, d, device=dev).bfloat16() for _ in range(3))
    gate = torch.randn(3, h, d, device=dev) if args.score == "gated" else None
    cases = []
    for deg in args.degrees:
        blk = regular_block(n, deg).to(dev)
        fns = passes(q, k, v, blk, gate, args.score, args.norm)          # also the warm-up call of the forward
        fns["bwd"]()
        cases.append((deg, fns))
    torch.cuda.synchronize()
    order = []
    torch.cuda.profiler.start()
    for deg, fns in cases:
        by = pass_bytes(n, deg, h * d, 2)
        for name, fn in fns.items():
            fn()
            order.append(dict(call=name, degree=deg, rows=n, heads=h, head_dim=d, model_bytes=by[name]))
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("NCU_ORDER " + json.dumps(order), flush=True)
    if args.order:
        with open(args.order, "w") as f:
            json.dump(order, f, indent=1)
    return order


if __name__ == "__main__":
    main()

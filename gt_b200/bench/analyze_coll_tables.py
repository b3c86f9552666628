"""Collective rates of several calibration runs side by side.

``python -m gt_b200.bench.hw_constants --only coll --out FILE`` stores, per collective kind, the fitted (latency, rate) pair and
the measured (MB per rank, ms) curve.  This tool reads any number of such files (different world sizes, transports,
``NCCL_*`` settings, nodes) and prints, per kind and payload size, the rate in GB/s of received bytes per rank of every file,
so that a slow configuration stands out.  Counterpart of the reference's ``gt3d/bench/analyze_rs_diag.py``.

    python -m gt_b200.bench.analyze_coll_tables run_a.json run_b.json [--kind rs]
"""
import argparse
import json
import os


def load(path):
    with open(path) as f:
        d = json.load(f)
    return d.get("_coll_curves_mb_ms") or {}, d.get("coll") or {}, d.get("_world")


def table(paths, kind):
    """``{"sizes": [...], "columns": [tag...], "rates": {size: [GB/s or None per column]}, "fit": [(alpha_us, GB/s) or None]}``."""
    cols, curves, fits = [], [], []
    for p in paths:
        cur, fit, world = load(p)
        cols.append(os.path.splitext(os.path.basename(p))[0] + (f"@{world}" if world else ""))
        curves.append({round(float(mb), 4): float(ms) for mb, ms in cur.get(kind, [])})
        fits.append(tuple(fit[kind]) if kind in fit else None)
    sizes = sorted({mb for c in curves for mb in c})
    rates = {mb: [round(mb * 2 ** 20 / (c[mb] * 1e-3) / 1e9, 1) if mb in c and c[mb] > 0 else None for c in curves] for mb in sizes}
    return dict(sizes=sizes, columns=cols, rates=rates, fit=fits)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("files", nargs="+")
    ap.add_argument("--kind", default=None, choices=["ag", "rs", "a2a", "ar", "p2p"], help="default: every kind found")
    args = ap.parse_args(argv)
    kinds = [args.kind] if args.kind else ["ag", "rs", "a2a", "ar", "p2p"]
    out = {}
    for kind in kinds:
        t = table(args.files, kind)
        if not t["sizes"]:
            continue
        out[kind] = t
        print(f"{kind.upper()}: GB/s per rank (received bytes / device time, max over ranks)")
        print(f"{'MB':>9s} " + " ".join(f"{c[-18:]:>18s}" for c in t["columns"]))
        for mb in t["sizes"]:
            print(f"{mb:9.2f} " + " ".join(f"{r:18.1f}" if r is not None else f"{'':>18s}" for r in t["rates"][mb]))
        print(f"{'fit':>9s} " + " ".join((f"{f[0]:7.1f}us {f[1]:6.0f}GB/s" if f else "").rjust(18) for f in t["fit"]))
        print()
    return out


if __name__ == "__main__":
    main()

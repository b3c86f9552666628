"""Figures from parsed logs (counterpart of the reference's ``gt3d/bench/plot_figures.py`` / ``plot_paper_figs.py``):

  ``scaling``  ms per epoch against the number of GPUs, one line per (model, hidden, layers), from ``STEADY`` lines;
  ``curves``   validation / test accuracy against training seconds, one line per log, from the epoch lines;
  ``sweep``    ns per row against edges per row of the regular-block sweep (``THEORY`` lines of ``kernel_theory``);
  ``time_to_acc``  training seconds until a log first reaches ``--target`` on ``--metric`` (one bar per log);
  ``model``    predicted against measured step time of every measured grid (the table behind ``validate_model``);
  ``versus``   speed-up of one benchmark arm over another per GPU count, from the JSON lines that ``bench.py`` prints
               (``logs`` = files holding the lines of both arms; ``--base reference`` names the arm in the denominator).

    python -m gt_b200.bench.plot_figures scaling logs/*.log --out scaling.png

The series are computed by plain functions (``scaling_series`` ...), usable without a plotting library; drawing needs
matplotlib (Agg backend, no display), which is imported only when a figure is written.
"""
import argparse
import json

from . import parse_logs


def scaling_series(rows):
    """``{(model, hidden, layers): [(world, ms_per_epoch, grid), ...]}`` sorted by world; the fastest grid per world size."""
    best = {}
    for r in rows:
        key = (r.get("model"), r.get("hidden"), r.get("layers"))
        w, ms = int(r["world"]), float(r["ms_per_epoch"])
        cur = best.setdefault(key, {})
        if w not in cur or ms < cur[w][1]:
            cur[w] = (w, ms, r.get("grid"))
    return {k: [v[w] for w in sorted(v)] for k, v in best.items()}


def efficiency(series):
    """Strong-scaling efficiency of a ``[(world, ms, grid)]`` series against its smallest world size."""
    if not series:
        return []
    w0, t0, _ = series[0]
    return [(w, (t0 * w0) / (t * w)) for w, t, _ in series]


def curve_series(rows, metric="val_acc"):
    out = {}
    for r in rows:
        out.setdefault(r["log"], []).append((r["train_seconds"], r[metric]))
    return out


def sweep_series(rows):
    out = {"fwd": [], "bwd": []}
    for r in rows:
        if r.get("tag") == "THEORY" and "degree" in r:
            for p in out:
                out[p].append((int(r["degree"]), float(r[p + "_ns_per_row"])))
    return {p: sorted(v) for p, v in out.items()}


def time_to_acc_series(rows, metric="val_acc", target=0.5):
    """``{log: seconds}``: cumulative training time at the first evaluated epoch whose ``metric`` reaches ``target`` (logs that
    never reach it are left out)."""
    out = {}
    for log, pts in curve_series(rows, metric).items():
        hit = [t for t, v in sorted(pts) if v >= target]
        if hit:
            out[log] = hit[0]
    return out


def model_series(rows=None):
    """``{"world N": [(measured ms, predicted ms, grid), ...]}`` for the measured grids (default: the package's table)."""
    from . import model_validation_data as mvd
    from .validate_model import predict
    out = {}
    for r in (rows if rows is not None else mvd.MEASURED):
        world = 1
        for p_ in r["grid"]:
            world *= p_
        out.setdefault(f"world {world}", []).append((float(r["ms"]), float(predict(r)), "x".join(map(str, r["grid"]))))
    return {k: sorted(v) for k, v in out.items()}


def versus_series(lines, base="reference"):
    """``[(n_gpus, speed-up)]`` of the other arm over ``base`` from benchmark JSON lines (dicts with ``impl``, ``n_gpus``,
    ``ms_per_step``); the last line of an (arm, GPU count) wins."""
    ms = {}
    for d in lines:
        if "ms_per_step" in d and "n_gpus" in d:
            ms[(d.get("impl", "gt_b200"), int(d["n_gpus"]))] = float(d["ms_per_step"])
    out = []
    for (impl, n), t in sorted(ms.items(), key=lambda kv: kv[0][1]):
        if impl != base and (base, n) in ms:
            out.append((n, ms[(base, n)] / t))
    return out


def _json_lines(paths):
    out = []
    for p_ in paths:
        with open(p_) as f:
            for ln in f:
                ln = ln.strip()
                if ln.startswith("{") and ln.endswith("}"):
                    try:
                        out.append(json.loads(ln))
                    except ValueError:
                        pass
    return out


def _pyplot():
    try:
        import matplotlib
    except ImportError as e:
        raise SystemExit("plot_figures: matplotlib is not installed; use parse_logs for CSV tables instead") from e
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    return plt


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["scaling", "curves", "sweep", "time_to_acc", "model", "versus"])
    ap.add_argument("logs", nargs="*")
    ap.add_argument("--out", default=None, help="image file; without it the series are printed as JSON")
    ap.add_argument("--metric", default="val_acc")
    ap.add_argument("--target", type=float, default=0.5)
    ap.add_argument("--base", default="reference")
    args = ap.parse_args(argv)
    if args.what == "scaling":
        series = {" ".join(str(v) for v in k): v for k, v in scaling_series(parse_logs.steady(args.logs)).items()}
        xlabel, ylabel, logx = "GPUs", "ms per epoch", True
    elif args.what == "curves":
        series = curve_series(parse_logs.curves(args.logs), args.metric)
        xlabel, ylabel, logx = "training seconds", args.metric, False
    elif args.what == "time_to_acc":
        tta = time_to_acc_series(parse_logs.curves(args.logs), args.metric, args.target)
        series = {"seconds to %s >= %g" % (args.metric, args.target): [(i, t) for i, (_, t) in enumerate(sorted(tta.items()))]}
        xlabel, ylabel, logx = "log", "training seconds", False
        if not args.out:
            print(json.dumps(tta))
            return tta
    elif args.what == "model":
        series = {k: [(m, p_) for m, p_, _ in v] for k, v in model_series().items()}
        xlabel, ylabel, logx = "measured ms per step", "predicted ms per step", False
    elif args.what == "versus":
        series = {"speed-up over " + args.base: versus_series(_json_lines(args.logs), args.base)}
        xlabel, ylabel, logx = "GPUs", "speed-up", True
    else:
        series = sweep_series(parse_logs.tagged_lines(args.logs, "THEORY"))
        xlabel, ylabel, logx = "edges per row", "ns per row", True
    if not args.out:
        print(json.dumps(series))
        return series
    plt = _pyplot()
    fig, ax = plt.subplots(figsize=(5, 3.5))
    for name, pts in series.items():
        ax.plot([p[0] for p in pts], [p[1] for p in pts], marker="o", label=str(name))
    if logx:
        ax.set_xscale("log", base=2)
    ax.set_xlabel(xlabel)
    ax.set_ylabel(ylabel)
    ax.legend(fontsize=7)
    fig.tight_layout()
    fig.savefig(args.out, dpi=150)
    return series


if __name__ == "__main__":
    main()

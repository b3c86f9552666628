"""Turn trainer and benchmark logs into tables (counterpart of the reference's ``gt3d/bench/extract_curves.py`` and
``parse_*.py`` helpers; reads files only).

  ``curves``   accuracy against training time from ``train_dist`` logs: one CSV row per printed epoch line;
  ``steady``   one CSV row per ``STEADY`` line (model, grid, world, hidden, layers, ms per epoch, peak GB): the scaling table;
  ``lines``    every tagged JSON line of the benches (``ATTN``, ``GEMM``, ``COLL``, ``OPTS``, ``ROWS``, ``THEORY``,
               ``SPARSITY``, ``RESULT`` ...) as CSV with the union of their keys, optionally one tag only.

    python -m gt_b200.bench.parse_logs curves logs/run_a.log logs/run_b.log > curves.csv
    python -m gt_b200.bench.parse_logs steady logs/*.log > scaling.csv
    python -m gt_b200.bench.parse_logs lines --tag ATTN logs/attn_*.log > attn.csv
"""
import argparse
import csv
import json
import re
import sys

EPOCH = re.compile(r"^epoch\s+(\d+)\s+loss\s+([\d.eE+-]+)\s+train\s+([\d.]+)\s+val\s+([\d.]+)\s+test\s+([\d.]+)\s+\|\s+best val\s+([\d.]+)"
                   r"\s+test\s+([\d.]+)\s+@\s+(-?\d+)\s+\|\s+([\d.]+)\s+ms/epoch")
STEADY = re.compile(r"^STEADY\s+(.*)$")
TAGGED = re.compile(r"^([A-Z][A-Z0-9_]+)\s+(\{.*\})\s*$")


def curves(paths):
    rows = []
    for p in paths:
        with open(p) as f:
            for line in f:
                m = EPOCH.match(line)
                if m:
                    ep, loss, tr, va, te, bv, bt, be, ms = m.groups()
                    # ms/epoch is the running mean over the epochs so far, so (epoch + 1) x mean is the time spent training
                    rows.append(dict(log=p, epoch=int(ep), train_seconds=(int(ep) + 1) * float(ms) / 1e3, loss=float(loss), train_acc=float(tr),
                                     val_acc=float(va), test_acc=float(te), best_val=float(bv), test_at_best_val=float(bt), best_epoch=int(be)))
    return rows


def curves_jsonl(paths):
    """The rows of :func:`curves` from ``train_dist --metrics_jsonl`` files (one JSON object per evaluated epoch).  The training
    time of an epoch row is the sum of the device times of the evaluated epochs so far, scaled to the epochs in between."""
    import json
    rows = []
    for p in paths:
        seconds, last_epoch = 0.0, -1
        with open(p) as f:
            for line in f:
                line = line.strip()
                if not line.startswith("{"):
                    continue
                d = json.loads(line)
                seconds += (d["epoch"] - last_epoch) * d["epoch_ms"] / 1e3
                last_epoch = d["epoch"]
                rows.append(dict(log=p, epoch=int(d["epoch"]), train_seconds=seconds, loss=float(d["loss"]), train_acc=float(d["train"]),
                                 val_acc=float(d["val"]), test_acc=float(d["test"]), best_val=float(d["best_val"]),
                                 test_at_best_val=None, best_epoch=int(d["best_epoch"])))
    return rows


def steady(paths):
    rows = []
    for p in paths:
        with open(p) as f:
            for line in f:
                m = STEADY.match(line)
                if m:
                    row = dict(log=p)
                    for kv in m.group(1).split():
                        if "=" in kv:
                            k, v = kv.split("=", 1)
                            try:
                                row[k] = float(v) if any(c in v for c in ".eE") and not v.replace(".", "").isalpha() else int(v)
                            except ValueError:
                                row[k] = v
                    rows.append(row)
    return rows


def tagged_lines(paths, tag=None):
    rows = []
    for p in paths:
        with open(p) as f:
            for line in f:
                m = TAGGED.match(line)
                if not m or (tag and m.group(1) != tag):
                    continue
                try:
                    rec = json.loads(m.group(2))
                except json.JSONDecodeError:
                    continue
                if isinstance(rec, dict):
                    flat = {k: (json.dumps(v) if isinstance(v, (dict, list)) else v) for k, v in rec.items()}
                    rows.append(dict(log=p, tag=m.group(1), **flat))
    return rows


def write_csv(rows, file=None):
    file = file or sys.stdout
    keys = []
    for r in rows:
        for k in r:
            if k not in keys:
                keys.append(k)
    w = csv.DictWriter(file, fieldnames=keys)
    w.writeheader()
    w.writerows(rows)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["curves", "steady", "lines"])
    ap.add_argument("logs", nargs="+")
    ap.add_argument("--tag", default=None)
    args = ap.parse_args(argv)
    rows = curves(args.logs) if args.what == "curves" else steady(args.logs) if args.what == "steady" else tagged_lines(args.logs, args.tag)
    write_csv(rows)
    return rows


if __name__ == "__main__":
    main()

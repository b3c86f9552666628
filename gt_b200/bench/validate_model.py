"""Compare the performance model's predictions with the measured table (``model_validation_data.MEASURED``) or with
``STEADY`` / bench JSON lines given on the command line; prints the ratio per row and the ranking agreement per world
size (counterpart of the reference's ``gt3d/bench/validate_model.py``).  Pure host arithmetic.

    python -m gt_b200.bench.validate_model
    python -m gt_b200.bench.validate_model --constants my_constants.json --log run1.log run2.log
"""
import argparse
import json
import re

from ..perf import grid_select as gs
from .model_validation_data import ARXIV_CL, MEASURED


def graph_of(spec):
    n, e = spec["n"], spec["e_graph"]
    e_attn = gs.attention_edges(n, e, spec["exp_deg"]) - n + (2 * n if spec.get("virtual_node") else 0)
    return gs.Graph(n, e_attn, e + n, spec["f_in"], spec["name"], classes=spec.get("classes", 40), exp_deg=spec["exp_deg"],
                    skew=spec.get("skew", 1.0), token=bool(spec.get("virtual_node")))


def predict(row):
    g = graph_of(row["graph"])
    hidden, heads, layers = row["model"]
    m = gs.Model(hidden, heads, layers, transport=row.get("transport", "nccl"))
    grid = tuple(row["grid"])
    if len(grid) == 3:
        return gs.predict_head_ms(*grid, g, m)
    return gs.predict_fused_ms(grid[0], grid[1], g, m)


def rows_from_logs(paths):
    """``STEADY model=.. grid=AxB world=.. hidden=.. layers=.. ms_per_epoch=..`` lines and bench JSON lines."""
    rows = []
    for p in paths:
        for line in open(p):
            mt = re.search(r"STEADY model=(\w+) grid=([\dx]+) world=(\d+) hidden=(\w+) layers=(\w+) ms_per_epoch=([\d.]+)", line)
            if mt:
                hidden = int(mt.group(4)) if mt.group(4).isdigit() else 256
                layers = int(mt.group(5)) if mt.group(5).isdigit() else 4
                rows.append(dict(graph=ARXIV_CL, model=(hidden, 8, layers), grid=tuple(int(v) for v in mt.group(2).split("x")),
                                 ms=float(mt.group(6))))
            elif line.startswith("{") and '"ms_per_step"' in line:
                j = json.loads(line)
                par = j.get("config", {}).get("grid") or {1: (1, 1), 2: (2, 1), 4: (2, 2), 8: (4, 2)}[j["n_gpus"]]
                rows.append(dict(graph=ARXIV_CL, model=(256, 8, 4), grid=tuple(par), ms=j["ms_per_step"],
                                 transport=j.get("config", {}).get("comm", "nccl")))
    return rows


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--constants", default=None)
    ap.add_argument("--log", nargs="*", default=[])
    args = ap.parse_args(argv)
    if args.constants:
        gs.load_constants(args.constants)
    rows = list(MEASURED) + rows_from_logs(args.log)
    by_world = {}
    print(f"{'grid':>8s} {'transport':>9s} {'measured':>9s} {'model':>9s} {'ratio':>6s}")
    worst = 1.0
    for r in rows:
        pred = predict(r)
        ratio = pred / r["ms"]
        worst = max(worst, ratio, 1 / ratio)
        world = 1
        for s in r["grid"]:
            world *= s
        by_world.setdefault((world, r.get("transport", "nccl")), []).append((r["grid"], r["ms"], pred))
        print(f"{'x'.join(map(str, r['grid'])):>8s} {r.get('transport', 'nccl'):>9s} {r['ms']:9.2f} {pred:9.2f} {ratio:6.2f}")
    for (world, tr), lst in sorted(by_world.items()):
        if len(lst) > 1:
            a = [g for g, _, _ in sorted(lst, key=lambda v: v[1])]
            b = [g for g, _, _ in sorted(lst, key=lambda v: v[2])]
            print(f"world {world} ({tr}): measured order {a}, model order {b}: {'AGREE' if a[0] == b[0] else 'DIFFER'} on the best grid")
    print(f"worst ratio {worst:.2f}")
    from .model_validation_data import OTHER_CONFIGS
    print("other configurations (measured, not modelled):")
    for r in OTHER_CONFIGS:
        print(f"  {'x'.join(map(str, r['grid'])):>6s} {r['ms']:9.1f} ms {r['peak_gb']:6.1f} GB  {r['name']}")
    return worst


if __name__ == "__main__":
    main()

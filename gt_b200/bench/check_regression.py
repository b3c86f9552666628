"""Timing regression check: does the benchmark step still run as fast as the recorded measurement of its grid?

Runs ``bench.py`` on N GPUs (or reads result lines that were produced elsewhere), looks up the recorded time of the same grid in
``gt_b200.bench.model_validation_data.MEASURED`` and fails when the step is slower than the record by more than the tolerance;
a run whose clock record shows thermal or hardware slow-down is reported as inconclusive instead.  The counterpart of the
reference's post-integration check that compares steady-state epoch times with its result table
(``gt3d/scripts/sbatch_integration_check.sh``).

    python -m gt_b200.bench.check_regression --gpus 1 8                 # runs bench.py at 1 and 8 GPUs
    python -m gt_b200.bench.check_regression --from_json BENCH.json     # checks lines / files produced earlier
"""
import argparse
import json
import os
import subprocess
import sys

from .model_validation_data import LATEST_MS, MEASURED

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
BAD_CLOCK_REASONS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown")


def recorded_ms(grid, transport=None):
    """Recorded ms per step of ``grid`` on the benchmark configuration, or ``None``."""
    if tuple(grid) in LATEST_MS:
        return LATEST_MS[tuple(grid)]
    for row in MEASURED:
        if tuple(row["grid"]) == tuple(grid) and (transport is None or row["transport"] == transport or tuple(grid) == (1, 1)):
            return row["ms"]
    return None


def assess(result, tolerance=0.10):
    """``(verdict, text)`` for one result line of ``bench.py``: verdict in ok / slower / inconclusive / unknown."""
    if result.get("impl") == "reference":
        return "unknown", "line of the reference arm: not compared"
    cfg = result.get("config", {})
    grid = tuple(cfg.get("grid") or ())
    if not grid and str(cfg.get("parallelism", "")).startswith("grid "):
        grid = tuple(int(v) for v in cfg["parallelism"][5:].split("x"))
    ms = result.get("ms_per_step")
    if not grid or ms is None:
        return "unknown", "not a bench.py result line"
    reasons = [r for r in result.get("clocks", {}).get("reasons", []) if r in BAD_CLOCK_REASONS]
    ref = recorded_ms(grid)
    name = "x".join(map(str, grid))
    if reasons:
        return "inconclusive", f"grid {name}: {ms:.2f} ms under {', '.join(reasons)}: measure again"
    if ref is None:
        return "unknown", f"grid {name}: {ms:.2f} ms, no recorded time for this grid"
    ratio = ms / ref
    if ratio > 1.0 + tolerance:
        return "slower", f"grid {name}: {ms:.2f} ms against {ref:.2f} ms recorded ({ratio:.2f} x): REGRESSION"
    return "ok", f"grid {name}: {ms:.2f} ms against {ref:.2f} ms recorded ({ratio:.2f} x)"


def run_bench(n, steps, warmup, extra):
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--gpus", str(n), "--steps", str(steps), "--warmup", str(warmup)] + extra
    if n > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(n), "--master-addr", "127.0.0.1",
               "--master-port", str(29500 + n)] + cmd[1:]
    out = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True)
    for line in reversed(out.stdout.splitlines()):
        if line.startswith("{"):
            return json.loads(line)
    raise RuntimeError(f"bench.py on {n} GPUs printed no result line (exit {out.returncode}): {out.stderr[-400:]}")


def read_results(path):
    text = open(path).read().strip()
    try:
        blob = json.loads(text)
        if isinstance(blob, list):
            return blob
        for key in ("parsed", "result"):                     # wrappers that keep the result line under a key
            if isinstance(blob.get(key), dict) and "ms_per_step" in blob[key]:
                return [blob[key]]
        return [blob]
    except json.JSONDecodeError:
        return [json.loads(line) for line in text.splitlines() if line.startswith("{")]


def main(argv=None):
    ap = argparse.ArgumentParser(description="compare benchmark step times with the recorded measurements")
    ap.add_argument("--gpus", type=int, nargs="+", default=[1])
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--tolerance", type=float, default=0.10, help="allowed slow-down relative to the record")
    ap.add_argument("--from_json", nargs="+", default=None, metavar="FILE", help="check result lines from files instead of running bench.py")
    ap.add_argument("bench_args", nargs=argparse.REMAINDER, help="after --: passed on to bench.py")
    args = ap.parse_args(argv)
    extra = [a for a in args.bench_args if a != "--"]
    results = [r for f in args.from_json for r in read_results(f)] if args.from_json else [run_bench(n, args.steps, args.warmup, extra) for n in args.gpus]
    verdicts = []
    for r in results:
        v, text = assess(r, args.tolerance)
        verdicts.append(v)
        print(f"[{v}] {text}")
    return 1 if "slower" in verdicts else (2 if "inconclusive" in verdicts else 0)


if __name__ == "__main__":
    raise SystemExit(main())

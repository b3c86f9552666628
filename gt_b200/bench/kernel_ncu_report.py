"""Join an Nsight Compute capture of ``kernel_ncu`` (``--page raw --csv``, one line per kernel launch) with the launch
order that workload wrote, and print per (call, degree): the kernels that ran, their duration, measured DRAM bytes against
the bytes of the analytic model, DRAM throughput, registers and achieved occupancy.  Counterpart of the reference's
``gt3d/bench/kernel_ncu_report.py``; reads files only (no GPU).

    python -m gt_b200.bench.kernel_ncu_report kernel_ncu.csv kernel_ncu_order.json

A forward call launches one main kernel (plus a combine kernel when hub rows are split); a backward call launches the row
pass and the column pass.  Launches are assigned to calls in order by kernel name: ``attn_fwd`` starts a forward call,
``attn_bwd_row`` a backward call.
"""
import csv
import json
import sys

METRICS = {
    "ms": ("gpu__time_duration.sum",),
    "dram_read": ("dram__bytes_read.sum",),
    "dram_write": ("dram__bytes_write.sum",),
    "dram_pct": ("gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed",),
    "regs": ("launch__registers_per_thread",),
    "occupancy_pct": ("sm__warps_active.avg.pct_of_peak_sustained_active",),
}
_SCALE = {"ns": 1e-6, "us": 1e-3, "ms": 1.0, "s": 1e3, "byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}


def read_capture(path):
    """Rows of a raw-page CSV as dicts ``{column: float or str}``; the unit row that follows the header scales the values."""
    with open(path) as f:
        lines = [ln for ln in f if ln.startswith('"')]
    rd = list(csv.reader(lines))
    if len(rd) < 3:
        return []
    head, units = rd[0], rd[1]
    out = []
    for rec in rd[2:]:
        row = {}
        for name, unit, val in zip(head, units, rec):
            try:
                row[name] = float(val.replace(",", "")) * _SCALE.get(unit, 1.0)
            except ValueError:
                row[name] = val
        out.append(row)
    return out


def pick(row, key):
    for name in METRICS[key]:
        if name in row and isinstance(row[name], float):
            return row[name]
    return None


def join(rows, order):
    """Group kernel rows into the calls of ``order`` (see the module text for the rule)."""
    groups, cur = [], None
    for r in rows:
        name = str(r.get("Kernel Name", ""))
        if "attn_fwd_kernel" in name or "attn_fwd_async" in name or "attn_bwd_row" in name:
            cur = []
            groups.append(cur)
        if cur is not None:
            cur.append(r)
    report = []
    for call, kernels in zip(order, groups):
        ms = sum(pick(k, "ms") or 0.0 for k in kernels)
        rd = sum(pick(k, "dram_read") or 0.0 for k in kernels)
        wr = sum(pick(k, "dram_write") or 0.0 for k in kernels)
        main = max(kernels, key=lambda k: pick(k, "ms") or 0.0)
        report.append(dict(call=call["call"], degree=call["degree"], kernels=len(kernels), ms=ms, dram_bytes=rd + wr,
                           model_bytes=call["model_bytes"], dram_over_model=(rd + wr) / max(call["model_bytes"], 1),
                           dram_pct=pick(main, "dram_pct"), regs=pick(main, "regs"), occupancy_pct=pick(main, "occupancy_pct"),
                           main_kernel=str(main.get("Kernel Name", ""))[:60]))
    return report


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 2:
        print(__doc__)
        return 2
    rows = read_capture(argv[0])
    with open(argv[1]) as f:
        order = json.load(f)
    rep = join(rows, order)
    if len(rep) != len(order):
        print(f"warning: {len(order)} calls in the order file, {len(rep)} matched in the capture")
    print(f"{'call':5s} {'deg':>4s} {'krn':>3s} {'ms':>8s} {'DRAM MB':>9s} {'model MB':>9s} {'ratio':>6s} {'DRAM %':>7s} {'regs':>5s} {'occ %':>6s}")
    for r in rep:
        f = lambda v, spec: format(v, spec) if v is not None else "-"                # noqa: E731
        print(f"{r['call']:5s} {r['degree']:4d} {r['kernels']:3d} {r['ms']:8.4f} {r['dram_bytes'] / 1e6:9.1f} {r['model_bytes'] / 1e6:9.1f} "
              f"{r['dram_over_model']:6.2f} {f(r['dram_pct'], '7.1f')} {f(r['regs'], '5.0f')} {f(r['occupancy_pct'], '6.1f')}")
    return rep


if __name__ == "__main__":
    main()

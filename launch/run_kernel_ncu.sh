#!/usr/bin/env bash
# Nsight Compute capture of the attention kernels on regular blocks (one GPU), then the report that sets measured DRAM bytes
# against the analytic model.  The workload runs once without the profiler first; the capture only starts if that run exits 0.
# Clocks are left alone (--clock-control none); the case is small (131,072 rows, about a dozen launches, a few metrics).
#   launch/run_kernel_ncu.sh [OUT_DIR] [extra arguments of gt_b200.bench.kernel_ncu, e.g. --degrees 1 16]
set -euo pipefail
cd "$(dirname "$0")/.."
OUT="${1:-ncu_out}"; shift || true
mkdir -p "$OUT"
METRICS=gpu__time_duration.sum,dram__bytes_read.sum,dram__bytes_write.sum,gpu__dram_throughput.avg.pct_of_peak_sustained_elapsed,launch__registers_per_thread,sm__warps_active.avg.pct_of_peak_sustained_active
WORKLOAD=(python -m gt_b200.bench.kernel_ncu --order "$OUT/kernel_ncu_order.json" "$@")
"${WORKLOAD[@]}" > "$OUT/plain.log" 2>&1 &&
ncu --profile-from-start off --clock-control none -k regex:attn_ --metrics "$METRICS" --csv --page raw \
    --log-file "$OUT/kernel_ncu.csv" "${WORKLOAD[@]}" > "$OUT/ncu.log" 2>&1
python -m gt_b200.bench.kernel_ncu_report "$OUT/kernel_ncu.csv" "$OUT/kernel_ncu_order.json" | tee "$OUT/report.txt"

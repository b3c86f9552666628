#!/usr/bin/env bash
# Re-measure the constants of the performance model on this machine (one GPU; the collective section needs all GPUs of the node).
#   launch/calibrate.sh [OUT.json]            writes the overlay read by gt_b200.perf.grid_select.load_constants
#   NGPU=8 launch/calibrate.sh                also measures the collectives over NGPU ranks
set -euo pipefail
cd "$(dirname "$0")/.."
OUT="${1:-gt_b200/perf/b200_constants.json}"
python -m gt_b200.bench.hw_constants --only hbm,gap,ew,gemm --out "$OUT"
python -m gt_b200.bench.kernel_constants --out "$OUT"
python -m gt_b200.bench.kernel_theory --out "${OUT%.json}_theory.json"
python -m gt_b200.bench.graph_constants --graph exphormer_arxiv --out "${OUT%.json}_graph_exphormer_arxiv.json"
if [ "${NGPU:-1}" -gt 1 ]; then
  python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "${PORT:-29533}" \
      -m gt_b200.bench.hw_constants --only coll --out "$OUT"
fi
python -m gt_b200.bench.validate_model

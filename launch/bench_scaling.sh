#!/usr/bin/env bash
# The headline benchmark at 1, 2, 4 and 8 GPUs of one node, this package and the reference arm; one JSON line per run.
#   launch/bench_scaling.sh [steps] [warmup] [extra bench.py flags, e.g. --comm p2p]
#   launch/bench_scaling.sh > lines.txt && python -m gt_b200.bench.check_regression --from_json lines.txt     # against the recorded times
set -euo pipefail
cd "$(dirname "$0")/.."
STEPS=${1:-20}; WARMUP=${2:-5}; shift $(( $# > 2 ? 2 : $# ))
for N in 1 2 4 8; do
  for IMPL in reference ours; do
    if [ "$N" = 1 ]; then
      python bench.py --impl "$IMPL" --gpus 1 --steps "$STEPS" --warmup "$WARMUP" "$@"
    else
      python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" --master-addr 127.0.0.1 --master-port $((29500 + N)) \
        bench.py --impl "$IMPL" --gpus "$N" --steps "$STEPS" --warmup "$WARMUP" "$@"
    fi
  done
done

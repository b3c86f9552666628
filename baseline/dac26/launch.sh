#!/usr/bin/env bash
# The DAC'26 baseline strategies on one node, one process per GPU (stock PyTorch operators, NCCL collectives).
#   baseline/dac26/launch.sh 4 --graph exphormer_arxiv --strategy gp_ag
#   baseline/dac26/launch.sh 8 --graph exphormer_arxiv --strategy gp_a2a          (needs the GPU count to divide the heads)
#   baseline/dac26/launch.sh 1 --graph exphormer_arxiv --strategy single
#   baseline/dac26/launch.sh 1 --graph exphormer_arxiv --micro                    (MM / SpMM / SDDMM on one device)
set -euo pipefail
GPUS=${1:?number of GPUs}; shift
cd "$(dirname "$0")/../.."
if [ "$GPUS" -le 1 ]; then
  exec python baseline/dac26/dac26_sga.py "$@"
fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29650}" \
    baseline/dac26/dac26_sga.py "$@"

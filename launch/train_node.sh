#!/usr/bin/env bash
# One node, one process per GPU.  Usage: launch/train_node.sh <gpus> [train_dist flags...]
#   launch/train_node.sh 8 --grid 4 2 --fused --synthetic exphormer_arxiv --bf16 --norm ln --cuda_graph --comm p2p
set -euo pipefail
GPUS=${1:?number of GPUs}; shift
cd "$(dirname "$0")/.."
export NCCL_NVLS_ENABLE=${NCCL_NVLS_ENABLE:-1}
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" \
    -m gt_b200.train.train_dist "$@"

#!/usr/bin/env bash
# Restart-from-checkpoint supervisor for one node: runs train_dist under torchrun and, when the run ends with an error (a rank
# died, a peer wait expired, PeerFailure from --heartbeat), starts it again from the last checkpoint, up to MAX_RESTARTS times.
#   launch/train_resilient.sh <gpus> <checkpoint.pt> [train_dist flags...]
#   MAX_RESTARTS=5 SAVE_EVERY=20 launch/train_resilient.sh 8 run.pt --grid 4 2 --fused --synthetic exphormer_arxiv --bf16 --norm ln \
#       --cuda_graph --comm p2p --epochs 500 --heartbeat 60
# <gpus> = 0 runs a single CPU process (tests).
set -uo pipefail
GPUS=${1:?number of GPUs (0 = one CPU process)}; CKPT=${2:?checkpoint file}; shift 2
MAX_RESTARTS=${MAX_RESTARTS:-3}
SAVE_EVERY=${SAVE_EVERY:-10}
cd "$(dirname "$0")/.."
attempt=0
while :; do
  resume=()
  if [ -f "$CKPT" ]; then resume=(--resume "$CKPT"); fi
  if [ "$GPUS" -le 0 ]; then
    python -m gt_b200.train.train_dist "$@" --save "$CKPT" --save_every "$SAVE_EVERY" "${resume[@]}"
  else
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" \
        -m gt_b200.train.train_dist "$@" --save "$CKPT" --save_every "$SAVE_EVERY" "${resume[@]}"
  fi
  rc=$?
  if [ $rc -eq 0 ]; then echo "[resilient] finished after $attempt restart(s)"; exit 0; fi
  attempt=$((attempt + 1))
  if [ $attempt -gt "$MAX_RESTARTS" ]; then echo "[resilient] giving up after $MAX_RESTARTS restarts (last exit code $rc)" >&2; exit $rc; fi
  echo "[resilient] run ended with exit code $rc; restart $attempt of $MAX_RESTARTS from ${CKPT} ($( [ -f "$CKPT" ] && echo found || echo 'no checkpoint yet' ))" >&2
  sleep "${RESTART_DELAY:-2}"
done

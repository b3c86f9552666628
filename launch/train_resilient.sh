#!/usr/bin/env bash
# Restart-from-checkpoint supervisor for one node: runs train_dist under torchrun and, when the run ends with an error (a rank
# died, a peer wait expired, PeerFailure from --heartbeat), starts it again from the last checkpoint, up to MAX_RESTARTS times.
#   launch/train_resilient.sh <gpus> <checkpoint.pt> [train_dist flags...]
#   MAX_RESTARTS=5 SAVE_EVERY=20 launch/train_resilient.sh 8 run.pt --grid 4 2 --fused --synthetic exphormer_arxiv --bf16 --norm ln \
#       --cuda_graph --comm p2p --epochs 500 --heartbeat 60
# A run that ends with an out-of-memory error is started again with per-layer activation checkpointing (--checkpoint), once: the
# model and its checkpoint files are the same with and without it.
# <gpus> = 0 runs a single CPU process (tests).
set -uo pipefail
GPUS=${1:?number of GPUs (0 = one CPU process)}; CKPT=${2:?checkpoint file}; shift 2
MAX_RESTARTS=${MAX_RESTARTS:-3}
SAVE_EVERY=${SAVE_EVERY:-10}
PYTHON=${PYTHON:-python}
cd "$(dirname "$0")/.."
ERRLOG=$(mktemp)
trap 'rm -f "$ERRLOG"' EXIT
attempt=0
extra=()
while :; do
  resume=()
  if [ -f "$CKPT" ]; then resume=(--resume "$CKPT"); fi
  if [ "$GPUS" -le 0 ]; then
    "$PYTHON" -m gt_b200.train.train_dist "$@" "${extra[@]}" --save "$CKPT" --save_every "$SAVE_EVERY" "${resume[@]}" 2> >(tee "$ERRLOG" >&2)
  else
    "$PYTHON" -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" \
        -m gt_b200.train.train_dist "$@" "${extra[@]}" --save "$CKPT" --save_every "$SAVE_EVERY" "${resume[@]}" 2> >(tee "$ERRLOG" >&2)
  fi
  rc=$?
  if [ $rc -eq 0 ]; then echo "[resilient] finished after $attempt restart(s)"; exit 0; fi
  sleep 0.2                                                  # let the copy of the error stream settle
  if [ ${#extra[@]} -eq 0 ] && grep -qi "out of memory" "$ERRLOG"; then
    extra=(--checkpoint)
    echo "[resilient] the run ran out of memory: next attempt with per-layer activation checkpointing (--checkpoint)" >&2
  fi
  attempt=$((attempt + 1))
  if [ $attempt -gt "$MAX_RESTARTS" ]; then echo "[resilient] giving up after $MAX_RESTARTS restarts (last exit code $rc)" >&2; exit $rc; fi
  echo "[resilient] run ended with exit code $rc; restart $attempt of $MAX_RESTARTS from ${CKPT} ($( [ -f "$CKPT" ] && echo found || echo 'no checkpoint yet' ))" >&2
  sleep "${RESTART_DELAY:-2}"
done

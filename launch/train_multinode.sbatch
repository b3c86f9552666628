#!/usr/bin/env bash
#SBATCH --job-name=gt_b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --time=00:30:00
# Multi-node launch under Slurm: one torchrun agent per node, 8 ranks each (one per B200).  Ranks are laid out so that a
# row group (P_o <= 8 consecutive ranks) stays inside an NVSwitch domain; see gt_b200/perf/grid_select.py placement().
#   sbatch --nodes 4 launch/train_multinode.sbatch --grid 4 8 --fused --data /data/papers100M_p32 --bf16 --norm ln
# With --comm p2p the groups whose ranks all sit on one node (here: the row groups) move their rows through peer memory, the
# groups that cross nodes (the column groups, the gradient all-reduce) stay on NCCL.
set -euo pipefail
cd "${SLURM_SUBMIT_DIR:-$(dirname "$0")/..}"
HEAD=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export NCCL_SOCKET_IFNAME=${NCCL_SOCKET_IFNAME:-^lo,docker}
srun --kill-on-bad-exit=1 python -m torch.distributed.run --nnodes="$SLURM_NNODES" --nproc-per-node 8 \
    --rdzv-backend c10d --rdzv-endpoint "$HEAD:${MASTER_PORT:-29500}" --rdzv-id "$SLURM_JOB_ID" \
    -m gt_b200.train.train_dist "$@"

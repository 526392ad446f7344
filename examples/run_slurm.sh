#!/bin/bash
#SBATCH --gpus-per-node=8
#SBATCH --ntasks-per-node=8
#SBATCH --time=00:10:00
# Multi-node launch under SLURM, one process per GPU (the single-box launcher is run_8.sh).
#
#   sbatch -N <nodes> run_slurm.sh <G_INTRA_R> <G_INTRA_C> <G_INTRA_D> <TRIAL_NUM> [train.py flags]
#
# Mirrors the reference's examples/run_4.sh: srun starts the tasks, get_rank.sh exports
# RANK / LOCAL_RANK from SLURM's variables, MASTER_ADDR is the first node of the allocation.
# Peer-memory (fused) collectives need every rank of a grid axis on one NVSwitch box; axes that
# cross nodes must use --comm nccl.
set -euo pipefail
if [ "$#" -lt 4 ]; then
  echo "Usage: sbatch -N <nodes> $0 <G_INTRA_R> <G_INTRA_C> <G_INTRA_D> <TRIAL_NUM> [train.py flags]"
  exit 1
fi
R=$1; C=$2; D=$3; TRIAL=$4; shift 4
HERE="$(cd "$(dirname "$0")" && pwd)"
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export MASTER_PORT=${MASTER_PORT:-29500}
export WORLD_SIZE=$((SLURM_JOB_NUM_NODES * GPUS_PER_NODE))
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1}
COMM=${COMM:-nccl}
OUT=${OUT_DIR:-.}/plexus_X${R}Y${C}Z${D}_${TRIAL}.txt
srun -N "$SLURM_JOB_NUM_NODES" -n "$WORLD_SIZE" --ntasks-per-node "$GPUS_PER_NODE" \
  "${HERE}/get_rank.sh" python "${HERE}/train.py" --G_intra_r "$R" --G_intra_c "$C" --G_intra_d "$D" \
  --gpus_per_node "$GPUS_PER_NODE" --num_epochs 10 --comm "$COMM" "$@" > "$OUT" 2>&1
python "${HERE}/parse_results.py" "$OUT" 2

#!/bin/bash
# Launch the training example on the 8 B200s of one NVSwitch box, one process per GPU.
#
#   ./run_8.sh <G_INTRA_R> <G_INTRA_C> <G_INTRA_D> <TRIAL_NUM> [extra train.py flags]
#   ./run_8.sh auto 0 --synthetic 2449029,60634000,100,47 --hidden_size 256
#
# The reference's launcher is a SLURM script for 4-GPU Perlmutter nodes (srun + a wrapper that
# exports RANK); on a single box torchrun provides RANK / LOCAL_RANK / WORLD_SIZE directly.
set -euo pipefail
GPUS=${GPUS:-8}
HERE="$(cd "$(dirname "$0")" && pwd)"
export MASTER_ADDR=127.0.0.1
export MASTER_PORT=${MASTER_PORT:-29500}
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1}
ulimit -c 0

if [ "${1:-}" = "auto" ]; then
  TRIAL=${2:-0}; shift 2 || true
  GRID_ARGS="--grid auto"; TAG="auto"
else
  if [ "$#" -lt 4 ]; then
    echo "Usage: $0 <G_INTRA_R> <G_INTRA_C> <G_INTRA_D> <TRIAL_NUM> [train.py flags] | $0 auto <TRIAL_NUM> [flags]"
    exit 1
  fi
  GRID_ARGS="--G_intra_r $1 --G_intra_c $2 --G_intra_d $3"; TAG="X$1Y$2Z$3"; TRIAL=$4; shift 4
fi
OUT=${OUT_DIR:-.}/plexus_${TAG}_${TRIAL}.txt
CMD="python -m torch.distributed.run --nnodes=1 --nproc-per-node ${GPUS} --master-addr ${MASTER_ADDR} --master-port ${MASTER_PORT} ${HERE}/train.py ${GRID_ARGS} --gpus_per_node ${GPUS} --num_epochs 10 --comm fused $*"
echo "$CMD > $OUT"
$CMD > "$OUT" 2>&1
python "${HERE}/parse_results.py" "$OUT" 2

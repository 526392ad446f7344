#!/bin/bash
# srun wrapper: torch.distributed reads RANK / LOCAL_RANK / WORLD_SIZE from the environment.
export RANK=${SLURM_PROCID:-0}
export LOCAL_RANK=${SLURM_LOCALID:-0}
ulimit -c 0
exec "$@"

#!/bin/bash
# Shared launcher: one rank per GPU of this node (or of every node of a SLURM job).
#   launch/common.sh <module> <config.yml>
# Multi-node: export MASTER_ADDR / MASTER_PORT / NNODES / NODE_RANK (or run under srun with the SLURM variables set).
set -euo pipefail
MODULE=$1
CONFIG=$2
GPUS_PER_NODE=${GPUS_PER_NODE:-$(nvidia-smi -L | wc -l)}
NNODES=${NNODES:-${SLURM_NNODES:-1}}
NODE_RANK=${NODE_RANK:-${SLURM_NODEID:-0}}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
export TOKENIZERS_PARALLELISM=false
exec python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$GPUS_PER_NODE" \
    --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" -m "$MODULE" --config "$CONFIG"

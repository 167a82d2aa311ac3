#!/bin/bash
#SBATCH --job-name=lm-engine-pretrain
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --exclusive
# sbatch launch/slurm_pretrain.sbatch configs/pretraining/dense-8b-fsdp.yml
export MASTER_ADDR=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
export MASTER_PORT=29500
export NCCL_NVLS_ENABLE=1
srun --kill-on-bad-exit=1 launch/pretrain.sh "$1"

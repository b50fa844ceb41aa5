#!/bin/bash
# Two nodes x 8 B200: pipeline stages across all 16 GPUs (reference test/multinode_trainer.slurm launches its trainer
# the same way on 2 x 8 GPUs).  Inside a node the fused DP / TP / EP kernels use NVLink peer memory; between nodes only
# the pipeline's NCCL send / recv cross the network, so PP is the dimension to put across nodes.
#SBATCH --job-name=pippy_b200
#SBATCH --nodes=2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH --cpus-per-task=64
#SBATCH --time=01:00:00

export PYTHONFAULTHANDLER=1
export NCCL_DEBUG=WARN
export LOGLEVEL=INFO

nodes=( $(scontrol show hostnames "$SLURM_JOB_NODELIST") )
head_node=${nodes[0]}
head_node_ip=$(srun --nodes=1 --ntasks=1 -w "$head_node" hostname --ip-address)

srun torchrun --nnodes 2 --nproc_per_node 8 \
     --rdzv_id "$SLURM_JOB_ID" --rdzv_backend c10d --rdzv_endpoint "$head_node_ip:29500" \
     examples/llama/train_llama.py --schedule zero_bubble --layers 32 --dim 4096 --heads 32 --ffn 11008 \
     --batch 64 --seq 4096 --microbatches 64

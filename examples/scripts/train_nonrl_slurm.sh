#!/bin/bash
# SFT / RM / DPO under SLURM: one task per node starts torchrun, which starts one process per GPU.
#SBATCH -J openrlhf_b200_sft
#SBATCH -N 2
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH -t 24:00:00
#SBATCH -o slurm-%j.out
set -x
nodes=($(scontrol show hostnames "$SLURM_JOB_NODELIST"))
head_addr=$(srun -N1 -n1 -w "${nodes[0]}" hostname --ip-address | awk '{print $1}')
# for reward-model or DPO training replace train_sft by train_rm / train_dpo (and the dataset keys)
srun torchrun --nnodes "$SLURM_JOB_NUM_NODES" --nproc-per-node 8 --rdzv-backend c10d --rdzv-endpoint "${head_addr}:29500" \
   -m openrlhf.cli.train_sft \
   --model.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.dataset ${DATA:-"synthetic://sft?n=65536&len=2048&vocab=150000"} --data.input_key input --data.output_key output \
   --data.max_len 4096 --train.batch_size 256 --train.micro_batch_size 4 --train.max_epochs 1 \
   --ds.zero_stage 2 --ds.packing_samples --adam.lr 5e-6 --model.gradient_checkpointing_enable \
   --ckpt.output_dir ./ckpt/sft_slurm --ckpt.save_steps 500 --ckpt.path ./ckpt/sft_slurm/state

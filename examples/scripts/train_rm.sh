#!/bin/bash
# Pairwise reward model (value head "score" on the base model, chosen || rejected in one packed batch).
set -x
torchrun --nnodes=1 --nproc-per-node ${GPUS:-8} --master-addr 127.0.0.1 --master-port 29500 -m openrlhf.cli.train_rm \
   --model.model_name_or_path ${MODEL:-qwen2.5-1.5b} \
   --data.dataset ${DATA:-"synthetic://preference?n=4096&len=512&vocab=150000"} --data.prompt_key prompt --data.chosen_key chosen --data.rejected_key rejected \
   --data.max_len 4096 --train.batch_size 128 --train.micro_batch_size 4 --train.max_epochs 1 \
   --ds.zero_stage 2 --ds.packing_samples --adam.lr 9e-6 --ckpt.output_dir ./ckpt/rm

#!/bin/bash
# DPO (policy + frozen reference on every rank; --model.ipo_enable / --model.label_smoothing select IPO / cDPO).
set -x
torchrun --nnodes=1 --nproc-per-node ${GPUS:-8} --master-addr 127.0.0.1 --master-port 29500 -m openrlhf.cli.train_dpo \
   --model.model_name_or_path ${MODEL:-llama3-8b} --ref.model_name_or_path ${MODEL:-llama3-8b} \
   --data.dataset ${DATA:-"synthetic://preference?n=4096&len=512&vocab=128000"} --data.prompt_key prompt --data.chosen_key chosen --data.rejected_key rejected \
   --data.max_len 4096 --train.batch_size 128 --train.micro_batch_size 2 --model.beta 0.1 \
   --ds.zero_stage 2 --ds.packing_samples --adam.lr 5e-7 --ckpt.output_dir ./ckpt/dpo

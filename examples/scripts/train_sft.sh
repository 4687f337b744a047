#!/bin/bash
# Supervised fine-tuning (SPMD: one rank per GPU under torchrun, ZeRO-2, packed samples).
set -x
torchrun --nnodes=1 --nproc-per-node ${GPUS:-8} --master-addr 127.0.0.1 --master-port 29500 -m openrlhf.cli.train_sft \
   --model.model_name_or_path ${MODEL:-qwen2.5-1.5b} \
   --data.dataset ${DATA:-"synthetic://sft?n=4096&len=512&vocab=150000"} --data.input_key input --data.output_key output \
   --data.max_len 4096 --train.batch_size 128 --train.micro_batch_size 4 --train.max_epochs 1 \
   --ds.zero_stage 2 --ds.packing_samples --adam.lr 5e-6 --lr_scheduler cosine_with_min_lr \
   --ckpt.output_dir ./ckpt/sft --ckpt.save_steps 200 --logger.logging_steps 1

#!/bin/bash
# LoRA fine-tuning of a mixture-of-experts model (adapters on all linear layers, MoE auxiliary loss on), followed by
# merging the adapters into the base weights.
set -x
torchrun --nnodes=1 --nproc-per-node ${GPUS:-8} --master-addr 127.0.0.1 --master-port 29500 -m openrlhf.cli.train_sft \
   --model.model_name_or_path ${MODEL:-qwen3-30b-a3b} --model.aux_loss_coef 0.001 \
   --data.dataset ${DATA:-"synthetic://sft?n=4096&len=512&vocab=150000"} --data.input_key input --data.output_key output \
   --data.max_len 2048 --train.batch_size 128 --train.micro_batch_size 2 \
   --ds.zero_stage 2 --ds.packing_samples --ds.lora.rank 64 --ds.lora.alpha 64 --adam.lr 5e-6 \
   --ckpt.output_dir ./ckpt/moe_lora
python -m openrlhf.cli.lora_combiner --model_path ${MODEL:-qwen3-30b-a3b} --lora_path ./ckpt/moe_lora --output_path ./ckpt/moe_merged

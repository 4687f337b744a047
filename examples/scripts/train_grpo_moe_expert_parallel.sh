#!/bin/bash
# GRPO on a mixture-of-experts policy (Qwen3-30B-A3B architecture) with expert parallelism over the 8 GPUs of a node:
# every GPU computes 16 of the 128 experts of each layer, token rows travel to their experts and back over NVLink peer
# memory, ZeRO-3 shards everything else (a rank gathers only the experts it computes).
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --ref.num_nodes 1 --ref.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.5 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-qwen3-30b-a3b} --ds.expert_parallel_size 8 --actor.aux_loss_coef 1e-3 \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=1024&vocab=150000"} --data.input_key input --data.label_key label \
   --reward.remote_url examples/python/math_reward_func.py \
   --algo.advantage.estimator group_norm --algo.kl.init_coef 1e-3 --algo.kl.use_loss --algo.kl.estimator k3 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 4096 --data.max_len 5120 \
   --train.batch_size 128 --train.micro_batch_size 1 --rollout.micro_batch_size 4 \
   --ds.zero_stage 3 --ds.packing_samples --actor.gradient_checkpointing_enable \
   --actor.adam.lr 1e-6 --ckpt.output_dir ./ckpt/grpo_moe

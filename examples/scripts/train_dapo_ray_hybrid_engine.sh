#!/bin/bash
# DAPO: asymmetric clip, dynamic filtering of all-equal-reward groups with replacement prompts, overlong penalty,
# token-level loss.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.6 \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=1024&vocab=150000"} --data.input_key input \
   --reward.remote_url examples/python/math_reward_func.py \
   --algo.advantage.estimator group_norm --algo.kl.init_coef 0 \
   --actor.eps_clip_low_high 0.2 0.28 --algo.dynamic_filtering_enable --algo.dynamic_filtering_range 0.01 0.99 \
   --reward.overlong_buffer_len 1024 --reward.overlong_penalty_factor 1.0 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 8192 --data.max_len 10240 \
   --train.batch_size 128 --train.micro_batch_size 2 --rollout.micro_batch_size 4 \
   --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 1e-6 --ckpt.output_dir ./ckpt/dapo

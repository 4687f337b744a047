#!/bin/bash
# GRPO with the hybrid engine on one 8xB200 node: every GPU hosts actor + rollout (+ reference), weights are shared.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.5 \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=512&vocab=150000"} --data.input_key input \
   --reward.remote_url examples/python/reward_func.py \
   --algo.advantage.estimator group_norm --algo.kl.init_coef 1e-3 --algo.kl.use_loss --algo.kl.estimator k3 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 2048 --data.max_len 4096 \
   --train.batch_size 128 --train.micro_batch_size 4 --rollout.micro_batch_size 8 \
   --ds.zero_stage 3 --ds.packing_samples --actor.adam.lr 5e-7 \
   --ckpt.output_dir ./ckpt/grpo --ckpt.path ./ckpt/grpo/checkpoints --ckpt.save_steps 20 --ckpt.max_num 3

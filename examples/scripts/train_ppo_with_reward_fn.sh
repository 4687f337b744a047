#!/bin/bash
# PPO with a critic and a Python reward function instead of a reward model: --reward.remote_url names a file that
# defines reward_func(queries, prompts, labels) -> {"rewards", "scores", "extra_logs"}.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --ref.num_nodes 1 --ref.num_gpus_per_node 8 \
   --critic.num_nodes 1 --critic.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.5 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=2048&len=512&vocab=150000"} --data.input_key input --data.label_key label \
   --reward.remote_url examples/python/reward_func.py \
   --algo.advantage.estimator gae --algo.advantage.gamma 1.0 --algo.advantage.lambd 0.95 --algo.kl.init_coef 1e-3 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 1 --rollout.max_new_tokens 1024 --data.max_len 2048 \
   --train.batch_size 128 --train.micro_batch_size 8 --rollout.micro_batch_size 16 --train.max_epochs 1 \
   --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 5e-7 --critic.adam.lr 9e-6 \
   --ckpt.output_dir ./ckpt/ppo_reward_fn

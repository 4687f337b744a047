#!/bin/bash
# PPO with a critic, hybrid engine on one 8xB200 node: every GPU hosts actor, critic, reference and a rollout engine.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --critic.num_nodes 1 --critic.num_gpus_per_node 8 \
   --ref.num_nodes 1 --ref.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.5 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-llama3-8b} --critic.model_name_or_path ${MODEL:-llama3-8b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=1024&vocab=128000"} --data.input_key input \
   --reward.remote_url examples/python/reward_func.py \
   --algo.advantage.estimator gae --algo.advantage.gamma 1.0 --algo.advantage.lambd 1.0 --algo.kl.init_coef 0.01 \
   --rollout.batch_size 1024 --rollout.n_samples_per_prompt 1 --rollout.max_new_tokens 1024 --data.max_len 2048 \
   --train.batch_size 128 --train.micro_batch_size 8 --rollout.micro_batch_size 16 \
   --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 5e-7 --critic.adam.lr 9e-6 \
   --ckpt.output_dir ./ckpt/ppo --ckpt.save_steps 20

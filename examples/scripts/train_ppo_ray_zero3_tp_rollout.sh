#!/bin/bash
# PPO with a critic, a reference and a reward model on one 8xB200 node, hybrid engine: all four models are sharded with
# ZeRO-3, pairs of GPUs form one tensor-parallel rollout engine (4 engines x TP 2), and every step the engines' shards
# are refreshed straight from the ZeRO-3 parameter slices by one copy kernel. A worker that dies makes the launcher
# restart the job from its last checkpoint (at most twice).
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --critic.num_nodes 1 --critic.num_gpus_per_node 8 \
   --ref.num_nodes 1 --ref.num_gpus_per_node 8 --reward.num_nodes 1 --reward.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 4 --vllm.tensor_parallel_size 2 --vllm.gpu_memory_utilization 0.5 --vllm.enable_sleep \
   --vllm.enable_prefix_caching \
   --actor.model_name_or_path ${MODEL:-llama3-8b} --critic.model_name_or_path ${MODEL:-llama3-8b} \
   --reward.model_name_or_path ${REWARD_MODEL:-llama3-8b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=1024&vocab=128000"} --data.input_key input \
   --algo.advantage.estimator gae --algo.advantage.gamma 1.0 --algo.advantage.lambd 0.95 --algo.kl.init_coef 0.01 \
   --rollout.batch_size 256 --rollout.n_samples_per_prompt 1 --rollout.max_new_tokens 1024 --data.max_len 2048 \
   --train.batch_size 128 --train.micro_batch_size 2 --rollout.micro_batch_size 8 \
   --ds.zero_stage 3 --ds.packing_samples --actor.gradient_checkpointing_enable \
   --actor.adam.lr 5e-7 --critic.adam.lr 9e-6 --ckpt.output_dir ./ckpt/ppo_zero3 --ckpt.path ./ckpt/ppo_zero3/checkpoints --ckpt.save_steps 20 \
   --train.max_restarts 2

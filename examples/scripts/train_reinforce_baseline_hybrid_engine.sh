#!/bin/bash
# REINFORCE++-baseline (no critic), hybrid engine, long context with context-parallel attention over 4 GPUs
# (--ds.ring_attn_size): the benchmark configuration of this repository at ring size 1 is bench.py.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --ref.num_nodes 1 --ref.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.6 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=2048&vocab=150000"} --data.input_key input \
   --reward.remote_url examples/python/math_reward_func.py \
   --algo.advantage.estimator reinforce_baseline --algo.kl.init_coef 1e-5 --algo.kl.use_loss --algo.kl.estimator k2 \
   --rollout.batch_size 64 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 16384 --data.max_len 18432 \
   --train.batch_size 512 --train.dynamic_batch_enable --train.max_tokens_per_gpu 32768 --rollout.max_tokens_per_gpu 65536 \
   --ds.zero_stage 2 --ds.packing_samples --ds.ring_attn_size ${RING:-4} --actor.adam.lr 5e-7 \
   --actor.gradient_checkpointing_enable --ckpt.output_dir ./ckpt/rfpp

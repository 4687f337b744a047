#!/bin/bash
# Asynchronous agent RL: rollout engines and trainers on disjoint GPUs, generation one step ahead of training,
# multi-turn environment from an agent function file.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 4 --ref.num_nodes 1 --ref.num_gpus_per_node 4 --train.colocate_actor_ref \
   --vllm.num_engines 4 --vllm.tensor_parallel_size 1 --train.async_enable --train.async_queue_size 1 \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=512&vocab=150000"} --data.input_key input \
   --train.agent_func_path examples/python/agent_func.py \
   --algo.advantage.estimator reinforce_baseline --algo.kl.init_coef 1e-5 --algo.kl.use_loss --algo.kl.estimator k2 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 2048 --data.max_len 8192 \
   --train.batch_size 128 --train.micro_batch_size 4 --rollout.micro_batch_size 8 \
   --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 5e-7 --ckpt.output_dir ./ckpt/agent

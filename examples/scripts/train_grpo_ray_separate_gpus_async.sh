#!/bin/bash
# GRPO with the rollout engines on their own GPUs: 4 GPUs train (ZeRO-3), 4 GPUs generate (2 engines x TP 2). The
# engines receive new weights over the weight-update group after every step, and with --train.async_enable generation
# of the next batch overlaps with training on the current one.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 4 --ref.num_nodes 1 --ref.num_gpus_per_node 4 --train.colocate_actor_ref \
   --vllm.num_engines 2 --vllm.tensor_parallel_size 2 --vllm.gpu_memory_utilization 0.9 --vllm.enable_prefix_caching \
   --train.async_enable --train.async_queue_size 1 \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=512&vocab=150000"} --data.input_key input --data.label_key label \
   --reward.remote_url examples/python/math_reward_func.py \
   --algo.advantage.estimator group_norm --algo.kl.init_coef 1e-3 --algo.kl.use_loss --algo.kl.estimator k3 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 2048 --data.max_len 2560 \
   --train.batch_size 128 --train.micro_batch_size 2 --rollout.micro_batch_size 8 \
   --ds.zero_stage 3 --ds.packing_samples --actor.adam.lr 1e-6 --ckpt.output_dir ./ckpt/grpo_async

#!/bin/bash
# ProRL-v2 style math RL: REINFORCE++-baseline, decoupled clipping, dynamic filtering of prompts whose n samples are
# all right or all wrong, and the stop-properly penalty that scales the reward of responses cut off at the length
# limit. The math grader lives in examples/python/math_reward_func.py.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --ref.num_nodes 1 --ref.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.6 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=4096&len=1024&vocab=150000"} --data.input_key input --data.label_key label \
   --reward.remote_url examples/python/math_reward_func.py --reward.stop_properly_penalty_coef 0.0 \
   --algo.advantage.estimator reinforce_baseline --algo.kl.init_coef 1e-4 --algo.kl.use_loss --algo.kl.estimator k2 \
   --algo.dynamic_filtering_enable --algo.dynamic_filtering_range 0.0 1.0 \
   --actor.eps_clip_low_high 0.2 0.27 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 8192 --data.max_len 9216 \
   --train.batch_size 1024 --train.dynamic_batch_enable --train.max_tokens_per_gpu 32768 --rollout.max_tokens_per_gpu 65536 \
   --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 1e-6 --actor.gradient_checkpointing_enable \
   --ckpt.output_dir ./ckpt/prorl_v2

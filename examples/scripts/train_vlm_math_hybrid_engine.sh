#!/bin/bash
# Vision-language RL (Qwen2-VL architecture): REINFORCE++-baseline on image + text prompts with a rule reward.
# Dataset rows: {"prompt": "<image> Find x.", "images": ["/path/or/url/or/base64"], "label": "3"}; the processor
# expands every image into its placeholder tokens, the rollout engine prefills with the vision tower's embeddings
# and M-RoPE positions, and the trainer re-runs the tower on the stored patches. --actor.freeze_visual_encoder
# trains only the language model.
set -x
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --ref.num_nodes 1 --ref.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.6 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-qwen2-vl-2b} --actor.freeze_visual_encoder \
   --data.prompt_dataset ${DATA:-"synthetic://vlm_prompts?n=4096&len=256&vocab=150000&image=448"} \
   --data.input_key input --data.label_key label --data.image_key images --data.max_images_per_prompt 1 \
   --reward.remote_url examples/python/math_reward_func.py \
   --algo.advantage.estimator reinforce_baseline --algo.kl.init_coef 0 --algo.kl.use_loss --algo.kl.estimator k2 \
   --rollout.batch_size 128 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 2048 --data.max_len 4096 \
   --train.batch_size 1024 --train.micro_batch_size 4 --rollout.micro_batch_size 8 \
   --ds.zero_stage 2 --actor.adam.lr 2e-6 --actor.gradient_checkpointing_enable \
   --ckpt.output_dir ./ckpt/vlm_rl --ckpt.save_steps 5 --ckpt.path ./ckpt/vlm_rl/state

#!/bin/bash
# RL under SLURM. The controller of this framework needs no cluster daemon: it starts one worker process per GPU of the
# node it runs on (an 8 x B200 node holds policy, reference and rollout engine of models up to ~70B with ZeRO-3), so
# the job asks for one whole node. The SPMD trainers (train_nonrl_slurm.sh) span nodes through torchrun.
#SBATCH -J openrlhf_b200_rl
#SBATCH -N 1
#SBATCH --ntasks-per-node=1
#SBATCH --gpus-per-node=8
#SBATCH -t 48:00:00
#SBATCH -o slurm-%j.out
set -x
srun python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 8 --ref.num_nodes 1 --ref.num_gpus_per_node 8 --train.colocate_all \
   --vllm.num_engines 8 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.6 --vllm.enable_sleep \
   --actor.model_name_or_path ${MODEL:-qwen2.5-7b} \
   --data.prompt_dataset ${DATA:-"synthetic://prompts?n=8192&len=1024&vocab=150000"} --data.input_key input \
   --reward.remote_url examples/python/math_reward_func.py \
   --algo.advantage.estimator reinforce_baseline --algo.kl.init_coef 1e-4 --algo.kl.use_loss --algo.kl.estimator k2 \
   --rollout.batch_size 256 --rollout.n_samples_per_prompt 8 --rollout.max_new_tokens 4096 --data.max_len 5120 \
   --train.batch_size 2048 --train.micro_batch_size 4 --rollout.micro_batch_size 8 \
   --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 1e-6 --ckpt.output_dir ./ckpt/rl_slurm

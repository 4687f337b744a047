#!/bin/bash
# RL launcher on 2 GPUs with tensor-parallel training (--ds.tensor_parallel_size 2): both workers train one shard each,
# see the same samples, and the rollout engines are refreshed from the gathered shards.
set -e
cd "$(dirname "$0")/../.."
OUT=${1:-/tmp/cli_ppo_tp_out}
python -m openrlhf.cli.train_ppo_ray \
   --actor.num_nodes 1 --actor.num_gpus_per_node 2 --ref.num_nodes 1 --ref.num_gpus_per_node 2 --train.colocate_all \
   --vllm.num_engines 2 --vllm.tensor_parallel_size 1 --vllm.gpu_memory_utilization 0.3 \
   --actor.model_name_or_path tiny-qwen2-gqa --ds.tensor_parallel_size 2 \
   --data.prompt_dataset "synthetic://prompts?n=64&len=24&vocab=2000" --data.input_key input --data.label_key label \
   --reward.remote_url examples/python/reward_func.py \
   --algo.advantage.estimator reinforce_baseline --algo.kl.init_coef 1e-3 --algo.kl.use_loss --algo.kl.estimator k2 \
   --rollout.batch_size 8 --rollout.n_samples_per_prompt 4 --rollout.max_new_tokens 32 --data.max_len 128 \
   --train.batch_size 16 --train.micro_batch_size 4 --rollout.micro_batch_size 8 --train.max_epochs 1 \
   --train.num_episodes 1 --data.max_samples 16 --ds.zero_stage 2 --ds.packing_samples --actor.adam.lr 1e-5 \
   --ckpt.output_dir "$OUT"
test -f "$OUT/config.json"
python - "$OUT" <<'PY'
import json, sys
cfg = json.load(open(sys.argv[1] + "/config.json"))
assert cfg["num_attention_heads"] == 4 and cfg["intermediate_size"] == 512, cfg     # exported in the full layout
print("CLI_PPO_TP_OK")
PY

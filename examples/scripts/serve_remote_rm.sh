#!/bin/bash
# HTTP reward server: POST /get_reward {"query": [...]} -> {"rewards": [...], "scores": [...], "extra_logs": {...}}
set -x
python -m openrlhf.cli.serve_rm --reward.model_name_or_path ${RM:-./ckpt/rm} --port 5000 --data.max_len 8192 --batch_size 16

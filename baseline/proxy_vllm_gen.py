"""Reference-dataflow proxy, generation phase: vLLM (as installed in the image) on the benchmark workload of bench.py:
16 prompts x 512 tokens, n = 8 samples, 2048 new tokens each, EOS ignored, Qwen2.5-1.5B architecture with dummy
weights, prefix caching on, CUDA graphs on. Not the reference itself (its launcher needs Ray and DeepSpeed, which the
image lacks): the rollout engine the reference would drive, timed alone on one GPU.

    python baseline/proxy_vllm_gen.py
"""
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from openrlhf_b200.models.config import PRESETS
cfg = PRESETS["qwen2.5-1.5b"]
d = tempfile.mkdtemp()
cfg.save_pretrained(d)
c = json.load(open(d + "/config.json")); c.pop("head_dim", None); c.pop("attention_bias", None)
c["sliding_window"] = None; c["use_sliding_window"] = False; c["max_window_layers"] = 28
json.dump(c, open(d + "/config.json", "w"))
from vllm import LLM, SamplingParams
t0 = time.time()
llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", gpu_memory_utilization=0.6,
          max_model_len=2560, max_num_seqs=128, enable_prefix_caching=True)
print("engine up in", time.time() - t0, flush=True)
g = torch.Generator().manual_seed(0)
def run(new):
    prompts = [{"prompt_token_ids": torch.randint(0, 150000, (512,), generator=g).tolist()} for _ in range(16)]
    sp = SamplingParams(n=8, temperature=1.0, max_tokens=new, ignore_eos=True, detokenize=False, logprobs=0)
    torch.cuda.synchronize(); t = time.time()
    outs = llm.generate(prompts, sp, use_tqdm=False)
    torch.cuda.synchronize(); dt = time.time() - t
    n = sum(len(o.token_ids) for r in outs for o in r.outputs)
    return dt, n
run(64)
dt, n = run(2048)
print(f"VLLM_PROXY generation 16x512 prompts n=8 2048 new: {dt:.2f} s, {n} tokens, {n/dt:.0f} tok/s", flush=True)

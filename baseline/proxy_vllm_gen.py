"""Reference-dataflow proxy, generation phase: vLLM (as installed in the image) on a benchmark workload of bench.py
(default: 16 prompts x 512 tokens, n = 8 samples, 2048 new tokens each, EOS ignored, Qwen2.5-1.5B architecture) with
dummy weights, prefix caching on, CUDA graphs on. Not the reference itself (its launcher needs Ray and DeepSpeed, which
the image lacks): the rollout engine the reference would drive, timed alone on one GPU.

    python baseline/proxy_vllm_gen.py [model preset] [prompts] [prompt length] [n] [new tokens]
    python baseline/proxy_vllm_gen.py qwen2.5-7b 8 512 8 1024      # the per-GPU share of the GRPO config
"""
import json
import os
import sys
import tempfile
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
from openrlhf_b200.models.config import PRESETS
argv = sys.argv[1:] + [None] * 5
MODEL = argv[0] or "qwen2.5-1.5b"
P, PLEN, NS, NEW = (int(v) if v else d for v, d in zip(argv[1:5], (16, 512, 8, 2048)))
cfg = PRESETS[MODEL]
d = tempfile.mkdtemp()
cfg.save_pretrained(d)
c = json.load(open(d + "/config.json")); c.pop("head_dim", None); c.pop("attention_bias", None)
c["sliding_window"] = None; c["use_sliding_window"] = False; c["max_window_layers"] = cfg.num_hidden_layers
json.dump(c, open(d + "/config.json", "w"))
from vllm import LLM, SamplingParams
t0 = time.time()
llm = LLM(model=d, load_format="dummy", skip_tokenizer_init=True, dtype="bfloat16", gpu_memory_utilization=0.6,
          max_model_len=PLEN + NEW, max_num_seqs=P * NS, enable_prefix_caching=True)
print("engine up in", time.time() - t0, flush=True)
g = torch.Generator().manual_seed(0)
def run(new):
    prompts = [{"prompt_token_ids": torch.randint(0, 150000, (PLEN,), generator=g).tolist()} for _ in range(P)]
    sp = SamplingParams(n=NS, temperature=1.0, max_tokens=new, ignore_eos=True, detokenize=False, logprobs=0)
    torch.cuda.synchronize(); t = time.time()
    outs = llm.generate(prompts, sp, use_tqdm=False)
    torch.cuda.synchronize(); dt = time.time() - t
    n = sum(len(o.token_ids) for r in outs for o in r.outputs)
    return dt, n
run(64)
dt, n = run(NEW)
print(f"VLLM_PROXY {MODEL} generation {P}x{PLEN} prompts n={NS} {NEW} new: {dt:.2f} s, {n} tokens, {n/dt:.0f} tok/s",
      flush=True)

"""Reference-dataflow proxy, training side: the HF Qwen2 model class the reference instantiates (Qwen2.5-1.5B
architecture, random weights, bf16) with flash-attn 2 on a packed batch of 4 x 2560 tokens, fp32 log-softmax of the
logits as in the reference's Actor.forward, fused torch AdamW. Times one forward + backward micro-batch, one optimizer
step and one no-grad forward on one GPU.

    python baseline/proxy_hf_train.py
"""
import time

import torch
from transformers import Qwen2Config, Qwen2ForCausalLM
cfg = Qwen2Config(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_hidden_layers=28, num_attention_heads=12,
                  num_key_value_heads=2, max_position_embeddings=32768, rope_theta=1e6, tie_word_embeddings=True, rms_norm_eps=1e-6)
cfg._attn_implementation = "flash_attention_2"
torch.manual_seed(0)
with torch.device("cuda"):
    m = Qwen2ForCausalLM(cfg).to(torch.bfloat16)
m.train()
opt = torch.optim.AdamW(m.parameters(), lr=1e-6, fused=True)
T, n = 2560, 4
ids = torch.randint(0, 150000, (1, n * T), device="cuda")
pos = torch.arange(T, device="cuda").repeat(n)[None]
cu = torch.arange(0, (n + 1) * T, T, device="cuda", dtype=torch.int32)
def step():
    out = m(input_ids=ids, position_ids=pos, cu_seq_lens_q=cu, cu_seq_lens_k=cu, max_length_q=T, max_length_k=T, use_cache=False)
    logits = out.logits.float()
    lp = torch.log_softmax(logits[0, :-1], -1).gather(-1, ids[0, 1:, None]).squeeze(-1)
    (-lp.mean()).backward()
for _ in range(3): step()
torch.cuda.synchronize(); t = time.time()
for _ in range(5): step()
torch.cuda.synchronize(); dt = (time.time() - t) / 5
opt.step(); torch.cuda.synchronize(); t = time.time(); opt.step(); torch.cuda.synchronize(); do = time.time() - t
print(f"HF_PROXY train micro-batch 4x2560 (HF Qwen2 + flash-attn 2 packed, fp32 log-softmax): {dt*1e3:.1f} ms fwd+bwd, fused AdamW step {do*1e3:.1f} ms", flush=True)
with torch.no_grad():
    torch.cuda.synchronize(); t = time.time()
    for _ in range(5):
        out = m(input_ids=ids, position_ids=pos, cu_seq_lens_q=cu, cu_seq_lens_k=cu, max_length_q=T, max_length_k=T, use_cache=False)
        lp = torch.log_softmax(out.logits.float()[0, :-1], -1).gather(-1, ids[0, 1:, None])
    torch.cuda.synchronize(); print(f"HF_PROXY no-grad forward 4x2560: {(time.time()-t)/5*1e3:.1f} ms", flush=True)

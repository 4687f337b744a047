"""Tensor-parallel rollout engine on N GPUs against the single-GPU engine with the same weights: greedy tokens and
their log-probs."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    import dataclasses

    from openrlhf_b200.models.config import PRESETS
    from openrlhf_b200.models.transformer import TransformerLM
    from openrlhf_b200.ops import _lib
    from openrlhf_b200.rollout.engine import RolloutEngine, SamplingParams
    from openrlhf_b200.rollout.tp_engine import make_tp_engine

    cfg = dataclasses.replace(PRESETS["tiny-qwen2"], num_attention_heads=4, num_key_value_heads=2, hidden_size=512,
                              intermediate_size=1024, num_hidden_layers=3, head_dim=128)
    full = TransformerLM(cfg, device="cuda", seed=0, init_std=0.05)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (37, 200, 5, 129)]
    sp = SamplingParams(temperature=0.0, max_tokens=24, n=2, logprobs=1, ignore_eos=True)
    ref = RolloutEngine(full, max_num_seqs=16, max_model_len=512, num_pages=64, use_cuda_graph=True)
    out_ref = ref.generate(prompts, sp)
    eng = make_tp_engine(cfg, full.flat, None, max_num_seqs=16, max_model_len=512, num_pages=64, use_cuda_graph=True)
    out_tp = eng.generate(prompts, sp)
    torch.cuda.synchronize()
    _lib.check_status()
    tot = same = 0
    worst = 0.0
    for a, b in zip(out_ref, out_tp):
        for ca, cb in zip(a.outputs, b.outputs):
            n = min(len(ca.token_ids), len(cb.token_ids))
            # compare up to the first divergence (bf16 summation order differs between TP=1 and TP=2)
            k = next((i for i in range(n) if ca.token_ids[i] != cb.token_ids[i]), n)
            tot += n
            same += k
            for i in range(k):
                worst = max(worst, abs(ca.logprob_values[i] - cb.logprob_values[i]))
    # every rank must have produced the same tokens
    mine = torch.tensor([t for o in out_tp for c in o.outputs for t in c.token_ids], device="cuda")
    other = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(other, mine)
    assert all(torch.equal(other[0], t) for t in other), "TP ranks sampled different tokens"
    print(f"rank {rank}: {same}/{tot} greedy tokens equal before first divergence, max |dlogp| {worst:.3e}", flush=True)
    # a random-init model has many near-ties, so greedy paths may part ways after a while; what must hold is that the
    # common prefix is substantial and that log-probs agree on it
    assert same >= 0.5 * tot and worst < 0.1, (same, tot, worst)
    # stochastic sampling also stays in lockstep across ranks
    sp2 = SamplingParams(temperature=1.0, max_tokens=16, n=2, logprobs=1, ignore_eos=True)
    o2 = eng.generate(prompts, sp2)
    mine = torch.tensor([t for o in o2 for c in o.outputs for t in c.token_ids], device="cuda")
    other = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(other, mine)
    assert all(torch.equal(other[0], t) for t in other), "TP ranks drew different samples"
    dist.barrier()
    if rank == 0:
        print("TP_ROLLOUT_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()

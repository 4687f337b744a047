"""The reward-model server: its proxy scores text with the reward model, and the HTTP route returns the contract the
remote-reward client of the RL launcher expects ({"rewards", "scores", "extra_logs"})."""
import torch


def _proxy():
    from openrlhf_b200.cli import flags as F
    from openrlhf_b200.cli.serve_rm import RewardModelProxy, build_parser

    args = F.finalize(build_parser(), ["--reward.model_name_or_path", "tiny-llama", "--data.max_len", "64",
                                       "--batch_size", "2", "--ds.packing_samples"])
    return RewardModelProxy(args)


def test_proxy_scores_match_the_reward_model_and_batching_is_invisible():
    proxy = _proxy()
    queries = ["a short query", "a somewhat longer query with more words in it", "third"]
    got = proxy.get_reward(queries)
    assert len(got) == 3 and all(isinstance(x, float) and x == x for x in got)
    enc = proxy.tokenizer(queries, return_tensors="pt", add_special_tokens=False, max_length=64, padding=True,
                          truncation=True)
    with torch.no_grad():
        want = proxy.reward_model(enc["input_ids"], enc["attention_mask"]).float().tolist()
    assert max(abs(a - b) for a, b in zip(got, want)) < 5e-2          # batches of 2 + 1 vs one batch of 3 (bf16)


def test_http_route_returns_the_remote_reward_contract():
    from fastapi.testclient import TestClient

    from openrlhf_b200.cli.serve_rm import build_app

    proxy = _proxy()
    client = TestClient(build_app(proxy))
    r = client.post("/get_reward", json={"query": ["hello world", "x y z"], "prompts": ["hello", "x"], "labels": ["", ""]})
    assert r.status_code == 200
    body = r.json()
    assert set(body) == {"rewards", "scores", "extra_logs"} and len(body["rewards"]) == 2
    assert body["rewards"] == body["scores"] == body["extra_logs"]["dummy_scores"]

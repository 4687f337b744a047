"""A user of the reference switches by import path only: the loss-aggregation API under ``openrlhf.*`` gives the values
that the reference's own loss-aggregation scenarios expect (hand-computed here from the scenario tensors; the
scenarios are those of the reference's tests/test_loss_aggregation.py, read as text)."""
import pytest
import torch

from openrlhf.models.loss import PolicyLoss, aggregate_loss
from openrlhf.utils.loss_utils import get_loss_batch_info, iter_grad_accum_global_norm


@pytest.mark.parametrize("token_level,loss,mask,split,expected", [
    # global token mean: (1 + 2 + 3 + 4 + 5 + 7) / 6
    (True, [[1., 2., 0.], [3., 4., 5.], [7., 0., 0.]], [[1., 1., 0.], [1., 1., 1.], [1., 0., 0.]], 2, 22. / 6.),
    # mean over sequences of per-sequence token means: (2 + 3 + 8) / 3
    (False, [[1., 3., 9.], [2., 4., 0.], [8., 0., 0.]], [[1., 1., 0.], [1., 1., 0.], [1., 0., 0.]], 2, 13. / 3.),
])
def test_two_data_parallel_ranks_average_to_the_global_value(token_level, loss, mask, split, expected):
    loss, mask = torch.tensor(loss), torch.tensor(mask)
    whole = aggregate_loss(loss, mask, token_level_loss=token_level)
    assert whole.item() == pytest.approx(expected)
    norm = dict(batch_num_tokens=mask.sum()) if token_level else dict(global_batch_size=torch.tensor(float(len(mask))))
    halves = [aggregate_loss(loss[s], mask[s], token_level_loss=token_level, dp_size=2, **norm)
              for s in (slice(0, split), slice(split, None))]
    # the engine averages gradients over data-parallel ranks; the dp_size factor compensates for that
    assert ((halves[0] + halves[1]) / 2).item() == pytest.approx(expected)


def test_fully_masked_sequences_do_not_count_as_samples():
    loss, mask = torch.tensor([[1., 3.], [5., 7.]]), torch.tensor([[1., 1.], [0., 0.]])
    info = get_loss_batch_info(strategy=object(), loss_mask=mask)
    assert float(info["global_batch_size"]) == 1.0
    assert aggregate_loss(loss, mask, token_level_loss=False, **info).item() == pytest.approx(2.0)


def test_policy_loss_sharded_over_two_ranks_equals_the_full_batch():
    logp = torch.tensor([[-0.20, -0.40, -0.10], [-0.70, -0.30, -0.20], [-0.60, -0.10, -0.50]])
    old = logp - torch.tensor([[0.03, -0.04, 0.01], [0.02, 0.05, -0.03], [0.04, 0.0, -0.02]])
    adv = torch.tensor([[1.0, -0.5, 0.0], [0.3, -1.2, 0.5], [1.5, 0.0, -0.7]])
    mask = torch.tensor([[1., 1., 0.], [1., 1., 1.], [1., 0., 1.]])
    fn = PolicyLoss(clip_eps_low=0.2, clip_eps_high=0.2)
    full = fn(logp, old, adv, action_mask=mask)[0]
    # by hand: no ratio leaves [0.8, 1.2], so the loss is -mean(ratio * advantage) over the 7 masked tokens
    ratio = (logp - old).exp()
    assert full.item() == pytest.approx(float(-(ratio * adv * mask).sum() / mask.sum()), rel=1e-6)
    parts = [fn(logp[s], old[s], adv[s], action_mask=mask[s], dp_size=2, batch_num_tokens=mask.sum())[0]
             for s in (slice(0, 2), slice(2, 3))]
    assert ((parts[0] + parts[1]) / 2).item() == pytest.approx(full.item(), rel=1e-6)


def test_ppo_kl_metric_is_the_policy_ratio_even_with_rollout_correction_and_is_not_clamped():
    fn = PolicyLoss(enable_vllm_is_correction=True, vllm_is_truncated_threshold=[0.1, 10.0],
                    vllm_is_correction_type="tis")
    logp, old, rollout = torch.tensor([[-0.2, -0.4]]), torch.tensor([[-0.3, -0.1]]), torch.tensor([[-1.3, -1.1]])
    _, _, ppo_kl, vllm_kl = fn(logp, old, torch.ones(1, 2), action_mask=torch.ones(1, 2), rollout_log_probs=rollout)
    assert ppo_kl.item() == pytest.approx(0.1) and vllm_kl.item() == pytest.approx(-1.0)
    _, _, far, _ = PolicyLoss()(torch.tensor([[100.0]]), torch.zeros(1, 1), torch.ones(1, 1), action_mask=torch.ones(1, 1))
    assert far.item() == pytest.approx(-100.0)


def test_gradient_accumulation_window_is_normalised_by_its_global_token_count():
    micro = [(torch.tensor([[1., 2., 0.]]), torch.tensor([[1., 1., 0.]])),                       # 2 tokens
             (torch.tensor([[3., 4., 5.], [6., 7., 0.]]), torch.tensor([[1., 1., 1.], [1., 1., 0.]]))]  # 5 tokens
    gas, total = 2, 0.0
    emitted = list(iter_grad_accum_global_norm(micro, strategy=object(), accumulated_gradient=gas,
                                               mask_fn=lambda item: item[1]))
    assert len(emitted) == 2
    for (loss, mask), info in emitted:
        assert float(info["batch_num_tokens"]) == pytest.approx(7 / gas)          # window count, folded by gas
        norm = {k: v for k, v in info.items() if k != "global_batch_size"}
        total = total + aggregate_loss(loss, mask, **norm) / gas                  # the engine scales by 1 / gas
    assert float(total) == pytest.approx(28. / 7.)                                # one token mean over the window
    per_micro = (aggregate_loss(*micro[0]) + aggregate_loss(*micro[1])) / 2
    assert float(per_micro) != pytest.approx(28. / 7.)                            # (1.5 + 5) / 2: not the same thing


def test_reference_import_paths_resolve_to_this_package():
    """Module paths and public names a user of the reference imports (its __init__ export lists, the places its RL
    utilities live, the strategy class name) resolve to the same module objects as this package's own paths."""
    import importlib

    expected = {
        "openrlhf.models": ["Actor", "SFTLoss", "DPOLoss", "GPTLMLoss", "LogExpLoss", "PairWiseLoss", "PolicyLoss",
                            "ValueLoss", "aggregate_loss", "get_llm_for_sequence_regression"],
        "openrlhf.datasets": ["PromptDataset", "RewardDataset", "SFTDataset"],
        "openrlhf.utils": ["extract_boxed_answer", "grade_answer", "get_strategy", "get_tokenizer"],
        "openrlhf.utils.utils": ["get_strategy", "get_tokenizer"],
        "openrlhf.utils.agent": ["AgentExecutorBase", "AgentInstanceBase"],
        "openrlhf.utils.deepspeed": ["DeepspeedStrategy"],
        "openrlhf.trainer.ppo_utils": ["AdaptiveKLController", "Experience", "FixedKLController", "NaiveReplayBuffer",
                                       "apply_length_penalties", "apply_overlong_penalty",
                                       "apply_stop_properly_penalty", "balance_experiences", "make_experience_batch",
                                       "split_experience_batch"],
        "openrlhf.trainer.ppo_utils.experience_maker": [],
        "openrlhf.trainer.ppo_utils.samples_generator": ["SamplesGenerator"],
        "openrlhf.trainer.ppo_trainer": ["PPOTrainer"],
        "openrlhf.trainer.ppo_trainer_async": ["PPOTrainerAsync"],
        "openrlhf.trainer.sft_trainer": ["SFTTrainer"],
        "openrlhf.trainer.rm_trainer": ["RewardModelTrainer"],
        "openrlhf.trainer.dpo_trainer": ["DPOTrainer"],
        "openrlhf.trainer.ray": ["batch_vllm_engine_call"],
        "openrlhf.trainer.ray.launcher": ["RayActorGroup"],
    }
    for path, names in expected.items():
        mod = importlib.import_module(path)
        missing = [n for n in names if not hasattr(mod, n)]
        assert not missing, (path, missing)
    import openrlhf.trainer.ppo_utils.experience as old_path
    import openrlhf_b200.rl.experience as new_path
    from openrlhf.utils.deepspeed import DeepspeedStrategy
    from openrlhf_b200.utils.strategy import Strategy

    assert old_path is new_path and DeepspeedStrategy is Strategy

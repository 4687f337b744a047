"""RL core on the host: experience containers, replay buffer, KL controllers, length penalties, advantage estimators,
sample generation and experience making (the reference keeps these under openrlhf/trainer/ppo_utils/)."""
from .experience import Experience, balance_experiences, make_experience_batch, split_experience_batch  # noqa: F401
from .kl_controller import AdaptiveKLController, FixedKLController  # noqa: F401
from .length_penalty import apply_length_penalties, apply_overlong_penalty, apply_stop_properly_penalty  # noqa: F401
from .replay_buffer import NaiveReplayBuffer  # noqa: F401

__all__ = [
    "AdaptiveKLController", "Experience", "FixedKLController", "NaiveReplayBuffer", "apply_length_penalties",
    "apply_overlong_penalty", "apply_stop_properly_penalty", "balance_experiences", "make_experience_batch",
    "split_experience_batch",
]

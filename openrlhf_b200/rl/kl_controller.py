"""KL coefficient controllers (fixed and adaptive, Ziegler et al. 2019), as in
openrlhf/trainer/ppo_utils/kl_controller.py:4-29."""
from __future__ import annotations


class FixedKLController:
    def __init__(self, kl_coef: float):
        self.value = kl_coef

    def update(self, current: float, n_steps: int) -> None:
        return None


class AdaptiveKLController:
    """beta <- beta * (1 + clip(kl/target - 1, -0.2, 0.2) * n_steps / horizon)"""

    def __init__(self, init_kl_coef: float, target: float, horizon: int):
        self.value = init_kl_coef
        self.target = target
        self.horizon = horizon

    def update(self, current: float, n_steps: int) -> None:
        err = min(max(current / self.target - 1.0, -0.2), 0.2)
        self.value *= 1.0 + err * n_steps / self.horizon

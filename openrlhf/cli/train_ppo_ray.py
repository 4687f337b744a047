"""``python -m openrlhf.cli.train_ppo_ray`` -> ``openrlhf_b200.cli.train_ppo_ray``."""
import runpy

from openrlhf_b200.cli.train_ppo_ray import *  # noqa: F401,F403

if __name__ == "__main__":
    runpy.run_module("openrlhf_b200.cli.train_ppo_ray", run_name="__main__")

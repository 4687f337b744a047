"""``python -m openrlhf.cli.train_dpo`` -> ``openrlhf_b200.cli.train_dpo``."""
import runpy

from openrlhf_b200.cli.train_dpo import *  # noqa: F401,F403

if __name__ == "__main__":
    runpy.run_module("openrlhf_b200.cli.train_dpo", run_name="__main__")

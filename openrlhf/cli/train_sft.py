"""``python -m openrlhf.cli.train_sft`` -> ``openrlhf_b200.cli.train_sft``."""
import runpy

from openrlhf_b200.cli.train_sft import *  # noqa: F401,F403

if __name__ == "__main__":
    runpy.run_module("openrlhf_b200.cli.train_sft", run_name="__main__")

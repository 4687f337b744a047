"""``python -m openrlhf.cli.train_rm`` -> ``openrlhf_b200.cli.train_rm``."""
import runpy

from openrlhf_b200.cli.train_rm import *  # noqa: F401,F403

if __name__ == "__main__":
    runpy.run_module("openrlhf_b200.cli.train_rm", run_name="__main__")

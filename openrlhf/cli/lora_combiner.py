"""``python -m openrlhf.cli.lora_combiner`` -> ``openrlhf_b200.cli.lora_combiner``."""
import runpy

from openrlhf_b200.cli.lora_combiner import *  # noqa: F401,F403

if __name__ == "__main__":
    runpy.run_module("openrlhf_b200.cli.lora_combiner", run_name="__main__")

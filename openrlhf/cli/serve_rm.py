"""``python -m openrlhf.cli.serve_rm`` -> ``openrlhf_b200.cli.serve_rm``."""
import runpy

from openrlhf_b200.cli.serve_rm import *  # noqa: F401,F403

if __name__ == "__main__":
    runpy.run_module("openrlhf_b200.cli.serve_rm", run_name="__main__")

"""Entry points: thin launchers that run the implementation modules of ``openrlhf_b200.cli``."""

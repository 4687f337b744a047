from .prompts_dataset import PromptDataset  # noqa: F401
from .reward_dataset import RewardDataset  # noqa: F401
from .sft_dataset import SFTDataset  # noqa: F401

from .actor import Actor  # noqa: F401
from .loss import (DPOLoss, GPTLMLoss, LogExpLoss, PairWiseLoss, PolicyLoss, SFTLoss, ValueLoss,  # noqa: F401
                   aggregate_loss)
from .model import get_llm_for_sequence_regression  # noqa: F401

from .config import hierarchize  # noqa: F401


_LAZY = {"get_strategy": ".strategy", "get_tokenizer": ".utils", "extract_boxed_answer": ".math_utils",
         "grade_answer": ".math_utils"}


def __getattr__(name):
    """`from openrlhf.utils import get_strategy, get_tokenizer, grade_answer, extract_boxed_answer` (the reference's
    public names), resolved on first use so that importing a light utility does not pull in torch.distributed."""
    if name in _LAZY:
        import importlib

        return getattr(importlib.import_module(_LAZY[name], __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")

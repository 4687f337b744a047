from .config import hierarchize  # noqa: F401

from .config import EvalConfig

__all__ = ["EvalConfig"]

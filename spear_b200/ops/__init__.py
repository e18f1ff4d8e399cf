from .btp import btp

__all__ = ["btp"]

from .swr import KVRepeat, Phalanx, SigmoidA

__all__ = ["Phalanx", "SigmoidA", "KVRepeat"]

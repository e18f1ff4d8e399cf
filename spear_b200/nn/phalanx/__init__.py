from .inference import JagState, parallel_jagged, step_jagged
from .swr import KVRepeat, Phalanx, SigmoidA

__all__ = ["Phalanx", "SigmoidA", "KVRepeat", "JagState", "parallel_jagged", "step_jagged"]

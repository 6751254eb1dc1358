from .matrix import Matrix
from .batch_matrix import BatchMatrix

__all__ = ["Matrix", "BatchMatrix"]

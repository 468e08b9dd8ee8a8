from .device import RowSampler
from .params import Sampling

__all__ = ["RowSampler", "Sampling"]

from .options import Options
from .sampler import DeviceSampler

__all__ = ["DeviceSampler", "Options"]

from .options import GenerationOptions, Sampling
from .host import SplitMix64, sample_host

__all__ = ["GenerationOptions", "Sampling", "SplitMix64", "sample_host"]

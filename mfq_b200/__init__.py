"""mfq_b200: mixed-format quantization and inference for Blackwell (sm_100a) GPUs."""

from ._version import __version__

__all__ = ["__version__"]

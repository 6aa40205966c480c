"""flashnystrom_b200: Nystrom attention (forward + exact backward) for NVIDIA B200 (sm_100a).

Drop-in for the reference project's Python API:

    from flashnystrom_b200 import flash_nystrom_attention, FlashNystromAttention, NystromConfig
"""
from .nystrom_config import NystromConfig
from .flash_nystrom import (FlashNystromAttention, FlashNystromFunction,
                            flash_nystrom_attention)

__version__ = "0.1.0"
__all__ = ["FlashNystromAttention", "FlashNystromFunction", "flash_nystrom_attention",
           "NystromConfig", "__version__"]

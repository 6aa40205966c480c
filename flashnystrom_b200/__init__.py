"""flashnystrom_b200: Nystrom attention (forward + exact backward) for NVIDIA B200 (sm_100a).

Drop-in for the reference project's Python API:

    from flashnystrom_b200 import flash_nystrom_attention, FlashNystromAttention, NystromConfig

Code written against the reference's package name keeps working after

    import flashnystrom_b200; flashnystrom_b200.install_as("flash_nystrom")

which makes `import flash_nystrom`, `from flash_nystrom import flash_nystrom_attention` and
`from flash_nystrom import _C` resolve to this package (flash_nystrom/__init__.py:30-60 exports the
same names).
"""
import sys

from .nystrom_config import NystromConfig
from .flash_nystrom import (HAS_CUDA, FlashNystromAttention, FlashNystromFunction,
                            flash_nystrom_attention)

__version__ = "0.2.0"
__all__ = ["FlashNystromAttention", "FlashNystromFunction", "flash_nystrom_attention",
           "NystromConfig", "HAS_CUDA", "install_as", "__version__"]


def install_as(name="flash_nystrom"):
    """Register this package (and its `_C`, `flash_nystrom` and `nystrom_config` modules) under
    another top-level name, so that imports written for the reference package find it."""
    from . import _C, flash_nystrom, nystrom_config
    pkg = sys.modules[__name__]
    sys.modules[name] = pkg
    sys.modules[name + "._C"] = _C
    sys.modules[name + ".flash_nystrom"] = flash_nystrom
    sys.modules[name + ".nystrom_config"] = nystrom_config
    return pkg

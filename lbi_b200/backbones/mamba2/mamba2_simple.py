"""The Mamba-2 mixer under the module name the reference uses (backbones/mamba2/mamba2_simple.py); the code is in ``mixer``."""
from .mixer import Mamba2Simple

__all__ = ["Mamba2Simple"]

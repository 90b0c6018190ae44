"""The Mamba-3 mixer under the module name the reference uses (backbones/mamba3/mamba3.py); the code is in ``mixer``."""
from .mixer import Mamba3, Mamba3ForwardCache

__all__ = ["Mamba3", "Mamba3ForwardCache"]

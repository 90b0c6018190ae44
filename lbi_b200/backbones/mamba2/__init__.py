from .block import Mamba2Block
from .mixer import Mamba2Simple
from .ssd import ssd_chunk_scan, ssd_recurrent_reference

__all__ = ["Mamba2Block", "Mamba2Simple", "ssd_chunk_scan", "ssd_recurrent_reference"]

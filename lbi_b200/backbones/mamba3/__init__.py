from .block import Mamba3Block
from .mixer import Mamba3, Mamba3ForwardCache
from .siso import angle_dt_cumsum, mamba3_siso_chunked, mamba3_siso_recurrent_reference

__all__ = [
    "Mamba3Block",
    "Mamba3",
    "Mamba3ForwardCache",
    "angle_dt_cumsum",
    "mamba3_siso_chunked",
    "mamba3_siso_recurrent_reference",
]

from .backward import NativeBackwardResult, _native_backward_step, native_backward_step
from .lbi1_checkpoint import is_lbi1_state_dict, migrate_lbi1_state_dict, migrate_lbi1_state_key
from .native_region_interface import (
    NativeRegionInterfaceModel,
    RegionForwardCache,
    RegionInterfaceCache,
    RegionMessageHead,
    build_region_slices,
)

__all__ = ["native_backward_step", "NativeBackwardResult", "_native_backward_step", "RegionForwardCache", "RegionInterfaceCache",
           "RegionMessageHead", "build_region_slices", "is_lbi1_state_dict", "migrate_lbi1_state_dict", "migrate_lbi1_state_key", "NativeRegionInterfaceModel"]

from .backward import native_backward_step
from .lbi1_checkpoint import is_lbi1_state_dict, migrate_lbi1_state_dict, migrate_lbi1_state_key
from .native_region_interface import NativeRegionInterfaceModel

__all__ = ["native_backward_step", "is_lbi1_state_dict", "migrate_lbi1_state_dict", "migrate_lbi1_state_key", "NativeRegionInterfaceModel"]

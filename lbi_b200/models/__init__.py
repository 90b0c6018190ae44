from .dense_language_model import DenseLanguageModel
from .lbi_language_model import LBICache, LBILanguageModel, LBIRegionCache
from .region_plan import RegionPlacement, RegionPlan, build_region_ranges, split_tokens

__all__ = [
    "DenseLanguageModel",
    "LBILanguageModel",
    "LBICache",
    "LBIRegionCache",
    "RegionPlan",
    "RegionPlacement",
    "build_region_ranges",
    "split_tokens",
]

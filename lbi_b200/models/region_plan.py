"""Region plans: how a model's computation is cut into regions that exchange only the interface state.

``axis="depth"``     region k = layers [l_k, l_{k+1}) over the full sequence; parameters are disjoint per
                     region; only the last region feeds the readout.  This is the reference's definition
                     (models/lbi_language_model.py:19-30, 170-204).
``axis="sequence"``  region k = tokens [t_k, t_{k+1}) through the whole stack; backbone parameters are shared
                     by all regions; every region feeds the readout and owns a share of the loss.  The
                     backward recursion then has an offset per region: g_k = b_k + A_k^T g_{k+1}.

``RegionPlacement`` maps regions to ranks in contiguous blocks, so K regions on G GPUs need only G - 1
cross-GPU handoffs.
"""
from __future__ import annotations

from dataclasses import dataclass


def build_region_ranges(layers: int, layers_per_region: int) -> list[tuple[int, int]]:
    if layers <= 0:
        raise ValueError("layers must be > 0")
    if layers_per_region <= 0:
        raise ValueError("layers_per_region must be > 0")
    return [(start, min(layers, start + layers_per_region)) for start in range(0, layers, layers_per_region)]


def split_tokens(seq_len: int, num_regions: int) -> list[tuple[int, int]]:
    """Cut ``seq_len`` tokens into ``num_regions`` contiguous spans whose sizes differ by at most one (longer spans first)."""
    if num_regions <= 0:
        raise ValueError("num_regions must be > 0")
    if seq_len < num_regions:
        raise ValueError("seq_len must be >= number of sequence regions")
    base, extra = divmod(seq_len, num_regions)
    out, start = [], 0
    for k in range(num_regions):
        end = start + base + (1 if k < extra else 0)
        out.append((start, end))
        start = end
    return out


@dataclass(frozen=True)
class RegionPlan:
    """How a model is cut into regions: the axis, the number of regions, the layer range of each; ``token_ranges(T)`` gives the spans."""

    axis: str
    num_regions: int
    layer_ranges: tuple[tuple[int, int], ...]

    @staticmethod
    def depth(layers: int, layers_per_region: int) -> "RegionPlan":
        ranges = tuple(build_region_ranges(layers, layers_per_region))
        return RegionPlan(axis="depth", num_regions=len(ranges), layer_ranges=ranges)

    @staticmethod
    def sequence(layers: int, num_regions: int) -> "RegionPlan":
        if num_regions <= 0:
            raise ValueError("num_regions must be > 0")
        return RegionPlan(axis="sequence", num_regions=num_regions, layer_ranges=tuple((0, layers) for _ in range(num_regions)))

    def token_ranges(self, seq_len: int) -> list[tuple[int, int]]:
        if self.axis == "depth":
            return [(0, seq_len)] * self.num_regions
        return split_tokens(seq_len, self.num_regions)

    def region_has_loss(self, k: int) -> bool:
        return self.axis == "sequence" or k == self.num_regions - 1

    @property
    def shares_backbone_parameters(self) -> bool:
        return self.axis == "sequence"


@dataclass(frozen=True)
class RegionPlacement:
    """Contiguous block assignment of regions to ranks."""

    num_regions: int
    world_size: int

    def __post_init__(self) -> None:
        if self.world_size <= 0 or self.num_regions <= 0:
            raise ValueError("num_regions and world_size must be > 0")
        if self.num_regions % self.world_size != 0:
            raise ValueError(f"num_regions ({self.num_regions}) must be divisible by world_size ({self.world_size})")

    @property
    def regions_per_rank(self) -> int:
        return self.num_regions // self.world_size

    def owner(self, region: int) -> int:
        return region // self.regions_per_rank

    def regions_of(self, rank: int) -> range:
        per = self.regions_per_rank
        return range(rank * per, (rank + 1) * per)

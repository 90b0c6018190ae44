"""Command-line entry of the first release, kept so that its launch lines keep working:

    python -m lbi_b200.legacy.train_region_interface --regime native_region_interface ...

Legacy regime names (``backprop_ref``, ``native_region_interface``) are mapped to the model variants (``dense``, ``lbi``) and
the run is handed to ``train.lbi.run_lbi_experiment``.  The reference's module of the same name
(legacy/train_region_interface.py:1-48) imports a ``config.lbi2`` bridge that its tree does not contain; here the mapping is
the one ``train.config`` already applies to ``--regime``.
"""
from __future__ import annotations

import json
from typing import Any

from ..train.config import LBITrainingConfig, RegionInterfaceConfig, build_arg_parser, config_from_args
from ..train.lbi import run_lbi_experiment


def _prepare_legacy_cfg(cfg: LBITrainingConfig) -> LBITrainingConfig:
    """A config written for the first release names its runs by ``regime`` only."""
    if not str(getattr(cfg, "variants", "") or "").strip():
        cfg.variants = cfg.regime
    return cfg


def run_training(cfg: LBITrainingConfig) -> dict[str, Any]:
    return run_lbi_experiment(_prepare_legacy_cfg(cfg))


def main() -> None:
    cfg = config_from_args(build_arg_parser().parse_args())
    print(json.dumps(run_training(cfg), indent=2, sort_keys=True))


__all__ = ["LBITrainingConfig", "RegionInterfaceConfig", "main", "run_training"]


if __name__ == "__main__":
    main()

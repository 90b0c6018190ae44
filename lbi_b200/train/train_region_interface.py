"""Historical entry-point name (``python -m lbi_b200.train.train_region_interface``); same program as ``train.lbi``.

The reference's module of this name imports a config module that no longer exists
(legacy/train_region_interface.py:6), so its paper launchers cannot start; this alias works.
"""
from .config import RegionInterfaceConfig, _build_arg_parser, _from_args, _validate_cfg  # noqa: F401
from .lbi import main, run_lbi_experiment, run_training  # noqa: F401

if __name__ == "__main__":
    main()

from .config import LBITrainingConfig, RegionInterfaceConfig, build_arg_parser, config_from_args, validate_config

__all__ = ["LBITrainingConfig", "RegionInterfaceConfig", "build_arg_parser", "config_from_args", "validate_config"]

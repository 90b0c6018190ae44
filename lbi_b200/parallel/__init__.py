from .comm import CollectiveComm, LocalComm, init_distributed_from_env
from .dense_engine import DenseFastEngine
from .engine import FastLBIEngine, StepResult
from .flat import FlatParams

__all__ = ["CollectiveComm", "LocalComm", "init_distributed_from_env", "DenseFastEngine", "FastLBIEngine", "StepResult", "FlatParams"]

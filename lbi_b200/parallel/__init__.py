from .comm import CollectiveComm, LocalComm, init_distributed_from_env
from .engine import FastLBIEngine, StepResult
from .flat import FlatParams

__all__ = ["CollectiveComm", "LocalComm", "init_distributed_from_env", "FastLBIEngine", "StepResult", "FlatParams"]

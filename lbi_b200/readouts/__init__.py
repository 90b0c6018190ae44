from .base import ReadoutCache, ReadoutModule
from .lm_head import NormLMHeadReadout

__all__ = ["ReadoutCache", "ReadoutModule", "NormLMHeadReadout"]

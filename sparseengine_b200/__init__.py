"""sparseengine_b200: a small, whole inference engine for one GPU (B200, sm_100a).

    from sparseengine_b200 import LLM, SamplingParams
"""
__version__ = "0.1.0"

from .config.engine_config import Config
from .sampling.params import SamplingParams


def __getattr__(name):
    if name == "LLM":
        from .engine.llm import LLM
        return LLM
    raise AttributeError(name)


__all__ = ["LLM", "SamplingParams", "Config"]

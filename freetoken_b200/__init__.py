"""freetoken_b200: a small, whole inference engine for one B200 (sm_100a).

Public entry points:

* :class:`freetoken_b200.engine.llm.LLM` and :class:`SamplingParams` for generation,
* :class:`freetoken_b200.engine.engine.Engine` for the step function,
* ``python -m freetoken_b200`` (command line) and ``bin/trace_run`` (trace replay).
"""

from .version import __version__

__all__ = ["__version__", "LLM", "SamplingParams", "Engine", "EngineConfig"]


def __getattr__(name):  # lazy: importing the package must not import torch-heavy modules
    if name == "LLM":
        from .engine.llm import LLM

        return LLM
    if name == "SamplingParams":
        from .sampling.params import SamplingParams

        return SamplingParams
    if name == "Engine":
        from .engine.engine import Engine

        return Engine
    if name == "EngineConfig":
        from .config.engine_config import EngineConfig

        return EngineConfig
    raise AttributeError(name)

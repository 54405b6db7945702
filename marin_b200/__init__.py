"""marin_b200: a small, whole inference engine for the Qwen3 dense decoder on one B200.

    from marin_b200 import Engine, SamplingParams
    engine = Engine("path/to/model", dtype="bfloat16", ctx=4096)
    out = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0, max_tokens=16))
"""
from .config import ConfigError, ModelConfig, Qwen3Config, load_config
from .engine import Engine, Generation, Runner, Scheduler, StepEntry, StopReason
from .sampling import Sampler, SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["ConfigError", "ModelConfig", "Qwen3Config", "load_config", "Engine", "Generation", "Runner",
           "Scheduler", "StepEntry", "StopReason", "Sampler", "SamplingParams", "WeightError", "write_random_model"]
__version__ = "0.1.0"

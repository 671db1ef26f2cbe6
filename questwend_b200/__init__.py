"""questwend_b200: a small generation library for one B200, built from what
kishida/questwend computes for its Qwen3 dense architecture.

    from questwend_b200 import Engine, SamplingParams, generate
    engine = Engine.from_folder("model_dir", dtype="bfloat16", max_tokens=8192)
    out = generate(engine, [[1, 2, 3]], max_new_tokens=16, sampling=SamplingParams(temperature=0))
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, load_config, register_architecture
from .engine import Engine, EngineError, StepEntry, generate, GenerationResult, GenerationStats, StepProfile
from .sampling import SamplingParams, GREEDY
from .weights import WeightsError, write_model_folder

__all__ = ["Engine", "EngineError", "StepEntry", "generate", "GenerationResult", "GenerationStats", "StepProfile",
           "SamplingParams", "GREEDY", "ConfigError", "load_config", "register_architecture", "WeightsError",
           "write_model_folder"]

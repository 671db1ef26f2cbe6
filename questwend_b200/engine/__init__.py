from .plan import LayerSpec, ModelPlan, Run
from .model import Model
from .engine import Engine, EngineError, StepEntry
from .generate import generate, plan_batches, GenerationResult, GenerationStats, StepProfile

__all__ = ["LayerSpec", "ModelPlan", "Run", "Model", "Engine", "EngineError", "StepEntry", "generate",
           "plan_batches", "GenerationResult", "GenerationStats", "StepProfile"]

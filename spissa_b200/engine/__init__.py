"""Model assembly, the step function and the generation loop."""
from .batch import StepBatch, pack_step
from .model import Model
from .engine import Engine, StepEntry, StepError
from .generate import GenerationMetrics, GenerationResult, generate, plan_batches

__all__ = ["StepBatch", "pack_step", "Model", "Engine", "StepEntry", "StepError", "GenerationMetrics",
           "GenerationResult", "generate", "plan_batches"]

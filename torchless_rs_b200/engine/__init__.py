from .batch import BatchStager, StepBatch, layout_step
from .engine import Engine
from .model import DecoderModel, expected_tensors
from .generate import GenerationResult, generate, plan_batches

__all__ = ["BatchStager", "StepBatch", "layout_step", "Engine", "DecoderModel",
           "expected_tensors", "GenerationResult", "generate", "plan_batches"]

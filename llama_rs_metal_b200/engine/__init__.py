from .batch import StepContext, StepEntry
from .generate import GenerationResult, generate, plan_batches
from .model import DecoderModel
from .step import StepRunner, classify_step, validate_entries

__all__ = ["StepContext", "StepEntry", "GenerationResult", "generate", "plan_batches",
           "DecoderModel", "StepRunner", "classify_step", "validate_entries"]

from .generate import GenerationResult, generate, plan_batches, run_batch, token_budget
from .model import DecoderModel, StepEntry, parse_dtype

__all__ = ["DecoderModel", "StepEntry", "parse_dtype", "GenerationResult", "generate", "plan_batches", "run_batch",
           "token_budget"]

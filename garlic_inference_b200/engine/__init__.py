from .api import AutoConfig, AutoModel, LanguageModel, engine_dtype
from .generate import (GenerationError, GenerationLoop, GenParams, GenStats, finished, plan_batches,
                       tokens_held)
from .model import DecoderModel, wanted_tensors
from .step import Engine, StepEntry, StepError

__all__ = ["AutoConfig", "AutoModel", "LanguageModel", "engine_dtype", "GenerationError", "GenerationLoop",
           "GenParams", "GenStats", "finished", "plan_batches", "tokens_held", "DecoderModel",
           "wanted_tensors", "Engine", "StepEntry", "StepError"]

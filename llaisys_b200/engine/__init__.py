from .context import StepContext
from .engine import Engine, StepEntry, StepError, build_engine
from .generate import Generation, GenerationLoop
from .model import DecoderModel

__all__ = ["DecoderModel", "Engine", "Generation", "GenerationLoop", "StepContext", "StepEntry", "StepError", "build_engine"]

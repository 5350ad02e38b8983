from .engine import Engine, EngineOptions, parse_dtype  # noqa: F401
from .generate import Generation, GenerationError, generate  # noqa: F401
from .model import DecoderModel  # noqa: F401
from .step import StepContext, StepError, Stepper  # noqa: F401

"""A small model library with generation of its own for NVIDIA B200 (sm_100a): the
Qwen2.5 dense decoder, from a model folder's tokens to the next token.

    from friday_inference_engine_b200 import Engine
    eng = Engine(model_path="/models/qwen2.5-7b", dtype="bfloat16", max_ctx=8192, max_batch=8)
    out = eng.generate([[1, 2, 3], [4, 5]], max_new_tokens=32, temperature=0.8, seed=7, stop_token_ids=[151645])
"""
from . import architectures  # noqa: F401
from .config import ConfigError, Qwen2Config  # noqa: F401
from .engine import Engine, EngineOptions, Generation  # noqa: F401
from .parts import register_part  # noqa: F401
from .registry import register_architecture  # noqa: F401

__version__ = "0.1.0"

"""A small model library with generation of its own for NVIDIA B200 (sm_100a): the
Qwen2.5 dense decoder, from a model folder's tokens to the next token.

The library is C++ and CUDA (libfriday_engine.so with include/friday/engine.h, and one
kernel library per file of csrc/); this package builds it on first use and binds it.

    from friday_inference_engine_b200 import Engine
    eng = Engine(model_path="/models/qwen2.5-7b", dtype="bfloat16", max_ctx=8192, max_batch=8)
    out = eng.generate([[1, 2, 3], [4, 5]], max_new_tokens=32, temperature=0.8, seed=7, stop_token_ids=[151645])
"""
from .native import (BuildError, CacheError, CacheFull, ConfigError, FridayError, GenerationError,  # noqa: F401
                     KernelError, StepError, WeightsError)
from .config import describe_model, read_config, registered_architectures  # noqa: F401
from .engine import Decoder, Engine, EngineOptions, Generation  # noqa: F401
from .parts import build_plugin, load_plugin, registered_parts  # noqa: F401
from .weights import check_weights, write_model_dir  # noqa: F401

__version__ = "0.2.0"

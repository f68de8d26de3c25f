"""A small single-GPU generation library for the Llama-family decoder, written for B200 (sm_100a).

Entry points::

    from exl3_server_b200 import Engine, generate, GenerateOptions
    engine = Engine.from_folder(model_dir, dtype="bfloat16", max_tokens=8192)
    results = generate(engine, prompts=[[1, 2, 3]], options=GenerateOptions(max_tokens=16))
"""
from . import models  # noqa: F401  (registers the architectures)
from .config import ConfigError, LlamaConfig, register_architecture, resolve_architecture
from .engine import (Engine, GenerateOptions, GenerateResult, Model, StepEntry, StepError, generate,
                     load_model)
from .sampling import SampleOptions
from .weights import WeightsError
from .weights.random_init import write_random_model

__all__ = ["ConfigError", "LlamaConfig", "register_architecture", "resolve_architecture", "Engine", "Model", "GenerateOptions", "GenerateResult", "SampleOptions", "generate",
           "StepEntry", "StepError", "load_model", "WeightsError", "write_random_model"]

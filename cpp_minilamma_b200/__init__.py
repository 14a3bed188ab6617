"""cpp_minilamma_b200: a small, whole Llama inference library for one NVIDIA B200.

From a model folder (config.json + safetensors) or seeded random weights to generated
token ids: typed configuration and architecture registry, weights by tensor name, models
put together from parts, a paged sequence cache, one step function, a generation loop,
device sampling, and hand-written CUDA kernels for sm_100a (no CPU path).
"""
from . import models  # noqa: F401  (registers architectures)
from .api import LLM, EngineBackend, build_model, load, parse_dtype, random_model
from .config import ConfigError, LlamaConfig, config_from_dict, load_config, register_architecture
from .engine import Completion, Engine, Model, StepEntry, StepError
from .parts import register_part
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__all__ = ["LLM", "load", "random_model", "build_model", "LlamaConfig", "load_config", "config_from_dict",
           "register_architecture", "register_part", "Engine", "Model", "StepEntry", "SamplingParams",
           "WeightError", "ConfigError", "write_random_model", "Completion", "StepError", "EngineBackend",
           "parse_dtype"]

"""A B200-native inference engine for the Qwen2 dense decoder, shaped after the CPU engine hf.cpu.

Sub-packages: ``config`` (typed configuration, registry), ``weights`` (safetensors by name, random
weights), ``parts`` (norm, position encoding, mixer, feed-forward, block), ``models`` (a model put
together from a plan), ``cache`` (paged keys/values, state slots), ``engine`` (step function,
scheduler), ``sampling``, ``kernels`` (binding of the CUDA library built from ``csrc``), ``cli``.
"""
from . import config, weights, parts, models, cache, engine, sampling  # noqa: F401
from .config import load_config, register_architecture
from .engine import Engine, StepEntry
from .models import Model, load_model, random_model
from .parts import register_part
from .weights import write_random_model
from .api import Completion, Session, generate
from .sampling import SamplingParams

__version__ = "0.1.0"
__all__ = ["load_config", "register_architecture", "register_part", "Engine", "StepEntry", "Model",
           "load_model", "random_model", "write_random_model", "Session", "generate", "Completion",
           "SamplingParams"]

"""axon_b200: a small, whole LLM inference engine for one NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) to generated tokens: a typed
configuration and an architecture registry, weights by tensor name, layers put
together from parts, a paged cache manager, one step function for mixed batches, a
continuous-batching scheduler, sampling, and hand-written CUDA kernels.  The public
names follow the library API of the engine it is modelled on (``load``, ``Backend``,
``BackendOptions``, ``generate``, ``GenOpts``, ``GenStats``).
"""

__version__ = "0.1.0"

from .api import (Backend, BackendCache, BackendOptions, GenOpts, GenStats, Model, argmax, generate, load)
from .config import ConfigError, Qwen2Config, load_config, register_architecture
from .engine.step import Engine, OutOfPages, StepEntry, StepError
from .parts import register_part
from .sampling.sampler import SampleArgs, SampleCfg
from .weights import WeightsError, write_random_model

__all__ = [
    "Backend", "BackendCache", "BackendOptions", "ConfigError", "Engine", "GenOpts", "GenStats", "Model",
    "OutOfPages", "Qwen2Config", "SampleArgs", "SampleCfg", "StepEntry", "StepError", "WeightsError",
    "argmax", "generate", "load", "load_config", "register_architecture", "register_part",
    "write_random_model",
]

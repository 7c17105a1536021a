"""metallix_b200: a small, whole inference engine for one B200.

From a model folder (``config.json`` + safetensors) to the next token on one
GPU, for the Qwen3 dense decoder: typed configuration and architecture
registry, by-name weight loading, layers put together from parts, a paged
cache manager, one step function for mixed batches, a continuous-batching
scheduler, sampling, and hand-written sm_100a kernels with a true float32 path.
"""
from . import parts  # noqa: F401  (registers the built-in parts)
from .config import ConfigError, Qwen3Config, parse_config, read_config
from .weights import CheckpointError, load_tensors, random_tensors, write_model_folder

__version__ = "0.1.0"

__all__ = ["ConfigError", "Qwen3Config", "parse_config", "read_config", "CheckpointError",
           "load_tensors", "random_tensors", "write_model_folder", "Engine", "StepEntry",
           "generate"]


def __getattr__(name):
    # The engine pulls in the CUDA build; config and weights stay importable
    # on a machine without a GPU.
    if name in ("Engine", "StepEntry", "StepError"):
        from . import engine
        return getattr(engine, name)
    if name in ("generate", "GenerationResult", "Generator"):
        from .engine import generate as _generate
        return getattr(_generate, name)
    raise AttributeError(name)

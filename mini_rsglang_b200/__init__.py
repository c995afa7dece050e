"""mini_rsglang_b200: a small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) or seeded random weights to generated tokens:
typed configuration and an architecture registry, weights bound by name, layers put together
from parts, a paged cache manager, one step function for mixed batches, a continuous-batching
scheduler, samplers, a command line, and hand-written CUDA kernels."""
from .config import ModelConfig, Qwen3Config, RuntimeConfig
from .errors import BackendError, CapacityError, EngineError, EngineStopped, InvalidRequest
from .sampling.params import SamplingParams


def __getattr__(name):
    """The engine classes import torch-side modules; they are loaded at first use."""
    if name in ("EngineHandle", "GenerateRequest", "TokenIds", "Token", "Finished", "Error", "GenerationResult",
                "ModelRunner", "SequenceStep", "Scheduler"):
        from . import engine

        return getattr(engine, name)
    raise AttributeError(name)


__version__ = "0.1.0"

__all__ = ["ModelConfig", "Qwen3Config", "RuntimeConfig", "BackendError", "CapacityError", "EngineError",
           "EngineStopped", "InvalidRequest", "SamplingParams", "EngineHandle", "GenerateRequest", "TokenIds",
           "__version__"]

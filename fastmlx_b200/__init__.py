"""fastmlx_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

Everything between a request's tokens and its next token: typed configuration and a
registry of architectures, weights by tensor name, layers assembled from parts, a paged
cache with block tables, one step function over ragged batches, a continuous-batching
scheduler, sampling, a command line and this Python entry point.  It follows the shape of
tamnd/fastmlx's compute engine (compute/, enginecore/, scheduler/) and is written for
Blackwell from scratch.
"""
from . import models as _models  # noqa: F401  (registers the architectures)
from .config import ConfigError, LlamaConfig
from .registry import build_model, register, registered_model_types
from .weights import WeightError, load_checkpoint, write_random_model

__version__ = "0.1.0"


def __getattr__(name):
    # The engine classes pull in torch.cuda state; import them on first use.
    if name in ("Engine", "SamplingParams", "RequestOutput", "EngineConfig"):
        from .engine import api
        return getattr(api, name)
    raise AttributeError(name)


__all__ = ["ConfigError", "LlamaConfig", "WeightError", "build_model", "register", "registered_model_types",
           "load_checkpoint", "write_random_model", "Engine", "SamplingParams", "RequestOutput", "EngineConfig"]

"""From a model folder to a model on the device, as every entry point does it."""
from __future__ import annotations

import torch

from .. import registry
from ..parts.base import Runtime
from ..weights import load_checkpoint
from ..weights.random_init import random_tensors

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {name}")
        return name
    try:
        return DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"unknown dtype {name!r} (bfloat16 or float32)") from None


def make_runtime(dtype, device="cuda", kernels=None) -> Runtime:
    """The product runtime computes on CUDA with the package's kernels.  `kernels` lets a
    test put plain stand-ins in their place; nothing in the package does."""
    dev = torch.device(device)
    if kernels is None:
        if dev.type != "cuda":
            raise RuntimeError("fastmlx_b200 computes on a CUDA device only; there is no CPU path")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible; fastmlx_b200 has no CPU path")
        from .. import kernels as k
        kernels = k
    return Runtime(dev, parse_dtype(dtype), kernels)


def load_model(model_dir: str, dtype="bfloat16", device="cuda", kernels=None):
    """-> (typed config, model with bound weights, runtime)."""
    config, tensors = load_checkpoint(model_dir)
    cfg, model = registry.build_model(config)
    rt = make_runtime(dtype, device, kernels)
    model.load_weights(tensors, rt)
    return cfg, model, rt


def random_model(config: dict, seed: int, dtype="bfloat16", device="cuda", kernels=None, store_dtype=torch.bfloat16):
    """A model with seeded random weights made straight on the device (no folder)."""
    cfg, model = registry.build_model(config)
    rt = make_runtime(dtype, device, kernels)
    gen_device = rt.device if rt.device.type == "cuda" else "cpu"
    tensors = random_tensors(model, seed, store_dtype, gen_device)
    model.load_weights(tensors, rt)
    return cfg, model, rt

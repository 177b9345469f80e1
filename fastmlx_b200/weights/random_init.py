"""Random weights from a configuration and a seed, written as a model folder.

tamnd/fastmlx has no such mode; its tests fabricate one-element tensors
(compute/models/llama_forward_test.go:28-39).  Each tensor's values come from a
generator keyed by (seed, tensor name), so they do not depend on the order in which
tensors are made or on sharding: matrices, embeddings and biases N(0, 0.02), norm
weights 1 + N(0, 0.02), drawn in 32-bit and then cast to the stored dtype.
"""
from __future__ import annotations

import hashlib
import json
import os

import torch

from .. import registry
from . import safetensors_io as st

INIT_STD = 0.02


def _seed_for(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & (2**63 - 1)


def random_tensor(seed: int, name: str, shape, kind: str, dtype=torch.bfloat16, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, name))
    t = torch.randn(tuple(shape), generator=g, dtype=torch.float32, device=device) * INIT_STD
    if kind == "norm":
        t += 1.0
    return t.to(dtype)


def random_tensors(model, seed: int, dtype=torch.bfloat16, device="cpu") -> dict[str, torch.Tensor]:
    """Every tensor the model's parts declare (name, shape, kind)."""
    return {spec.name: random_tensor(seed, spec.name, spec.shape, spec.kind, dtype, device)
            for spec in model.weight_specs()}


def write_random_model(model_dir: str, config: dict, seed: int, dtype=torch.bfloat16,
                       max_shard_bytes: int | None = None) -> str:
    """Write config.json and model.safetensors (or shards plus an index when
    `max_shard_bytes` is given) for the architecture that `config` names."""
    os.makedirs(model_dir, exist_ok=True)
    cfg, model = registry.build_model(config)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config, f, indent=2)
    tensors = random_tensors(model, seed, dtype)
    if max_shard_bytes is None:
        st.write_file(os.path.join(model_dir, "model.safetensors"), tensors,
                      {"format": "pt", "seed": seed})
        return model_dir
    shards: list[dict] = [{}]
    used = 0
    for name in sorted(tensors):
        nbytes = tensors[name].numel() * tensors[name].element_size()
        if shards[-1] and used + nbytes > max_shard_bytes:
            shards.append({})
            used = 0
        shards[-1][name] = tensors[name]
        used += nbytes
    weight_map, total = {}, 0
    for i, sh in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        st.write_file(os.path.join(model_dir, fname), sh, {"format": "pt", "seed": seed})
        for name, t in sh.items():
            weight_map[name] = fname
            total += t.numel() * t.element_size()
    st.write_index(os.path.join(model_dir, st.INDEX_NAME), weight_map, total)
    return model_dir

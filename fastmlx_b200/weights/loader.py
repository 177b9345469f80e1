"""A model folder -> (config dict, tensors by name), as stored.

Folder layout and shard choice follow tamnd/fastmlx compute/checkpoint.go:31-89: read
config.json; when model.safetensors.index.json exists load exactly the shard files it
names (other files are ignored), else every *.safetensors in sorted order; a name found
in two shards is an error (compute/loader.go:90-105).  Dtype policy: bfloat16 and 32-bit
tensors stay as stored, float16 becomes bfloat16, 64-bit integers become int32 after a
range check; FP8 tags are refused (compute/loader.go:14-47,71-74).
"""
from __future__ import annotations

import glob
import os

import torch

from ..config.base import read_config_json
from . import safetensors_io as st


class WeightError(ValueError):
    """Raised once, with every missing, unexpected and mis-shaped tensor listed."""


def shard_files(model_dir: str) -> list[str]:
    idx = os.path.join(model_dir, st.INDEX_NAME)
    if os.path.exists(idx):
        with open(idx, "rb") as f:
            _, shards, _ = st.parse_index(f.read())
        missing = [s for s in shards if not os.path.exists(os.path.join(model_dir, s))]
        if missing:
            raise WeightError(f"checkpoint: index names shard files that do not exist: {missing}")
        return [os.path.join(model_dir, s) for s in shards]
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise WeightError(f"checkpoint: no .safetensors file in {model_dir}")
    return files


def _as_held(name: str, t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype in (torch.int64, torch.int16, torch.int8, torch.uint8):
        if t.numel() and (int(t.max()) > 2**31 - 1 or int(t.min()) < -2**31):
            raise WeightError(f"checkpoint: integer tensor {name!r} does not fit int32")
        return t.to(torch.int32)
    raise WeightError(f"checkpoint: tensor {name!r} has unsupported dtype {t.dtype}")


def load_tensors(model_dir: str) -> dict[str, torch.Tensor]:
    merged: dict[str, torch.Tensor] = {}
    origin: dict[str, str] = {}
    for path in shard_files(model_dir):
        for name, t in st.read_file(path).items():
            if name in merged:
                raise WeightError(f"checkpoint: tensor {name!r} is present in more than one shard "
                                  f"({os.path.basename(origin[name])}, {os.path.basename(path)})")
            merged[name] = _as_held(name, t)
            origin[name] = path
    return merged


def load_checkpoint(model_dir: str) -> tuple[dict, dict[str, torch.Tensor]]:
    return read_config_json(model_dir), load_tensors(model_dir)

"""Reading and writing the safetensors container and its shard index.

Container: an 8-byte little-endian header length, a JSON header
{name: {dtype, shape, data_offsets}}, then the tensor bytes.  The checks are those of
tamnd/fastmlx compute/safetensors.go:106-169 (buffer long enough, header inside the
file, known dtype tag, begin <= end <= data length, numel * size == end - begin;
`__metadata__` kept apart) and of compute/safetensors_index.go:31-56 for the index
(`weight_map` must be a non-empty object; the shard list is its sorted unique values).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass

import torch

# tag -> (bytes per element, torch dtype or None when the engine cannot hold it)
DTYPES: dict[str, tuple[int, torch.dtype | None]] = {
    "BOOL": (1, torch.bool), "U8": (1, torch.uint8), "I8": (1, torch.int8),
    "F8_E5M2": (1, None), "F8_E4M3": (1, None),
    "I16": (2, torch.int16), "U16": (2, torch.uint16), "F16": (2, torch.float16),
    "BF16": (2, torch.bfloat16), "I32": (4, torch.int32), "U32": (4, torch.uint32),
    "F32": (4, torch.float32), "F64": (8, torch.float64), "I64": (8, torch.int64),
    "U64": (8, torch.uint64),
}
_TAG_OF = {torch.bfloat16: "BF16", torch.float32: "F32", torch.float16: "F16",
           torch.int32: "I32", torch.int64: "I64", torch.float64: "F64",
           torch.uint8: "U8", torch.int8: "I8", torch.bool: "BOOL", torch.int16: "I16"}

MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    pass


@dataclass(frozen=True)
class TensorInfo:
    name: str
    dtype: str
    shape: tuple[int, ...]
    begin: int
    end: int


def parse_header(buf) -> tuple[list[TensorInfo], dict, int]:
    """-> (tensors ordered by (begin, name), metadata, offset of the data section)."""
    total = len(buf)
    if total < 8:
        raise SafetensorsError("safetensors: buffer shorter than the 8-byte length prefix")
    (hlen,) = struct.unpack("<Q", bytes(buf[:8]))
    if hlen > MAX_HEADER:
        raise SafetensorsError(f"safetensors: header of {hlen} bytes is too large")
    if 8 + hlen > total:
        raise SafetensorsError(f"safetensors: header of {hlen} bytes does not fit a buffer of {total}")
    try:
        header = json.loads(bytes(buf[8:8 + hlen]))
    except (json.JSONDecodeError, UnicodeDecodeError) as e:
        raise SafetensorsError(f"safetensors: header is not JSON: {e}") from None
    if not isinstance(header, dict):
        raise SafetensorsError("safetensors: header must be a JSON object")
    data_len = total - 8 - hlen
    meta = header.pop("__metadata__", None) or {}
    infos = []
    for name, ent in header.items():
        try:
            tag, shape, (begin, end) = ent["dtype"], tuple(int(s) for s in ent["shape"]), ent["data_offsets"]
        except (KeyError, TypeError, ValueError):
            raise SafetensorsError(f"safetensors: malformed entry for {name!r}") from None
        if tag not in DTYPES:
            raise SafetensorsError(f"safetensors: {name!r} has unknown dtype {tag!r}")
        if not (0 <= begin <= end <= data_len):
            raise SafetensorsError(
                f"safetensors: {name!r} data_offsets [{begin}, {end}) lie outside the {data_len} data bytes")
        numel = 1
        for s in shape:
            if s < 0:
                raise SafetensorsError(f"safetensors: {name!r} has a negative dimension")
            numel *= s
        if numel * DTYPES[tag][0] != end - begin:
            raise SafetensorsError(
                f"safetensors: {name!r} {tag}{list(shape)} needs {numel * DTYPES[tag][0]} bytes, has {end - begin}")
        infos.append(TensorInfo(name, tag, shape, int(begin), int(end)))
    infos.sort(key=lambda t: (t.begin, t.name))
    return infos, meta, 8 + hlen


def read_file(path: str) -> dict[str, torch.Tensor]:
    """All tensors of one file, as stored (views of a private memory map)."""
    size = os.path.getsize(path)
    if size < 8:
        raise SafetensorsError(f"safetensors: {path}: shorter than the 8-byte length prefix")
    with open(path, "rb") as f:
        mm = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_COPY)
    try:
        infos, _, base = parse_header(mm)
    except SafetensorsError as e:
        raise SafetensorsError(f"{e} ({path})") from None
    out = {}
    for t in infos:
        width, dt = DTYPES[t.dtype]
        if dt is None:
            raise SafetensorsError(f"safetensors: {t.name!r}: unsupported dtype {t.dtype} ({path})")
        n = (t.end - t.begin) // width
        if n == 0:
            out[t.name] = torch.empty(t.shape, dtype=dt)
        else:
            out[t.name] = torch.frombuffer(mm, dtype=dt, count=n, offset=base + t.begin).view(t.shape)
    return out


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TAG_OF:
            raise SafetensorsError(f"safetensors: cannot store dtype {t.dtype} ({name!r})")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().contiguous().cpu()
            if t.numel():
                f.write(memoryview(t.view(torch.uint8).reshape(-1).numpy()))       # no second copy of the bytes
    os.replace(tmp, path)


INDEX_NAME = "model.safetensors.index.json"


def parse_index(body: bytes | str) -> tuple[dict[str, str], list[str], dict]:
    """-> (weight_map, sorted unique shard names, raw metadata)."""
    try:
        d = json.loads(body)
    except json.JSONDecodeError as e:
        raise SafetensorsError(f"safetensors index: not JSON: {e}") from None
    wm = d.get("weight_map") if isinstance(d, dict) else None
    if not isinstance(wm, dict) or not wm:
        raise SafetensorsError("safetensors index: weight_map is missing or empty")
    for k, v in wm.items():
        if not isinstance(v, str) or not v:
            raise SafetensorsError(f"safetensors index: weight_map[{k!r}] names no file")
    return dict(wm), sorted(set(wm.values())), d.get("metadata") or {}


def write_index(path: str, weight_map: dict[str, str], total_size: int) -> None:
    with open(path, "w") as f:
        json.dump({"metadata": {"total_size": total_size}, "weight_map": dict(sorted(weight_map.items()))}, f, indent=1)

"""safetensors files read and written by hand: an 8-byte little-endian header length, a JSON header
(name -> dtype, shape, data_offsets), then the raw little-endian data.

Only headers are parsed to list a folder's tensors; data is read per tensor at its offset. The
checks are the reference's (engine/models/lfm2_moe/pack.py:50-56 header, :163-200 index, shards,
duplicates, byte counts, truncation), each error naming the file or tensor.
"""

from __future__ import annotations

import json
import os
import struct
from dataclasses import dataclass

import numpy as np
import torch

_NP = {"F64": np.float64, "F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I64": np.int64,
       "I32": np.int32, "I16": np.int16, "I8": np.int8, "U8": np.uint8, "BOOL": np.bool_}
_SIZE = {"F64": 8, "F32": 4, "F16": 2, "BF16": 2, "I64": 8, "I32": 4, "I16": 2, "I8": 1, "U8": 1, "BOOL": 1}
_TAG = {torch.float64: "F64", torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16",
        torch.int64: "I64", torch.int32: "I32", torch.int16: "I16", torch.int8: "I8", torch.uint8: "U8",
        torch.bool: "BOOL"}


class CheckpointError(ValueError):
    """A model folder that cannot be read as written."""


@dataclass(frozen=True)
class StoredTensor:
    key: str            # the name as stored
    file: str
    dtype: str          # safetensors tag
    shape: tuple[int, ...]
    offset: int         # absolute byte offset in the file
    nbytes: int


def read_header(path: str) -> tuple[int, dict]:
    """(offset of the data section, header without __metadata__) of one file."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise CheckpointError(f"{path}: shorter than a safetensors header")
        n = struct.unpack("<Q", head)[0]
        if 8 + n > size:
            raise CheckpointError(f"{path}: header length {n} exceeds the file (truncated or not safetensors)")
        try:
            header = json.loads(f.read(n))
        except ValueError as e:
            raise CheckpointError(f"{path}: header is not JSON ({e})") from None
    header.pop("__metadata__", None)
    return 8 + n, header


def index_file(path: str) -> dict[str, StoredTensor]:
    start, header = read_header(path)
    size = os.path.getsize(path)
    out: dict[str, StoredTensor] = {}
    extent = 0
    for key, meta in header.items():
        dtype, shape = meta["dtype"], tuple(int(x) for x in meta["shape"])
        if dtype not in _SIZE:
            raise CheckpointError(f"{path}: tensor {key} has the unsupported dtype {dtype}")
        b0, b1 = meta["data_offsets"]
        want = int(np.prod(shape, dtype=np.int64)) * _SIZE[dtype] if shape else _SIZE[dtype]
        if b1 - b0 != want:
            raise CheckpointError(f"{path}: tensor {key} holds {b1 - b0} bytes, its shape {shape} {dtype} needs {want}")
        extent = max(extent, b1)
        out[key] = StoredTensor(key, path, dtype, shape, start + b0, b1 - b0)
    if start + extent > size:
        raise CheckpointError(f"{path}: {size} bytes on disk, the header describes {start + extent} (truncated or corrupt)")
    return out


def index_folder(folder: str) -> dict[str, StoredTensor]:
    """Every stored tensor of a model folder: `model.safetensors`, or the shards that
    `model.safetensors.index.json` names."""
    index_path = os.path.join(folder, "model.safetensors.index.json")
    single = os.path.join(folder, "model.safetensors")
    if os.path.isfile(index_path):
        with open(index_path) as f:
            weight_map = json.load(f).get("weight_map", {})
        shards = sorted(set(weight_map.values()))
        out: dict[str, StoredTensor] = {}
        for shard in shards:
            path = os.path.join(folder, shard)
            if not os.path.isfile(path):
                raise CheckpointError(f"{index_path} names the shard {shard}, which is not in the folder")
            for key, st in index_file(path).items():
                if key in out:
                    raise CheckpointError(f"tensor {key} is stored twice: {out[key].file} and {path}")
                out[key] = st
        lost = sorted(k for k in weight_map if k not in out)
        if lost:
            raise CheckpointError(f"{index_path} lists tensors no shard holds: {', '.join(lost[:8])}"
                                  + (f" and {len(lost) - 8} more" if len(lost) > 8 else ""))
        return out
    if os.path.isfile(single):
        return index_file(single)
    raise CheckpointError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def read_tensor(st: StoredTensor) -> torch.Tensor:
    """The tensor as stored (a CPU tensor that owns its memory)."""
    count = st.nbytes // _SIZE[st.dtype]
    arr = np.fromfile(st.file, dtype=_NP[st.dtype], count=count, offset=st.offset)
    if arr.size != count:
        raise CheckpointError(f"{st.file}: tensor {st.key} could not be read whole (truncated)")
    t = torch.from_numpy(arr)
    if st.dtype == "BF16":
        t = t.view(torch.bfloat16)
    return t.reshape(st.shape)


def write_file(path: str, tensors: dict[str, torch.Tensor], metadata: dict[str, str] | None = None) -> None:
    """Write `tensors` (CPU) as one safetensors file, names in sorted order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    blobs = []
    at = 0
    for name in sorted(tensors):
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _TAG:
            raise CheckpointError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        raw = (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t).numpy().tobytes()
        header[name] = {"dtype": _TAG[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)

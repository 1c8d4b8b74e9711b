"""Reading and writing the safetensors container, by tensor name.

The file is an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets"}}`` and one data block.  Tensors are
memory-mapped and only turned into torch tensors when asked for, so a loader can
check names and shapes of a large checkpoint before it touches the data.  The
reference goes through the ``safetensors`` package (engine/llama_weights.py:87-96);
this reader needs nothing but numpy and torch.
"""

from __future__ import annotations

import json
import mmap
import struct
import warnings
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch

# safetensors dtype tag -> (numpy dtype used to view the bytes, torch dtype of the result)
_DTYPES = {
    "F64": (np.dtype("<f8"), torch.float64),
    "F32": (np.dtype("<f4"), torch.float32),
    "F16": (np.dtype("<f2"), torch.float16),
    "BF16": (np.dtype("<u2"), torch.bfloat16),
    "I64": (np.dtype("<i8"), torch.int64),
    "I32": (np.dtype("<i4"), torch.int32),
    "I16": (np.dtype("<i2"), torch.int16),
    "I8": (np.dtype("i1"), torch.int8),
    "U8": (np.dtype("u1"), torch.uint8),
    "BOOL": (np.dtype("u1"), torch.bool),
}
_TAG_OF = {v[1]: k for k, v in _DTYPES.items()}


class CheckpointFormatError(ValueError):
    """A file that is not a well-formed safetensors container."""


@dataclass
class StoredTensor:
    """One tensor of a checkpoint: where it is and how to read it."""

    name: str
    dtype_tag: str
    shape: tuple[int, ...]
    file: "SafetensorsFile"
    begin: int
    end: int

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype_tag][1]

    def read(self) -> torch.Tensor:
        """The tensor as a CPU torch tensor backed by the mapped file (copy before the file closes)."""
        np_dtype, t_dtype = _DTYPES[self.dtype_tag]
        buf = self.file.data[self.begin:self.end]
        arr = np.frombuffer(buf, dtype=np_dtype).reshape(self.shape)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")      # the mapping is read-only; callers copy before writing
            t = torch.from_numpy(arr.copy() if arr.size == 0 else arr)
        if t_dtype is torch.bfloat16:
            t = t.view(torch.bfloat16)
        elif t_dtype is torch.bool:
            t = t.bool()
        return t


class SafetensorsFile:
    def __init__(self, path: str | Path):
        self.path = Path(path)
        with open(self.path, "rb") as f:
            head = f.read(8)
            if len(head) != 8:
                raise CheckpointFormatError(f"{self.path}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            size = self.path.stat().st_size
            if n <= 0 or 8 + n > size:
                raise CheckpointFormatError(f"{self.path}: header length {n} does not fit the file")
            try:
                header = json.loads(f.read(n).decode("utf-8"))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise CheckpointFormatError(f"{self.path}: header is not JSON ({e})") from None
            self._f = open(self.path, "rb")
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self.data = memoryview(self._map)[8 + n:]
        self.metadata = header.pop("__metadata__", {}) or {}
        self.tensors: dict[str, StoredTensor] = {}
        for name, info in header.items():
            tag = info.get("dtype")
            if tag not in _DTYPES:
                raise CheckpointFormatError(f"{self.path}: tensor {name!r} has unknown dtype {tag!r}")
            shape = tuple(int(s) for s in info["shape"])
            b, e = (int(x) for x in info["data_offsets"])
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[tag][0].itemsize if shape else _DTYPES[tag][0].itemsize
            if e - b != want or e > len(self.data) or b < 0:
                raise CheckpointFormatError(
                    f"{self.path}: tensor {name!r} of shape {shape} and dtype {tag} does not match its byte range")
            self.tensors[name] = StoredTensor(name, tag, shape, self, b, e)


def write_safetensors(path: str | Path, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Write CPU tensors under their names, in name order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name in sorted(tensors):
        t = tensors[name].detach().cpu().contiguous()
        if t.dtype not in _TAG_OF:
            raise ValueError(f"cannot store dtype {t.dtype}")
        if t.dtype is torch.bfloat16:
            raw = t.view(torch.int16).numpy().tobytes()
        elif t.dtype is torch.bool:
            raw = t.to(torch.uint8).numpy().tobytes()
        else:
            raw = t.numpy().tobytes()
        header[name] = {"dtype": _TAG_OF[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode("utf-8")
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for raw in blobs:
            f.write(raw)


def open_checkpoint(model_dir: str | Path) -> dict[str, StoredTensor]:
    """All tensors of a model folder, single-file or sharded.

    ``model.safetensors`` if present, else the shards that
    ``model.safetensors.index.json`` lists under ``weight_map``
    (engine/llama_weights.py:121-144 has the same order and the same errors).
    """
    model_dir = Path(model_dir)
    if not model_dir.is_dir():
        raise FileNotFoundError(f"model directory not found: {model_dir}")
    single = model_dir / "model.safetensors"
    index = model_dir / "model.safetensors.index.json"
    if single.is_file():
        return dict(SafetensorsFile(single).tensors)
    if index.is_file():
        with open(index) as f:
            weight_map = json.load(f)["weight_map"]
        out: dict[str, StoredTensor] = {}
        for shard in sorted(set(weight_map.values())):
            shard_path = model_dir / shard
            if not shard_path.is_file():
                raise FileNotFoundError(f"shard not found: {shard_path}")
            out.update(SafetensorsFile(shard_path).tensors)
        return out
    raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json found in {model_dir}")

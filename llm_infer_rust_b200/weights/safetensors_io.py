"""Reading and writing the safetensors container, tensor by tensor.

Format: 8 bytes little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": ...}``,
then the raw little-endian data.  The file is memory-mapped; a tensor is copied
only when it is asked for.

File discovery follows the reference (src/engine/model_loader.rs:124-175):
``model.safetensors``, else the shards named by ``model.safetensors.index.json``
(absolute paths and ``..`` are refused; a tensor name that appears in two shards
is an error, model_loader.rs:108-122).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(IOError):
    pass


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        self._fh = open(path, "rb")
        try:
            self._read_header()
            self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ)
        except Exception:
            self._fh.close()
            raise

    def _read_header(self) -> None:
        path = self.path
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short for a safetensors header")
        (header_len,) = struct.unpack("<Q", self._fh.read(8))
        if header_len > size - 8:
            raise SafetensorsError(f"{path}: header length {header_len} exceeds the file")
        try:
            header = json.loads(self._fh.read(header_len))
        except ValueError as err:
            raise SafetensorsError(f"{path}: header is not JSON: {err}") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        header.pop("__metadata__", None)
        self._data_start = 8 + header_len
        for name, info in header.items():
            try:
                code, shape, (begin, end) = info["dtype"], tuple(info["shape"]), info["data_offsets"]
                if any(isinstance(v, bool) or not isinstance(v, int) or v < 0 for v in shape + (begin, end)):
                    raise ValueError("sizes and offsets must be non-negative integers")
            except (KeyError, TypeError, ValueError) as err:
                raise SafetensorsError(f"{path}: tensor {name} has a malformed header entry: {err!r}") from None
            if code not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {code}")
            dtype = _DTYPES[code]
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * torch.empty(0, dtype=dtype).element_size() \
                    or self._data_start + end > size:
                raise SafetensorsError(f"{path}: tensor {name} has inconsistent offsets")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor that owns its memory (copied out of the mapping)."""
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        raw = np.frombuffer(self._map, dtype=np.uint8, count=end - begin,
                            offset=self._data_start + begin).copy()
        return torch.from_numpy(raw).view(dtype).reshape(shape)

    def close(self) -> None:
        try:
            self._map.close()
        except BufferError:
            pass
        self._fh.close()


def discover(model_dir: str) -> List[str]:
    """Paths of the safetensors files of a model folder."""
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.isfile(single):
        return [single]
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if not os.path.isfile(index):
        raise SafetensorsError(f"{model_dir}: neither model.safetensors nor "
                               f"model.safetensors.index.json is there")
    try:
        with open(index) as fh:
            weight_map = json.load(fh)["weight_map"]
        shards = sorted(set(weight_map.values()))
    except (ValueError, KeyError, TypeError, AttributeError) as err:
        raise SafetensorsError(f"{index}: invalid index: {err!r}") from None
    paths = []
    for shard in shards:
        if not isinstance(shard, str) or os.path.isabs(shard) or ".." in shard.split("/") \
                or "\\" in shard:
            raise SafetensorsError(f"{index}: shard path {shard!r} leaves the model folder")
        paths.append(os.path.join(model_dir, shard))
    if not paths:
        raise SafetensorsError(f"{index}: names no shard")
    return paths


class Checkpoint:
    """All tensors of a model folder, by name."""

    def __init__(self, model_dir: str):
        self.files = [SafetensorsFile(p) for p in discover(model_dir)]
        self._where: Dict[str, SafetensorsFile] = {}
        for f in self.files:
            for name in f.names():
                if name in self._where:
                    raise SafetensorsError(f"tensor {name} is stored in both {self._where[name].path} "
                                           f"and {f.path}")
                self._where[name] = f

    def names(self) -> List[str]:
        return list(self._where)

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def info(self, name: str):
        return self._where[name].info(name)

    def read(self, name: str) -> torch.Tensor:
        return self._where[name].read(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write (name, tensor) pairs; the tensors are stored in the order given."""
    header = {}
    blobs = []
    offset = 0
    for name, t in tensors:
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    text = json.dumps(header, separators=(",", ":")).encode()
    text += b" " * ((8 - len(text) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(text)))
        fh.write(text)
        for raw in blobs:
            fh.write(raw)

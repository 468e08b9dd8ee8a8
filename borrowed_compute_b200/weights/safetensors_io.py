"""Reading and writing safetensors files without any model library.

The format: eight bytes (little-endian length N of the header), N bytes of JSON mapping a
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to
the end of the header), then the raw little-endian data.  Files are memory-mapped; a
tensor is materialised only when asked for.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Mapping, Tuple

import torch

from ..config.errors import WeightsError

_DTYPES = {
    "F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        try:
            self._file = open(path, "rb")
        except OSError as e:
            raise WeightsError(f"cannot open {path}: {e}") from e
        head = self._file.read(8)
        if len(head) != 8:
            raise WeightsError(f"{path}: too short to be a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = os.path.getsize(path)
        if n <= 0 or 8 + n > size:
            raise WeightsError(f"{path}: header length {n} does not fit the file's {size} bytes")
        try:
            header = json.loads(self._file.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise WeightsError(f"{path}: the header is not JSON: {e}") from e
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + n
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            if e.get("dtype") not in _DTYPES:
                raise WeightsError(f"{path}: tensor {name} has unsupported dtype {e.get('dtype')!r}")
            dtype, shape = _DTYPES[e["dtype"]], tuple(int(s) for s in e["shape"])
            begin, end = (int(o) for o in e["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * dtype.itemsize or self._base + end > size or begin < 0:
                raise WeightsError(f"{path}: tensor {name} spans {end - begin} bytes, its shape {shape} needs {count * dtype.itemsize}")
            self.entries[name] = (dtype, shape, begin, end)

    def names(self) -> List[str]:
        return list(self.entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dtype, shape, _, _ = self.entries[name]
        return dtype, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped file (read-only: copy before writing)."""
        dtype, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        view = memoryview(self._map)[self._base + begin: self._base + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)   # the mapping is read-only on purpose
            return torch.frombuffer(view, dtype=dtype).reshape(shape)


def write_safetensors(path: str, tensors: Mapping[str, torch.Tensor], metadata: Mapping[str, str] | None = None) -> None:
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise WeightsError(f"cannot store tensor {name} of type {t.dtype}")
        n = t.numel() * t.dtype.itemsize
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
        offset += n
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")


class TensorSource:
    """All tensors of a model folder: ``model.safetensors``, or the shards that
    ``model.safetensors.index.json`` lists."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self._files: List[SafetensorsFile] = []
        self._where: Dict[str, SafetensorsFile] = {}
        if os.path.isfile(single):
            paths: Iterable[str] = [single]
        elif os.path.isfile(index):
            try:
                with open(index) as f:
                    weight_map = json.load(f)["weight_map"]
            except (OSError, KeyError, json.JSONDecodeError) as e:
                raise WeightsError(f"{index}: not a shard index: {e}") from e
            paths = sorted({os.path.join(folder, v) for v in weight_map.values()})
        else:
            raise WeightsError(f"{folder} has neither model.safetensors nor model.safetensors.index.json")
        for p in paths:
            f = SafetensorsFile(p)
            self._files.append(f)
            for name in f.names():
                self._where[name] = f

    def names(self) -> List[str]:
        return list(self._where)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        return self._where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self._where[name].tensor(name)

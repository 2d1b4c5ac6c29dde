"""Reader and writer for the safetensors container.

Format (as the reference reads it, src/frontend/loader/safetensor.cpp:105-150 and
:224-241): 8 bytes little-endian header length ``n``; ``n`` bytes of JSON mapping a
tensor name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (``__metadata__``
is skipped); then the data, offsets relative to byte ``8 + n``.  The reader maps the
file and hands out zero-copy views; bounds and sizes are checked before any view
is made.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Mapping, Tuple

import numpy as np
import torch

# name in the file → (bytes per element, numpy carrier dtype, torch dtype)
_DTYPES = {
    "BOOL": (1, np.uint8, torch.bool),
    "U8": (1, np.uint8, torch.uint8),
    "I8": (1, np.int8, torch.int8),
    "I16": (2, np.int16, torch.int16),
    "I32": (4, np.int32, torch.int32),
    "I64": (8, np.int64, torch.int64),
    "F16": (2, np.int16, torch.float16),
    "BF16": (2, np.int16, torch.bfloat16),
    "F32": (4, np.float32, torch.float32),
    "F64": (8, np.float64, torch.float64),
}
_TORCH_TO_NAME = {v[2]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "begin", "end", "file")

    def __init__(self, name: str, dtype: str, shape: Tuple[int, ...], begin: int, end: int, file: "SafetensorsFile"):
        self.name, self.dtype, self.shape, self.begin, self.end, self.file = name, dtype, shape, begin, end, file

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][2]

    def load(self) -> torch.Tensor:
        """A CPU tensor that views the mapped file (read-only memory: clone before writing)."""
        return self.file._view(self)


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too small to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not valid JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self._data_start = 8 + hlen
        data_len = size - self._data_start
        self.entries: Dict[str, TensorEntry] = {}
        for name, info in header.items():
            if name == "__metadata__":
                continue
            try:
                dtype = info["dtype"]
                shape = tuple(int(s) for s in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{path}: malformed entry for tensor '{name}': {e}") from e
            if dtype not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor '{name}' has unknown dtype {dtype!r}")
            if begin < 0 or end < begin or end > data_len:
                raise SafetensorsError(f"{path}: tensor '{name}' has invalid data_offsets [{begin}, {end}) "
                                       f"for {data_len} bytes of data")
            numel = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor '{name}' has a negative dimension in {shape}")
                numel *= s
            if numel * _DTYPES[dtype][0] != end - begin:
                raise SafetensorsError(f"{path}: tensor '{name}' of shape {list(shape)} and dtype {dtype} needs "
                                       f"{numel * _DTYPES[dtype][0]} bytes, but its data_offsets span {end - begin}")
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end, self)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def _view(self, e: TensorEntry) -> torch.Tensor:
        _, np_dtype, torch_dtype = _DTYPES[e.dtype]
        count = (e.end - e.begin) // np.dtype(np_dtype).itemsize
        arr = np.frombuffer(self._mm, dtype=np_dtype, count=count, offset=self._data_start + e.begin)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")   # torch warns that the mapped array is read-only
            t = torch.from_numpy(arr)
        if t.dtype != torch_dtype:
            t = t.view(torch_dtype)
        return t.reshape(e.shape)

    def close(self) -> None:
        # Views keep the map alive through numpy's buffer reference; dropping ours is enough.
        self._mm = None
        self._f.close()


def open_model_files(model_dir: str) -> List[SafetensorsFile]:
    """Every ``*.safetensors`` of a folder, in sorted order (src/frontend/loader/safetensor.cpp:268-304)."""
    if not os.path.isdir(model_dir):
        raise SafetensorsError(f"Model path does not exist: {model_dir}")
    names = sorted(n for n in os.listdir(model_dir) if n.endswith(".safetensors"))
    if not names:
        raise SafetensorsError(f"No .safetensors files found in {model_dir}")
    return [SafetensorsFile(os.path.join(model_dir, n)) for n in names]


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Mapping[str, str] | None = None) -> None:
    """Write tensors (any device; written from CPU copies) in name order."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _TORCH_TO_NAME:
            raise SafetensorsError(f"cannot store tensor '{name}' of dtype {t.dtype}")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _TORCH_TO_NAME[t.dtype], "shape": list(t.shape),
                        "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().to("cpu").contiguous()
            carrier = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64}[t.element_size()]
            f.write(t.view(carrier).numpy().tobytes())
    os.replace(tmp, path)


def iter_entries(files: Iterable[SafetensorsFile]):
    for f in files:
        for e in f.entries.values():
            yield e

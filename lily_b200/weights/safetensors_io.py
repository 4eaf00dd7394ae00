"""Reading and writing the safetensors container, by tensor name.

The format is an 8-byte little-endian header length, a JSON header
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}}``
and the raw little-endian tensor bytes.  Files are memory-mapped; a tensor is only
touched when it is asked for, so checks on names and shapes read the header alone.

Takes the place of ``safetensors.safe_open`` in lily/models/loader.py:55-56,87-95;
shard discovery follows loader.py:24-33.
"""

from __future__ import annotations

import glob
import json
import mmap
import os
import struct
import warnings
from typing import Callable, Dict, List, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


def safetensors_files(model_dir: str) -> List[str]:
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
        return [os.path.join(model_dir, x) for x in files]
    files = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no safetensors files in {model_dir}")
    return files


class SafetensorsFile:
    """One memory-mapped file: ``entries`` maps a name to (torch dtype, shape)."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{path}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n > size - 8 or n > (100 << 20):
                raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
            try:
                header = json.loads(f.read(n))
            except (UnicodeDecodeError, json.JSONDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self._base = 8 + n
        self.metadata: Dict[str, str] = header.pop("__metadata__", {}) or {}
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
        self._spans: Dict[str, Tuple[int, int]] = {}
        for name, info in header.items():
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {info['dtype']}")
            dtype, shape = _DTYPES[info["dtype"]], tuple(int(s) for s in info["shape"])
            begin, end = (int(x) for x in info["data_offsets"])
            count = 1
            for s in shape:
                count *= s
            if end - begin != count * torch.empty((), dtype=dtype).element_size() or self._base + end > size:
                raise SafetensorsError(f"{path}: tensor {name!r} {shape} does not match its bytes [{begin}, {end})")
            self.entries[name] = (dtype, shape)
            self._spans[name] = (begin, end)

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor that views the mapped file (copy it before the file is closed)."""
        dtype, shape = self.entries[name]
        begin, end = self._spans[name]
        if end == begin:
            return torch.empty(shape, dtype=dtype)
        buf = memoryview(self._map)[self._base + begin:self._base + end]
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)      # the mapping is read-only on purpose
            return torch.frombuffer(buf, dtype=dtype).view(shape)


def write_safetensors(path: str, tensors, metadata: Optional[Dict[str, str]] = None,
                      produce: Optional[Callable[[str], torch.Tensor]] = None) -> None:
    """Writes a file.  ``tensors`` is a dict name -> tensor, or, with ``produce``, a list of
    (name, dtype, shape) whose tensors ``produce(name)`` makes one at a time while the file
    is written (a large model is never held in memory whole)."""
    if produce is None:
        held = dict(tensors)
        entries = [(n, t.dtype, tuple(t.shape)) for n, t in held.items()]
        produce = held.__getitem__
    else:
        entries = [(n, d, tuple(s)) for n, d, s in tensors]
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    for name, dtype, shape in entries:
        if dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {dtype} ({name})")
        count = 1
        for s in shape:
            count *= s
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        header[name] = {"dtype": _NAMES[dtype], "shape": list(shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name, dtype, shape in entries:
            t = produce(name)
            if t.dtype != dtype or tuple(t.shape) != shape:
                raise SafetensorsError(f"{name}: produced {t.dtype} {tuple(t.shape)}, declared {dtype} {shape}")
            c = t.detach().contiguous().cpu().reshape(-1)
            if c.numel():
                f.write(c.view(torch.uint8).numpy().data)
    os.replace(tmp, path)

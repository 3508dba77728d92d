"""Minimal safetensors reader and writer (the format: 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}``, then raw
little-endian tensor bytes).  The reader maps the file and hands out zero-copy CPU
tensors; nothing is copied until a tensor is moved to the device.

The reference never reads safetensors at run time: an offline converter
(tools/prepare_model/utils.py:72-150) reads them and writes one ``model.pth``.
The discovery order here is the converter's (utils.py:80-104): a sharded index
first, then a single ``model.safetensors``.
"""
from __future__ import annotations

import json
import mmap
import struct
import warnings
from pathlib import Path
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16, "F64": torch.float64,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One mapped ``.safetensors`` file: ``entries`` is name -> (dtype, shape)."""

    def __init__(self, path):
        self.path = Path(path)
        self._fh = open(self.path, "rb")
        head = self._fh.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: not a safetensors file (too short)")
        (hlen,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if hlen > size - 8:
            raise ValueError(f"{self.path}: header length {hlen} exceeds file size {size}")
        header = json.loads(self._fh.read(hlen))
        self._base = 8 + hlen
        self._map = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None
        self._meta: Dict[str, dict] = {k: v for k, v in header.items() if k != "__metadata__"}
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...]]] = {}
        for name, m in self._meta.items():
            if m["dtype"] not in _DTYPES:
                raise ValueError(f"{self.path}: tensor '{name}' has unsupported dtype {m['dtype']}")
            self.entries[name] = (_DTYPES[m["dtype"]], tuple(m["shape"]))

    def tensor(self, name: str) -> torch.Tensor:
        m = self._meta[name]
        dtype, shape = self.entries[name]
        begin, end = m["data_offsets"]
        count = 1
        for s in shape:
            count *= s
        if count == 0:
            return torch.empty(shape, dtype=dtype)
        if (end - begin) != count * torch.empty((), dtype=dtype).element_size():
            raise ValueError(f"{self.path}: tensor '{name}' byte range does not match its shape")
        with warnings.catch_warnings():
            warnings.simplefilter("ignore", UserWarning)       # the read-only map is never written through
            t = torch.frombuffer(self._map, dtype=dtype, count=count, offset=self._base + begin)
        return t.reshape(shape)


def open_model_files(model_dir) -> List[SafetensorsFile]:
    model_dir = Path(model_dir)
    index = model_dir / "model.safetensors.index.json"
    if index.is_file():
        shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        missing = [s for s in shards if not (model_dir / s).is_file()]
        if missing:
            raise FileNotFoundError(f"{index} lists shards that are absent: {missing}")
        return [SafetensorsFile(model_dir / s) for s in shards]
    single = model_dir / "model.safetensors"
    if single.is_file():
        return [SafetensorsFile(single)]
    raise FileNotFoundError(f"no model.safetensors or model.safetensors.index.json in {model_dir}")


def write_safetensors(path, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write (name, CPU tensor) pairs in the given order; data 8-byte aligned."""
    items = [(n, t.detach().contiguous().cpu()) for n, t in tensors]
    header, offset = {}, 0
    for name, t in items:
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as fh:
        fh.write(struct.pack("<Q", len(blob)))
        fh.write(blob)
        for _, t in items:
            fh.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())

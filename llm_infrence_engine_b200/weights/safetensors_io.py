"""Reading and writing the safetensors container: an 8-byte header length, a JSON header, raw bytes.

Tensors are read one by one from a memory map by name, so a checkpoint never has to fit in host
memory twice. The reference merges every ``*.safetensors`` file of a folder into one dictionary
with the safetensors package (src/miniserve/loader.py:41-43); the container is simple enough to
read here directly.
"""
from __future__ import annotations

import json
import mmap
import struct
from pathlib import Path
from typing import Dict, Iterable, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """One open ``.safetensors`` file: ``names()``, ``info(name)`` and ``tensor(name)``."""

    def __init__(self, path: str | Path):
        self.path = Path(path)
        self._f = open(self.path, "rb")
        head = self._f.read(8)
        if len(head) != 8:
            raise ValueError(f"{self.path}: too short for a safetensors file")
        (n,) = struct.unpack("<Q", head)
        size = self.path.stat().st_size
        if n > size - 8:
            raise ValueError(f"{self.path}: header length {n} exceeds the file")
        try:
            self._header = json.loads(self._f.read(n))
        except json.JSONDecodeError as e:
            raise ValueError(f"{self.path}: header is not JSON: {e}") from None
        self._header.pop("__metadata__", None)
        self._base = 8 + n
        self._map = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > 0 else None

    def names(self) -> Iterable[str]:
        return self._header.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        e = self._header[name]
        if e["dtype"] not in _DTYPES:
            raise ValueError(f"{self.path}: tensor '{name}' has dtype {e['dtype']}, which is not read here")
        return _DTYPES[e["dtype"]], tuple(e["shape"])

    def tensor(self, name: str) -> torch.Tensor:
        """A copy of the tensor on the host, in the dtype it is stored in."""
        dtype, shape = self.info(name)
        begin, end = self._header[name]["data_offsets"]
        numel = 1
        for s in shape:
            numel *= s
        want = numel * torch.empty((), dtype=dtype).element_size()
        if end - begin != want:
            raise ValueError(f"{self.path}: tensor '{name}' has {end - begin} bytes, its shape needs {want}")
        if numel == 0:
            return torch.empty(shape, dtype=dtype)
        raw = bytearray(self._map[self._base + begin:self._base + end])  # a private, writable, aligned copy
        return torch.frombuffer(raw, dtype=dtype, count=numel).reshape(shape)

    def close(self) -> None:
        if self._map is not None:
            self._map.close()
            self._map = None
        self._f.close()


def write_safetensors(path: str | Path, tensors: Dict[str, torch.Tensor]) -> None:
    header, offset, blobs = {}, 0, []
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        if t.dtype not in _NAMES:
            raise ValueError(f"tensor '{name}' has dtype {t.dtype}, which cannot be written")
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + len(raw)]}
        offset += len(raw)
        blobs.append(raw)
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for raw in blobs:
            f.write(raw)


def write_safetensors_stream(path: str | Path, metas, produce) -> None:
    """The same file as ``write_safetensors``, one tensor at a time: ``metas`` lists ``(name, dtype, shape)`` in file order,
    ``produce(name)`` returns that tensor when its turn comes. Nothing but the tensor being written is held in memory,
    which lets folders of many gigabytes be written."""
    header, offset = {}, 0
    for name, dtype, shape in metas:
        if dtype not in _NAMES:
            raise ValueError(f"tensor '{name}' has dtype {dtype}, which cannot be written")
        n = torch.empty((), dtype=dtype).element_size()
        for d in shape:
            n *= int(d)
        header[name] = {"dtype": _NAMES[dtype], "shape": [int(d) for d in shape], "data_offsets": [offset, offset + n]}
        offset += n
    head = json.dumps(header, separators=(",", ":")).encode()
    head += b" " * (-len(head) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for name, dtype, shape in metas:
            t = produce(name).detach().cpu().contiguous()
            if t.dtype != dtype or tuple(t.shape) != tuple(shape):
                raise ValueError(f"tensor '{name}' came as {t.dtype} {list(t.shape)}, announced as {dtype} {list(shape)}")
            if t.numel():
                f.write(memoryview(t.view(torch.uint8).numpy().reshape(-1)))

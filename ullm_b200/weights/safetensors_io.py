"""Reading and writing the safetensors container without any library: an
8-byte little-endian header length, a JSON header {name: {dtype, shape,
data_offsets}}, then the raw little-endian tensor bytes.

ullm/model_loader.py:25-41 iterates (name, tensor) pairs out of every
*.safetensors file of the folder; `SafetensorsFile` gives the same by name,
memory-mapped, so a tensor's bytes are only touched when it is copied to the
device.
"""

from __future__ import annotations

import glob
import json
import mmap
import os
import struct
from typing import Iterable, Iterator

import torch

_DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F64": torch.float64,
    "I32": torch.int32,
    "I64": torch.int64,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        self._f = open(path, "rb")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n <= 0 or 8 + n > size:
            raise SafetensorsError(f"{path}: header length {n} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self.entries: dict[str, dict] = header
        self._base = 8 + n
        self._size = size
        self._mm = None
        for name, e in self.entries.items():
            if e.get("dtype") not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unknown dtype {e.get('dtype')!r}")
            b, end = e["data_offsets"]
            numel = 1
            for s in e["shape"]:
                numel *= s
            want = numel * torch.empty((), dtype=_DTYPES[e["dtype"]]).element_size()
            if end - b != want or self._base + end > size:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} {e['dtype']}{e['shape']} needs {want} bytes, "
                    f"offsets give {end - b} (file is truncated or corrupt)"
                )

    def names(self) -> list[str]:
        return list(self.entries)

    def shape(self, name: str) -> tuple[int, ...]:
        return tuple(self.entries[name]["shape"])

    def dtype(self, name: str) -> torch.dtype:
        return _DTYPES[self.entries[name]["dtype"]]

    def get(self, name: str) -> torch.Tensor:
        """A CPU tensor viewing the mapped file (read-only memory: copy, do not write)."""
        e = self.entries[name]
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        b, end = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        if end == b:
            return torch.empty(tuple(e["shape"]), dtype=dt)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            flat = torch.frombuffer(self._mm, dtype=torch.uint8, count=end - b, offset=self._base + b)
        return flat.view(dt).reshape(tuple(e["shape"]))

    def close(self) -> None:
        self._mm = None
        self._f.close()


def open_model_files(model_dir: str) -> list[SafetensorsFile]:
    paths = sorted(glob.glob(os.path.join(model_dir, "*.safetensors")))
    if not paths:
        raise FileNotFoundError(f"no *.safetensors file in {model_dir}")
    return [SafetensorsFile(p) for p in paths]


def write_safetensors(
    path: str,
    decls: list[tuple[str, torch.dtype, tuple[int, ...]]],
    tensors: Iterable[tuple[str, torch.Tensor]],
    metadata: dict[str, str] | None = None,
) -> None:
    """Streams tensors into `path`.  `decls` fixes order, dtype and shape up
    front (the header comes first in the file); `tensors` must yield the same
    names in the same order."""
    header: dict[str, dict] = {}
    off = 0
    for name, dt, shape in decls:
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * torch.empty((), dtype=dt).element_size()
        header[name] = {"dtype": _NAMES[dt], "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    if metadata:
        header["__metadata__"] = metadata
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * ((8 - len(raw) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        it: Iterator = iter(tensors)
        for name, dt, shape in decls:
            got_name, t = next(it)
            if got_name != name or t.dtype != dt or tuple(t.shape) != tuple(shape):
                raise SafetensorsError(
                    f"writer: expected {name} {dt} {tuple(shape)}, got {got_name} {t.dtype} {tuple(t.shape)}"
                )
            t = t.contiguous().cpu()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)


def save_tensors(path: str, tensors: dict[str, torch.Tensor], metadata=None) -> None:
    decls = [(n, t.dtype, tuple(t.shape)) for n, t in tensors.items()]
    write_safetensors(path, decls, tensors.items(), metadata)

"""Reading and writing the safetensors container.

Layout: an 8-byte little-endian header length, a JSON header mapping each tensor
name to ``{"dtype", "shape", "data_offsets": [begin, end]}`` (offsets relative to
the end of the header), then the payload.  The reference parses the same layout
in crates/shiso-modelfile/src/st_header.rs:1-25,37-46.  Files are memory-mapped
and tensors are views of the mapping until they are copied to the device.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from dataclasses import dataclass

import torch

_DTYPES = {
    "F32": torch.float32,
    "BF16": torch.bfloat16,
    "F16": torch.float16,
    "F64": torch.float64,
    "I64": torch.int64,
    "I32": torch.int32,
    "I16": torch.int16,
    "I8": torch.int8,
    "U8": torch.uint8,
    "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}
_MAX_HEADER = 100 * 1024 * 1024


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: tuple[int, ...]
    begin: int
    end: int


class SafetensorsFile:
    """A memory-mapped safetensors file: a directory of entries and lazy tensor views."""

    def __init__(self, path: str):
        self.path = path
        size = os.path.getsize(path)
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a header length")
        self._file = open(path, "rb")
        self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        (header_len,) = struct.unpack("<Q", self._map[:8])
        if header_len > _MAX_HEADER or 8 + header_len > size:
            raise SafetensorsError(f"{path}: header length {header_len} does not fit the file")
        try:
            header = json.loads(self._map[8 : 8 + header_len].decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from e
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not a JSON object")
        self._payload = 8 + header_len
        payload_size = size - self._payload
        self.metadata = header.pop("__metadata__", {}) or {}
        self.entries: dict[str, TensorEntry] = {}
        for name, info in header.items():
            try:
                dtype = _DTYPES[info["dtype"]]
                shape = tuple(int(d) for d in info["shape"])
                begin, end = (int(x) for x in info["data_offsets"])
            except (KeyError, TypeError, ValueError) as e:
                raise SafetensorsError(f"{path}: tensor {name!r}: bad header entry {info!r}") from e
            count = 1
            for d in shape:
                count *= d
            if begin < 0 or end > payload_size or end - begin != count * dtype.itemsize:
                raise SafetensorsError(
                    f"{path}: tensor {name!r}: offsets [{begin}, {end}) do not hold "
                    f"{count} x {info['dtype']} inside a payload of {payload_size} bytes"
                )
            self.entries[name] = TensorEntry(name, dtype, shape, begin, end)

    def names(self) -> list[str]:
        return list(self.entries)

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only view of the mapping; copy it before the file is closed."""
        entry = self.entries[name]
        count = 1
        for d in entry.shape:
            count *= d
        if count == 0:
            return torch.empty(entry.shape, dtype=entry.dtype)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes through the view
            flat = torch.frombuffer(
                self._map, dtype=entry.dtype, count=count, offset=self._payload + entry.begin
            )
        return flat.view(entry.shape)

    def close(self) -> None:
        # Tensor views keep the mapping alive through the buffer protocol; the
        # mapping is dropped with the last of them.
        self._file.close()


def write_safetensors(path: str, tensors: dict[str, torch.Tensor], metadata: dict | None = None) -> None:
    """Writes ``tensors`` (CPU, any supported dtype) in sorted-name order."""
    header: dict = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    order = sorted(tensors)
    for name in order:
        t = tensors[name]
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} has no safetensors name")
        nbytes = t.numel() * t.dtype.itemsize
        header[name] = {
            "dtype": _NAMES[t.dtype],
            "shape": list(t.shape),
            "data_offsets": [offset, offset + nbytes],
        }
        offset += nbytes
    blob = json.dumps(header, separators=(",", ":")).encode("utf-8")
    blob += b" " * ((8 - len(blob) % 8) % 8)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for name in order:
            t = tensors[name].detach().cpu().contiguous()
            f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    os.replace(tmp, path)

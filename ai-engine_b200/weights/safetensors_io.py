"""A reader and a writer for the safetensors container, by tensor name.

Format: 8 bytes little-endian header length N, N bytes of JSON
{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": {...}},
then the raw little-endian tensor bytes.  The reference reads it with the
safetensors crate over an mmap (crates/ai-engine-runtime/src/loader.rs:50-63);
this is the same access pattern without that library: the file is mapped, and
a tensor is a view of its byte range until it is copied to the device.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

# safetensors dtype name -> (torch dtype, numpy carrier dtype of the same width)
_DTYPES = {
    "F32": (torch.float32, np.dtype("<f4")),
    "F16": (torch.float16, np.dtype("<f2")),
    "BF16": (torch.bfloat16, np.dtype("<u2")),
    "F64": (torch.float64, np.dtype("<f8")),
    "I64": (torch.int64, np.dtype("<i8")),
    "I32": (torch.int32, np.dtype("<i4")),
    "I16": (torch.int16, np.dtype("<i2")),
    "I8": (torch.int8, np.dtype("i1")),
    "U8": (torch.uint8, np.dtype("u1")),
    "BOOL": (torch.bool, np.dtype("u1")),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One mapped *.safetensors file: `names()`, `info(name)`, `tensor(name)`."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._f = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open: {e}") from None
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file ({size} bytes)")
        (n,) = struct.unpack("<Q", self._f.read(8))
        if n > size - 8:
            raise SafetensorsError(f"{path}: header length {n} exceeds the file ({size} bytes): truncated?")
        try:
            header = json.loads(self._f.read(n))
        except (json.JSONDecodeError, UnicodeDecodeError) as e:
            raise SafetensorsError(f"{path}: header is not JSON: {e}") from None
        self.metadata = header.pop("__metadata__", None) or {}
        self._base = 8 + n
        self._entries: Dict[str, Tuple[str, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            dt, shape, (b, en) = e["dtype"], tuple(e["shape"]), e["data_offsets"]
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor `{name}` has unsupported dtype {dt}")
            want = int(np.prod(shape, dtype=np.int64)) * _DTYPES[dt][1].itemsize
            if en - b != want or self._base + en > size:
                raise SafetensorsError(
                    f"{path}: tensor `{name}` {dt}{list(shape)} needs {want} bytes but its range "
                    f"[{b}, {en}) holds {en - b} (file has {size - self._base} data bytes): truncated?")
            self._entries[name] = (dt, shape, b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self._entries[name]
        return _DTYPES[dt][0], shape

    def tensor(self, name: str) -> torch.Tensor:
        """A CPU tensor over the mapped bytes (read-only memory: copy before writing)."""
        dt, shape, b, e = self._entries[name]
        tdt, ndt = _DTYPES[dt]
        count = int(np.prod(shape, dtype=np.int64))
        if count == 0:
            return torch.empty(shape, dtype=tdt)
        arr = np.frombuffer(self._mm, dtype=ndt, count=count, offset=self._base + b)
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # non-writable buffer: it is only read
            t = torch.from_numpy(arr)
        if tdt == torch.bfloat16:
            t = t.view(torch.int16).view(torch.bfloat16)
        elif tdt == torch.bool:
            t = t != 0
        return t.reshape(shape)

    def close(self) -> None:
        if self._mm is not None:
            self._mm.close()
            self._mm = None
        self._f.close()


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]],
                      metadata: Dict[str, str] | None = None) -> None:
    """Write (name, tensor) pairs in order.  Tensors are taken one at a time so a
    generator can produce a model larger than memory would like."""
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = dict(metadata)
    tmp_data = path + ".data.tmp"
    offset = 0
    with open(tmp_data, "wb") as df:
        for name, t in tensors:
            if t.dtype not in _NAMES:
                raise SafetensorsError(f"tensor `{name}`: dtype {t.dtype} cannot be written")
            t = t.detach().cpu().contiguous()
            if t.dtype == torch.bfloat16:
                raw = t.view(torch.int16).numpy().tobytes()
            elif t.dtype == torch.bool:
                raw = t.to(torch.uint8).numpy().tobytes()
            else:
                raw = t.numpy().tobytes()
            header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                            "data_offsets": [offset, offset + len(raw)]}
            df.write(raw)
            offset += len(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as out, open(tmp_data, "rb") as df:
        out.write(struct.pack("<Q", len(hj)))
        out.write(hj)
        while True:
            chunk = df.read(1 << 24)
            if not chunk:
                break
            out.write(chunk)
    os.remove(tmp_data)

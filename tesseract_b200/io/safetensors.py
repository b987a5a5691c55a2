"""safetensors reader (mmap) and writer.

File layout (src/io/SafeTensors.cpp:291-462): 8-byte little-endian header length, a JSON object whose keys
are tensor names -> {"dtype", "shape", "data_offsets": [begin, end]} plus an optional "__metadata__"
string -> string map, then the raw little-endian data region. The reader validates every offset pair against
the data region and against shape x dtype size, rejects trailing garbage after the header object, skips
unknown per-tensor fields, and returns keys in header order. The reference only reads; the writer here emits
the same layout (sorted by name, 8-byte aligned header) so that checkpoints round-trip with Hugging Face tools.
"""
from __future__ import annotations

import json
import mmap
import struct
from typing import Dict, Iterable, List, Optional

import numpy as np
import torch

_DTYPES = {
    "F32": (torch.float32, 4), "F64": (torch.float64, 8), "F16": (torch.float16, 2), "BF16": (torch.bfloat16, 2),
    "I32": (torch.int32, 4), "I64": (torch.int64, 8), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1), "F8_E4M3": (torch.float8_e4m3fn, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafeTensorsError(ValueError):
    pass


class SafeTensors:
    """Read-only view of one file; tensors are copied out of the mapping on ``load``."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        try:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:
            self._f.close()
            raise SafeTensorsError(f"{path}: empty file") from None
        size = len(self._mm)
        if size < 8:
            raise SafeTensorsError(f"{path}: shorter than the 8-byte header length")
        (hlen,) = struct.unpack("<Q", self._mm[:8])
        if hlen < 2 or 8 + hlen > size:
            raise SafeTensorsError(f"{path}: header length {hlen} exceeds the file")
        raw = bytes(self._mm[8:8 + hlen])
        try:
            dec = json.JSONDecoder()
            text = raw.decode("utf-8")
            header, end = dec.raw_decode(text.lstrip())
            rest = text.lstrip()[end:]
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise SafeTensorsError(f"{path}: malformed header JSON ({e})") from None
        if rest.strip(" \t\r\n\x00") != "":
            raise SafeTensorsError(f"{path}: trailing bytes after the header object")
        if not isinstance(header, dict):
            raise SafeTensorsError(f"{path}: header is not a JSON object")
        self._data_start = 8 + hlen
        data_size = size - self._data_start
        self.metadata: Dict[str, str] = {}
        self._entries: Dict[str, tuple] = {}
        for name, ent in header.items():
            if name == "__metadata__":
                if not isinstance(ent, dict) or any(not isinstance(v, str) for v in ent.values()):
                    raise SafeTensorsError(f"{path}: __metadata__ must map strings to strings")
                self.metadata = dict(ent)
                continue
            try:
                dt, shape, (b, e) = ent["dtype"], list(ent["shape"]), ent["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafeTensorsError(f"{path}: entry {name!r} lacks dtype/shape/data_offsets") from None
            if dt not in _DTYPES:
                raise SafeTensorsError(f"{path}: entry {name!r} has unsupported dtype {dt!r}")
            n = 1
            for d in shape:
                if not isinstance(d, int) or d < 0:
                    raise SafeTensorsError(f"{path}: entry {name!r} has a bad shape")
                n *= d
            if not (0 <= b <= e <= data_size) or e - b != n * _DTYPES[dt][1]:
                raise SafeTensorsError(f"{path}: entry {name!r} has inconsistent data_offsets")
            self._entries[name] = (dt, shape, b, e)

    @classmethod
    def open(cls, path: str) -> "SafeTensors":
        return cls(path)

    def keys(self) -> List[str]:
        return list(self._entries.keys())

    def __contains__(self, name: str) -> bool:
        return name in self._entries

    def info(self, name: str):
        dt, shape, b, e = self._entries[name]
        return _DTYPES[dt][0], tuple(shape)

    def load(self, name: str, device=None) -> torch.Tensor:
        if name not in self._entries:
            raise KeyError(f"{self.path}: no tensor named {name!r}")
        dt, shape, b, e = self._entries[name]
        tdt = _DTYPES[dt][0]
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=e - b, offset=self._data_start + b).copy()
        t = torch.from_numpy(buf).view(tdt).reshape(shape) if e > b else torch.empty(shape, dtype=tdt)
        return t.to(device) if device is not None else t

    def close(self) -> None:
        try:
            self._mm.close()
        finally:
            self._f.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    """Write ``tensors`` (name -> CPU or CUDA tensor) as one safetensors file."""
    header: Dict[str, object] = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    off = 0
    order = sorted(tensors.keys())
    blobs = []
    for name in order:
        t = tensors[name].detach().contiguous().cpu()
        if t.dtype not in _NAMES:
            raise SafeTensorsError(f"save_file: dtype {t.dtype} of {name!r} is not representable")
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nbytes]}
        blobs.append(t)
        off += nbytes
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    pad = (8 - len(hjson) % 8) % 8
    hjson += b" " * pad
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for t in blobs:
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else t.reshape(1).view(torch.uint8).numpy().tobytes())


def load_file(path: str, device=None) -> Dict[str, torch.Tensor]:
    with SafeTensors.open(path) as st:
        return {k: st.load(k, device) for k in st.keys()}


def load_file_parallel(path: str, device=None, threads: int = 8, pin: bool = True) -> Dict[str, torch.Tensor]:
    """Whole-file load through the native host runtime: the data section is read by ``threads`` pread workers
    straight into ONE (pinned) host buffer, the tensors are views of it, and a CUDA ``device`` gets them with
    asynchronous copies from pinned memory. Falls back to ``load_file`` when the runtime is not built."""
    from .. import _native
    host = _native.host()
    if host is None:
        return load_file(path, device)
    with SafeTensors.open(path) as st:
        entries = {k: st._entries[k] for k in st.keys()}
        data_start = st._data_start
    total = max((e for _, _, _, e in entries.values()), default=0)
    buf = torch.empty(max(total, 1), dtype=torch.uint8)
    if pin and torch.cuda.is_available():
        buf = buf.pin_memory()
    if total:
        got = host.read_ranges(path, [data_start], [total], [buf.data_ptr()], threads)
        if got != total:
            raise SafeTensorsError(f"{path}: read {got} of {total} data bytes")
    out = {}
    for name, (dt, shape, b, e) in entries.items():
        tdt = _DTYPES[dt][0]
        if e > b:
            raw = buf[b:e]
            if b % tdt.itemsize:        # the format does not align tensors: a misaligned one is copied to offset 0
                raw = raw.clone()
            t = raw.view(tdt).reshape(shape)
        else:
            t = torch.empty(shape, dtype=tdt)
        out[name] = t.to(device, non_blocking=True) if device is not None else t
    if device is not None and torch.device(device).type == "cuda":
        torch.cuda.synchronize(device)
    return out

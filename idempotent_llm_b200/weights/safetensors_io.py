"""Reading and writing the safetensors container: an 8-byte little-endian header
length, a JSON header ``{name: {dtype, shape, data_offsets}}`` and the raw
tensor bytes (the reference parses the same header by hand in
scripts/quant_report.py:86-93 and loads tensors by name in
src/detllm/model.py:116).  Tensors are memory-mapped and handed out one by
one, so a checkpoint larger than host memory can be moved to the device tensor
by tensor.
"""

from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8,
    "U8": torch.uint8, "BOOL": torch.bool,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


class SafetensorsFile:
    """One ``*.safetensors`` file, memory-mapped read-only."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        size = os.fstat(self._f.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: too short to be a safetensors file")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen <= 0 or 8 + hlen > size:
            raise SafetensorsError(f"{path}: header length {hlen} does not fit the file ({size} bytes)")
        try:
            header = json.loads(self._f.read(hlen))
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        self.metadata = header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        for name, e in header.items():
            b, en = e["data_offsets"]
            # a dtype this reader does not know (an 8-bit float, say) is kept by its name: only asking for
            # such a tensor is an error, so a file may carry tensors the model never declares
            dt = _DTYPES.get(e["dtype"], str(e["dtype"]))
            n = 1
            for s in e["shape"]:
                n *= s
            if not 0 <= b <= en or self._base + en > size:
                raise SafetensorsError(f"{path}: tensor {name!r} has offsets {b}..{en} outside the file's data")
            if isinstance(dt, torch.dtype) and en - b != n * torch.empty((), dtype=dt).element_size():
                raise SafetensorsError(f"{path}: tensor {name!r} has inconsistent offsets")
            self._entries[name] = (dt, tuple(e["shape"]), b, en)
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ) if size > self._base else None

    def names(self) -> List[str]:
        return list(self._entries)

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        """(dtype, shape); the dtype is its name as a string if this reader does not know it."""
        dt, shape, _, _ = self._entries[name]
        return dt, shape

    def get(self, name: str) -> torch.Tensor:
        """A read-only view into the mapping; copy (``.to`` / ``.clone``) before the file closes."""
        dt, shape, b, e = self._entries[name]
        if not isinstance(dt, torch.dtype):
            raise SafetensorsError(f"{self.path}: tensor {name!r} has unsupported dtype {dt}")
        if e == b:
            return torch.empty(shape, dtype=dt)
        buf = memoryview(self._mm)[self._base + b:self._base + e]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # the mapping is read-only; nothing writes through it
            t = torch.frombuffer(buf, dtype=dt)
        return t.view(shape)


class SafetensorsDir:
    """All tensors of a model folder: ``model.safetensors`` alone, or the shards
    named by ``model.safetensors.index.json``."""

    def __init__(self, model_dir: str):
        index = os.path.join(model_dir, "model.safetensors.index.json")
        single = os.path.join(model_dir, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.isfile(single):
            f = SafetensorsFile(single)
            self._files[single] = f
            for n in f.names():
                self._where[n] = single
        elif os.path.isfile(index):
            with open(index) as fh:
                wm = json.load(fh)["weight_map"]
            for n, fname in wm.items():
                p = os.path.join(model_dir, fname)
                if p not in self._files:
                    self._files[p] = SafetensorsFile(p)
                self._where[n] = p
        else:
            raise SafetensorsError(f"{model_dir}: neither model.safetensors nor model.safetensors.index.json")

    def names(self) -> List[str]:
        return list(self._where)

    def info(self, name: str):
        return self._files[self._where[name]].info(name)

    def get(self, name: str) -> torch.Tensor:
        return self._files[self._where[name]].get(name)


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata=None) -> None:
    """Write tensors (an iterable of (name, CPU tensor), consumed twice if a list) to one file."""
    tensors = list(tensors)
    header = {}
    off = 0
    for name, t in tensors:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"cannot store dtype {t.dtype} ({name})")
        n = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + n]}
        off += n
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    hb = json.dumps(header, separators=(",", ":")).encode()
    hb += b" " * ((8 - len(hb) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hb)))
        f.write(hb)
        for _, t in tensors:
            t = t.detach().contiguous().cpu()
            if t.numel():
                f.write(t.view(torch.uint8).numpy().tobytes() if t.dim() else
                        t.reshape(1).view(torch.uint8).numpy().tobytes())

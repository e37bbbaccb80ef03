"""Dependency-free safetensors reader / writer (mmap-backed, zero-copy into torch).

File layout: 8-byte little-endian header length, JSON header mapping tensor name →
``{dtype, shape, data_offsets}``, then the raw bytes.

Parity: ``cpp/common/safetensorsUtils.{h,cpp}`` and ``cpp/common/mmapReader.*`` in the
reference (a C++ mmap reader used by the runtime weight loader).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        if hlen > 100 * 1024 * 1024:
            raise ValueError(f"{path}: implausible safetensors header of {hlen} bytes")
        self.header: Dict[str, dict] = json.loads(self._f.read(hlen).decode("utf-8"))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._mm: Optional[mmap.mmap] = None

    def keys(self) -> List[str]:
        return list(self.header.keys())

    def info(self, name: str) -> Tuple[torch.dtype, List[int]]:
        e = self.header[name]
        return _DTYPES[e["dtype"]], list(e["shape"])

    def get(self, name: str) -> torch.Tensor:
        """A tensor viewing the mapped file (copy before the file object is dropped if it must
        outlive it; ``.to(device)`` copies anyway)."""
        e = self.header[name]
        if self._mm is None:
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        lo, hi = e["data_offsets"]
        dt = _DTYPES[e["dtype"]]
        if hi == lo:
            return torch.empty(e["shape"], dtype=dt)
        buf = memoryview(self._mm)[self._base + lo:self._base + hi]
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            t = torch.frombuffer(buf, dtype=torch.uint8)
        return t.view(dt).reshape(e["shape"])

    def close(self):
        if self._mm is not None:
            try:
                self._mm.close()
            except BufferError:
                pass       # tensors still view the mapping; the OS unmaps at exit
            self._mm = None
        self._f.close()


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
    header: Dict[str, dict] = {}
    if metadata:
        header["__metadata__"] = metadata
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""    # reshape first: 0-d tensors cannot be re-viewed
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hjson = json.dumps(header, separators=(",", ":")).encode("utf-8")
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for b in blobs:
            f.write(b)


class CheckpointReader:
    """All shards of a checkpoint directory behind one name → tensor lookup."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        idx = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx, "r", encoding="utf-8") as f:
                self._where = dict(json.load(f)["weight_map"])
        else:
            for fn in sorted(os.listdir(model_dir)):
                # side files (reduced vocabulary, processed LoRA) are not model shards
                if fn.endswith(".safetensors") and fn not in ("vocab_map.safetensors", "lora_weights.safetensors"):
                    for k in self._open(fn).keys():
                        self._where[k] = fn

    def _open(self, fn: str) -> SafetensorsFile:
        if fn not in self._files:
            self._files[fn] = SafetensorsFile(os.path.join(self.model_dir, fn))
        return self._files[fn]

    def keys(self) -> Iterable[str]:
        return self._where.keys()

    def __contains__(self, name: str) -> bool:
        return name in self._where

    def get(self, name: str) -> torch.Tensor:
        return self._open(self._where[name]).get(name)

    def close(self):
        for f in self._files.values():
            f.close()

"""Checkpoint I/O: a small safetensors reader/writer (mmap + JSON header) and the
name maps that turn HF Llama / Qwen3.5-style checkpoints into this framework's fused
weight layout.  HF checkpoints load unchanged, including tied embeddings and loading a
hybrid checkpoint's draft as a plain autoregressive LM (reference behaviour:
smcsd/core/worker.py:39-58, smcsd/model_executor/smc_model_runner.py:241-250).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
import warnings
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2,
}
_DTYPE_NAMES = {v: k for k, v in _DTYPES.items()}


class SafetensorsFile:
    """Zero-copy view of one ``.safetensors`` file."""

    def __init__(self, path: str):
        self.path = path
        self._f = open(path, "rb")
        (hlen,) = struct.unpack("<Q", self._f.read(8))
        self.header: Dict[str, dict] = json.loads(self._f.read(hlen))
        self.metadata = self.header.pop("__metadata__", {})
        self._base = 8 + hlen
        self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

    def keys(self) -> List[str]:
        return list(self.header.keys())

    def __contains__(self, name: str) -> bool:
        return name in self.header

    def get(self, name: str) -> torch.Tensor:
        info = self.header[name]
        dt = _DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        shape = info["shape"]
        n = 1
        for s in shape:
            n *= s
        if n == 0:
            return torch.empty(shape, dtype=dt)
        with warnings.catch_warnings():         # the mapping is read-only by design; callers copy out of it
            warnings.simplefilter("ignore", UserWarning)
            t = torch.frombuffer(self._mm, dtype=dt, count=n, offset=self._base + b)
        return t.view(shape)

    def close(self) -> None:
        try:
            self._mm.close()
        finally:
            self._f.close()


def save_safetensors(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[dict] = None) -> None:
    header: Dict[str, dict] = {}
    off = 0
    blobs = []
    for name, t in tensors.items():
        t = t.detach().contiguous().cpu()
        raw = t.view(torch.uint8).reshape(-1).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _DTYPE_NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    if metadata:
        header["__metadata__"] = {k: str(v) for k, v in metadata.items()}
    hjson = json.dumps(header, separators=(",", ":")).encode()
    hjson += b" " * ((8 - len(hjson) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hjson)))
        f.write(hjson)
        for b in blobs:
            f.write(b)


class Checkpoint:
    """All tensors of a HF model directory (single file or sharded with an index)."""

    def __init__(self, path: str):
        self.path = path
        self.files: Dict[str, SafetensorsFile] = {}
        self.where: Dict[str, str] = {}
        idx = os.path.join(path, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                wm = json.load(f)["weight_map"]
            for name, fn in wm.items():
                self.where[name] = fn
        else:
            names = sorted(fn for fn in os.listdir(path) if fn.endswith(".safetensors"))
            if not names:
                raise FileNotFoundError(f"no .safetensors file under {path}")
            for fn in names:
                for name in self._open(fn).keys():
                    self.where[name] = fn

    def _open(self, fn: str) -> SafetensorsFile:
        if fn not in self.files:
            self.files[fn] = SafetensorsFile(os.path.join(self.path, fn))
        return self.files[fn]

    def __contains__(self, name: str) -> bool:
        return name in self.where

    def keys(self) -> Iterable[str]:
        return self.where.keys()

    def get(self, name: str) -> torch.Tensor:
        return self._open(self.where[name]).get(name)

    def first(self, *names: str) -> Tuple[str, torch.Tensor]:
        for n in names:
            if n in self.where:
                return n, self.get(n)
        raise KeyError(f"none of {names} in checkpoint {self.path}")

    def close(self) -> None:
        for f in self.files.values():
            f.close()


def strip_prefixes(ck: Checkpoint) -> str:
    """HF text models nest under ``model.`` or ``model.language_model.``; find which."""
    for pre in ("model.language_model.", "language_model.model.", "model.", ""):
        if f"{pre}embed_tokens.weight" in ck:
            return pre
    raise KeyError("cannot find embed_tokens.weight in checkpoint")


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[0] // world
    return t[rank * n:(rank + 1) * n]


def shard_cols(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = t.shape[1] // world
    return t[:, rank * n:(rank + 1) * n]

"""Helpers for the golden fixtures: tensor <-> .npz (bf16 travels as its uint16 bit
pattern), a platform-independent input pattern so inputs need not be stored, and a
content digest for outputs that must match bit for bit."""
from __future__ import annotations

import hashlib
from pathlib import Path

import numpy as np
import torch

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"

_TAGS = {torch.bfloat16: "bf16", torch.float16: "f16", torch.float32: "f32", torch.float64: "f64",
         torch.int64: "i64", torch.int32: "i32", torch.bool: "b1"}
_BY_TAG = {v: k for k, v in _TAGS.items()}


def save(name: str, tensors: dict, meta: dict | None = None) -> Path:
    arrays = {}
    for key, t in tensors.items():
        t = t.detach().cpu().contiguous()
        tag = _TAGS[t.dtype]
        arr = t.view(torch.int16).numpy() if t.dtype == torch.bfloat16 else t.numpy()
        arrays[f"{key}::{tag}"] = arr
    if meta:
        for k, v in meta.items():
            arrays[f"meta::{k}"] = np.array(v)
    path = GOLDEN_DIR / f"{name}.npz"
    np.savez_compressed(path, **arrays)
    return path


def load(name: str):
    """Returns (tensors, meta)."""
    data = np.load(GOLDEN_DIR / f"{name}.npz", allow_pickle=False)
    tensors, meta = {}, {}
    for key in data.files:
        if key.startswith("meta::"):
            v = data[key]
            meta[key[6:]] = v.item() if v.shape == () else v
            continue
        name_, tag = key.rsplit("::", 1)
        arr = data[key]
        if tag == "bf16":
            tensors[name_] = torch.from_numpy(arr.copy()).view(torch.bfloat16)
        else:
            tensors[name_] = torch.from_numpy(arr.copy()).to(_BY_TAG[tag])
    return tensors, meta


def pattern(shape, dtype: torch.dtype, seed: int, scale: float = 1.0) -> torch.Tensor:
    """Deterministic pseudo-random tensor from 64-bit integer arithmetic only (the same on
    every machine and torch version): values k/8192 with k in [-16384, 16384), times scale,
    rounded once to ``dtype``."""
    n = 1
    for d in shape:
        n *= int(d)
    idx = np.arange(n, dtype=np.uint64)
    with np.errstate(over="ignore"):
        h = idx * np.uint64(6364136223846793005) + np.uint64((seed * 1442695040888963407 + 1013904223) % (1 << 64))
        h ^= h >> np.uint64(29)
        h *= np.uint64(0xBF58476D1CE4E5B9)
        h ^= h >> np.uint64(32)
    k = (h & np.uint64(0x7FFF)).astype(np.int64) - 16384
    vals = torch.from_numpy(k.astype(np.float32) / 8192.0) * scale
    return vals.reshape(*shape).to(dtype)


def digest(t: torch.Tensor) -> str:
    """sha256 of the tensor's bytes in row-major order."""
    t = t.detach().cpu().contiguous()
    raw = t.view(torch.uint8) if t.dtype != torch.bool else t.to(torch.uint8)
    return hashlib.sha256(raw.numpy().tobytes()).hexdigest()

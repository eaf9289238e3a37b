"""safetensors in and out: a small writer (for synthetic checkpoints) and a reader over the native
mmap reader that hands out torch tensors without copying the file."""
from __future__ import annotations

import json
import os
import struct
import warnings
from typing import Dict

import numpy as np
import torch

_DT = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16", torch.int32: "I32", torch.int64: "I64",
       torch.int8: "I8", torch.uint8: "U8", torch.bool: "BOOL"}
_RDT = {v: k for k, v in _DT.items()}


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Dict[str, str] = None):
    header, off, blobs = {}, 0, []
    if metadata:
        header["__metadata__"] = metadata
    for name, t in tensors.items():
        t = t.detach().cpu().contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[name] = {"dtype": _DT[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        off += len(raw)
        blobs.append(raw)
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


class SafetensorsSet:
    """All shards of a snapshot; the index (``model.safetensors.index.json``) is the manifest when present."""

    def __init__(self, snapshot: str):
        from ..native import host as H
        self.dir = snapshot
        idx = os.path.join(snapshot, "model.safetensors.index.json")
        if os.path.exists(idx):
            with open(idx) as f:
                wm = json.load(f)["weight_map"]
            shards = sorted(set(wm.values()))
        else:
            shards = sorted(f for f in os.listdir(snapshot) if f.endswith(".safetensors"))
            wm = None
        if not shards:
            raise FileNotFoundError(f"no safetensors files in {snapshot}")
        self.files = {s: H.SafetensorsFile(os.path.join(snapshot, s)) for s in shards}
        self.where = {}
        for s, f in self.files.items():
            for n in f.names():
                self.where[n] = s
        if wm is not None:
            missing = [n for n, s in wm.items() if self.where.get(n) != s]
            if missing:
                raise ValueError(f"index names tensors that their shard does not hold: {missing[:3]} ...")

    def names(self):
        return list(self.where)

    def has(self, name: str) -> bool:
        return name in self.where

    def shape(self, name: str):
        return list(self.files[self.where[name]].shape(name))

    def dtype(self, name: str) -> str:
        return self.files[self.where[name]].dtype(name)

    def get(self, name: str, copy: bool = True) -> torch.Tensor:
        """The tensor as a CPU tensor.  ``copy=False`` returns a view of the mapped file, valid only while
        this object lives and read-only: move it to a device (or clone it) before the set is dropped."""
        f = self.files[self.where[name]]
        dt = _RDT[f.dtype(name)]
        shape = f.shape(name)
        mv = f.view(name)
        if len(mv) == 0:
            return torch.empty(shape, dtype=dt)
        arr = np.frombuffer(mv, dtype=np.uint8)
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")     # the mapping is read-only by design
            t = torch.from_numpy(arr).view(dt).reshape(shape)
        return t.clone() if copy else t

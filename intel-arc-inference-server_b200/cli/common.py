"""Shared start-up steps of the CLI programs: hardware gate, model loading, planning."""
from __future__ import annotations

import os
import sys

import torch

from ..models.config import PRESETS, preset
from ..models.weights import random_weights


def hardware_gate(min_devices: int = 1, out=sys.stderr):
    """Refuses to start on anything but Blackwell B200-class GPUs (compute capability 10.x) -- the
    reference checks vendor / device id / peer access before it reads a file (src/cli/hardware_check.h:53-88)."""
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this server runs on NVIDIA B200 (sm_100a) only")
    n = torch.cuda.device_count()
    if n < min_devices:
        raise SystemExit(f"{min_devices} GPUs are needed for this placement, {n} are visible")
    for i in range(min_devices):
        p = torch.cuda.get_device_properties(i)
        if p.major != 10:
            raise SystemExit(f"GPU {i} is {p.name} (sm_{p.major}{p.minor}); the kernels are built for sm_100a only")
        out.write(f"hardware: GPU {i} {p.name}, {p.total_memory / 2**30:.0f} GiB, {p.multi_processor_count} SMs\n")
    if min_devices > 1:
        for i in range(min_devices):
            for j in range(min_devices):
                if i != j and not torch.cuda.can_device_access_peer(i, j):
                    raise SystemExit(f"GPU {i} cannot access GPU {j} peer to peer")


def load_model(spec: str, device, seed: int = 0, int8_head: bool = False, tp=(0, 1)):
    """A preset name gives random-init weights in that shape; anything else is a snapshot."""
    if spec in PRESETS:
        cfg = preset(spec)
        sys.stderr.write(f"load: preset {spec} with random-init W4A16 weights (seed {seed})\n")
        return random_weights(cfg, device=device, seed=seed)
    from ..loader.loader import load
    return load(spec, device=device, int8_head=int8_head, tp=tp)


def find_tokenizer(spec: str):
    from ..server.iface import ByteTok, NativeTok
    if spec and os.path.isdir(spec) and os.path.exists(os.path.join(spec, "tokenizer.json")):
        return NativeTok(os.path.join(spec, "tokenizer.json"))
    sys.stderr.write("tokenizer: no tokenizer.json beside the model; serving with the byte-level stand-in\n")
    return ByteTok()

"""Snapshot resolution: a directory, or a Hugging Face repo id looked up in the local hub cache.

Never downloads (the reference's rule, src/loader/snapshot.cc:20, docs/13-loader.md:66-79):
``org/name`` resolves to ``$HF_HOME/hub/models--org--name/snapshots/<refs/main>``.
"""
from __future__ import annotations

import os


def resolve_snapshot(spec: str) -> str:
    if os.path.isdir(spec):
        return os.path.abspath(spec)
    if spec.count("/") == 1 and not spec.startswith((".", "/")):
        home = os.environ.get("HF_HOME", os.path.join(os.path.expanduser("~"), ".cache", "huggingface"))
        base = os.path.join(home, "hub", "models--" + spec.replace("/", "--"))
        ref = os.path.join(base, "refs", "main")
        if os.path.exists(ref):
            with open(ref) as f:
                snap = os.path.join(base, "snapshots", f.read().strip())
            if os.path.isdir(snap):
                return snap
        raise FileNotFoundError(f"{spec} is not in the local hub cache ({base}); this server never downloads")
    raise FileNotFoundError(f"no such snapshot directory: {spec}")

"""Builds the native host library in-tree: ``native/b200host.<abi>.so`` (pybind11 + g++).

The host library carries the request-path components that are native in the
reference as well: KV page pool, prefix cache, prompt lookup, speculative
control, tool-call parsers, tokenizer, scheduler, HTTP server, safetensors reader.
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "src")
EXT = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
LIB = os.path.join(HERE, "b200host" + EXT)
STAMP = os.path.join(HERE, "build", "digest.txt")
FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-pthread", "-Wall", "-Wno-sign-compare"]


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(SRC)):
        with open(os.path.join(SRC, f), "rb") as fh:
            h.update(f.encode()); h.update(fh.read())
    h.update(" ".join(FLAGS).encode()); h.update(EXT.encode())
    return h.hexdigest()


def is_current() -> bool:
    return os.path.exists(LIB) and os.path.exists(STAMP) and open(STAMP).read().strip() == _digest()


def build(force: bool = False) -> str:
    if not force and is_current():
        return LIB
    import pybind11
    inc = [f"-I{pybind11.get_include()}", f"-I{sysconfig.get_paths()['include']}", f"-I{SRC}"]
    srcs = [os.path.join(SRC, f) for f in sorted(os.listdir(SRC)) if f.endswith(".cc")]
    cmd = [os.environ.get("CXX", "g++"), *FLAGS, *inc, *srcs, "-o", LIB]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host library build failed:\n{r.stdout}\n{r.stderr}")
    os.makedirs(os.path.dirname(STAMP), exist_ok=True)
    with open(STAMP, "w") as fh:
        fh.write(_digest())
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))

"""Flag system: one annotated dataclass per program; the parser and ``--help`` are generated from it.

The reference derives its parsers from a struct by static reflection (src/cli/flags.h:1-146,
src/cli/b70_serve.cc:83-147); here ``dataclasses.fields`` plays that role.  A field's metadata
carries its help text and choices; ``positional`` marks the snapshot argument.
"""
from __future__ import annotations

import argparse
import dataclasses
from dataclasses import dataclass, field
from typing import Optional


def flag(default, help: str, choices=None, positional: bool = False):
    return field(default=default, metadata={"help": help, "choices": choices, "positional": positional})


def build_parser(cls, prog: str, description: str) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog=prog, description=description)
    for f in dataclasses.fields(cls):
        md = f.metadata
        name = f.name.replace("_", "-")
        if md.get("positional"):
            p.add_argument(f.name, nargs="?" if f.default is not None or f.default is None else None,
                           default=f.default, help=md["help"])
        elif f.type in (bool, "bool"):
            p.add_argument(f"--{name}", action="store_true", default=f.default, help=md["help"])
        else:
            kw = {"default": f.default, "help": md["help"] + f" (default: {f.default})"}
            if md.get("choices"):
                kw["choices"] = md["choices"]
            if isinstance(f.default, int) and not isinstance(f.default, bool):
                kw["type"] = int
            elif isinstance(f.default, float):
                kw["type"] = float
            p.add_argument(f"--{name}", **kw)
    return p


def parse(cls, argv, prog: str, description: str):
    ns = build_parser(cls, prog, description).parse_args(argv)
    return cls(**{f.name: getattr(ns, f.name) for f in dataclasses.fields(cls)})


@dataclass
class ServeFlags:
    """Flags of ``b200-serve`` (the reference's b70-serve surface, src/cli/b70_serve.cc:83-147)."""
    model: Optional[str] = flag(None, "snapshot directory, Hugging Face repo id, or a preset name "
                                      "(tiny-dense, small-dense, dense-27b, moe-35b-a3b) with random weights",
                                positional=True)
    spec: str = flag("auto", "speculative decoding", ["auto", "off", "mtp", "dflash", "lookup", "dflash-lookup"])
    spec_max: int = flag(3, "most drafts per step")
    draft_model: Optional[str] = flag(None, "drafter snapshot for --spec dflash")
    max_num_seqs: int = flag(4, "sequence slots (concurrent requests)")
    max_len: str = flag("auto", "context length, or auto for what fits")
    parallel: str = flag("auto", "device placement", ["auto", "1", "tp", "tp2", "tp4", "tp8", "ep", "ep2", "ep4",
                                                      "ep8", "replica", "pp", "pp2", "pp4", "pp8"])
    pipeline_split: str = flag("auto", "first layer of the second pipeline stage, or auto")
    host: str = flag("127.0.0.1", "listen address")
    port: int = flag(8000, "listen port")
    log_requests: Optional[str] = flag(None, "directory for one JSON file per request")
    prefix_cache_gb: str = flag("auto", "host prefix store size in GiB, auto, or 0 to turn it off")
    prefix_split_last: bool = flag(False, "keep the prompt's last position out of the cached prefix")
    kv_cache: str = flag("bf16", "KV cache element type", ["bf16", "int8"])
    prefill_backend: str = flag("auto", "prompt-pass GEMM path",
                                ["auto", "w4", "bf16", "bf16-resident", "int8", "l0", "l0-int8", "rows"])
    int8_head: bool = flag(False, "quantise lm_head to int8 with per-row scales")
    draft_vocab: int = flag(0, "reduced draft vocabulary size (0: full)")
    draft_vocab_ids: Optional[str] = flag(None, "file with the ranked ids of the draft vocabulary")
    candidate_head_int8: bool = flag(False, "block drafter: int8 copy of the draft-vocabulary head (half its bytes), candidates re-scored "
                                            "exactly; from 3 rows up the bf16 head is the faster one (it runs on the tensor cores)")
    tool_format: str = flag("qwen_xml", "tool-call syntax of the model", ["qwen_xml", "hermes"])
    seed: int = flag(0, "seed of random-init weights (preset models)")


@dataclass
class DecodeFlags:
    """Flags of ``b200-decode`` (the reference's b70-decode, src/cli/b70_decode.cc:104-149)."""
    model: Optional[str] = flag(None, "snapshot directory or preset name", positional=True)
    ids: Optional[str] = flag(None, "comma-separated prompt token ids, or @file")
    n: int = flag(32, "tokens to generate")
    prefill: bool = flag(False, "ingest the prompt with the chunked prompt pass instead of row steps")
    bench: bool = flag(False, "print a markdown row: t/s, ms/token, bytes/token, bandwidth utilisation")
    depth: int = flag(4096, "--bench / --profile: context depth the steps run at")
    tg: int = flag(128, "--bench: decode tokens timed")
    prefill_length: int = flag(0, "--bench: also time a prompt pass of this many tokens")
    prefill_chunk: int = flag(4096, "prompt chunk size")
    profile: bool = flag(False, "per-kernel device times of one decode step (CUDA events around every launch)")
    steps: int = flag(8, "--profile: steps averaged")
    repeats: int = flag(3, "--profile / --bench: repetitions, the median is reported")
    kv_cache: str = flag("bf16", "KV cache element type", ["bf16", "int8"])
    prefill_backend: str = flag("auto", "prompt-pass GEMM path", ["auto", "w4", "bf16", "bf16-resident", "int8", "rows"])
    int8_head: bool = flag(False, "int8 lm_head")
    seed: int = flag(0, "seed of random-init weights (preset models)")

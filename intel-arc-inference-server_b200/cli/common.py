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
    try:    # memory, BAR1 and NVLink report (read-only NVML queries); a warning, never a refusal
        from ..utils import vram
        gpus = vram.probe(indices=list(range(min_devices)))
        for line in vram.describe(gpus):
            out.write(line + "\n")
        for problem in vram.check_placement(gpus, need_nvlink=min_devices > 1):
            out.write(f"warning: {problem}: the fused collective kernels will run over PCIe\n")
    except Exception as e:  # noqa: BLE001   (no NVML in the container)
        out.write(f"memory: NVML probe unavailable ({type(e).__name__})\n")


def peek_config(spec: str):
    """The model's shape without loading a weight: a preset, or ``config.json`` of the snapshot."""
    if spec in PRESETS:
        return preset(spec)
    import json
    from ..loader.snapshot import resolve_snapshot
    from ..models.config import ModelConfig
    with open(os.path.join(resolve_snapshot(spec), "config.json")) as f:
        hf = json.load(f)
    if "text_config" in hf:
        hf = hf["text_config"]
    return ModelConfig.from_hf_config(hf)


def chat_format_for(spec: str):
    """The chat format of a snapshot, from ``config.json``'s ``model_type`` (None for presets and for every model
    type that reads as the default format, which then follows ``--tool-format``)."""
    if spec in PRESETS:
        return None
    import json
    from ..loader.snapshot import resolve_snapshot
    from ..server.chat_format import ChatFormat
    try:
        with open(os.path.join(resolve_snapshot(spec), "config.json")) as f:
            hf = json.load(f)
    except OSError:
        return None
    fmt = ChatFormat.for_model_type(hf.get("model_type") or hf.get("text_config", {}).get("model_type"))
    return fmt if fmt.kind != "qwen" else None


def parallel_auto(cfg, n_gpus: int, mem_bytes: int, max_seqs: int = 1, kv_dtype: str = "bf16", int8_head: bool = False,
                  min_len: int = 8192) -> str:
    """What ``--parallel auto`` means: one GPU when the model and ``min_len`` positions per sequence fit on it (a
    copy per GPU is opt-in: ``replica``); else the fewest GPUs that hold it -- tensor parallel 2 / 4 / 8 for dense
    models, expert parallel for mixture-of-experts models whose experts are what does not fit.  The reference
    chooses between one card, ``tp`` and ``pp`` the same way, from its planner's numbers
    (src/cli/b70_serve.cc:1310-1324, cli::parallel_auto)."""
    from ..runtime.memory_plan import plan

    def fits(tp=1, ep=1):
        try:
            plan(cfg, max_seqs, min_len, kv_dtype, int8_head, "bf16", tp=tp, ep=ep, budget=mem_bytes)
            return True
        except ValueError:
            return False
    if fits():
        return "1"
    for n in (2, 4, 8):
        if n > n_gpus:
            break
        heads_ok = cfg.n_kv_heads % n == 0 and cfg.n_q_heads % n == 0 and not cfg.n_gdn_layers
        if cfg.is_moe and cfg.n_experts % n == 0 and fits(ep=n):
            return f"ep{n}"
        if not cfg.is_moe and heads_ok and fits(tp=n):
            return f"tp{n}"
    raise SystemExit(f"{cfg.name} does not fit on {n_gpus} GPU(s) of {mem_bytes / 2**30:.0f} GiB in any placement")


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


def build_rank_engine(f, par: str) -> int:
    """One rank of ``serve --parallel ...`` (started by the torch launcher): builds this rank's engine, then
    rank 0 serves HTTP through a leader / router and the other ranks follow its commands."""
    import datetime
    import signal
    import torch
    import torch.distributed as dist
    from ..parallel import launch as L
    from ..parallel import tp as TP
    from ..runtime.engine import Engine
    from ..server.adapter import EngineAdapter
    rank, world, local = TP.init_dist()
    ctl = dist.new_group(backend="gloo", timeout=datetime.timedelta(days=7))     # control plane: host objects only
    plane = L.ControlPlane(ctl)
    kind, deg = L.parse_parallel(par)
    spec = "off"
    dev = torch.device("cuda", local)
    max_len = 4096 if f.max_len == "auto" else int(f.max_len)
    kw = dict(max_seqs=f.max_num_seqs, max_len=max_len, kv_dtype=f.kv_cache, int8_head=f.int8_head)
    if kind == "replica":
        engine = Engine(load_model(f.model, dev, f.seed, f.int8_head), **kw)
    elif kind == "tp":
        import dataclasses
        want_mtp = f.spec == "mtp"
        if f.spec not in ("auto", "off", "mtp", "dflash"):
            raise SystemExit("--parallel tpN serves with --spec mtp, --spec dflash or without a draft head")
        if f.model in PRESETS:
            cfg = preset(f.model)
            w = TP.random_shard(dataclasses.replace(cfg, mtp_layers=1) if want_mtp else cfg, rank, world, dev, f.seed)
        else:
            w = load_model(f.model, dev, f.seed, f.int8_head, tp=(rank, world))
        if f.spec in ("auto", "mtp") and w.mtp is not None:
            spec = "mtp"
            kw["extra_kv_layers"] = len(w.mtp.layers)
        elif want_mtp:
            raise SystemExit("--spec mtp needs a checkpoint with an MTP head")
        elif f.spec == "dflash":
            spec = "dflash"
            kw["extra_kv_layers"] = 2
        engine = TP.make_engine(w, mode="fused", **kw)
    elif kind == "pp":
        from ..parallel import pp as PP
        cfg = preset(f.model) if f.model in PRESETS else None
        if cfg is None:
            full = load_model(f.model, dev, f.seed, f.int8_head)
            a, b = PP.split_layers(full.cfg.n_layers, world)[rank]
            w = PP.stage_weights(full, a, b)
        else:
            a, b = PP.split_layers(cfg.n_layers, world)[rank]
            w = PP.random_stage(cfg, a, b, dev, f.seed)
        engine = PP.PipelineEngine(w, rank, world, **kw)
    else:
        raise SystemExit("--parallel ep serves through the expert-parallel prompt pass only: use tpN, ppN or replica")
    adapter = EngineAdapter(engine, eos_ids=(2,))
    if spec != "off":       # every rank carries its slice of the draft head and drafts in lockstep
        from ..runtime.spec import SpecAdapter
        adapter = SpecAdapter(adapter, spec, f.spec_max, f.draft_model)
    if rank != 0:
        n = L.serve_replica_worker(adapter, plane) if kind == "replica" else L.follow_lockstep(adapter, plane)
        sys.stderr.write(f"rank {rank}: {n} commands\n")
        return 0
    from ..server.app import Server, ServerOptions
    from ..server.chat_template import ChatTemplate
    front = L.ReplicaRouter(adapter, plane) if kind == "replica" else L.lockstep_leader(adapter, plane)
    tok = find_tokenizer(f.model)
    template = ChatTemplate.from_snapshot(f.model) if f.model not in PRESETS else ChatTemplate()
    opts = ServerOptions(model_name=engine.cfg.name, log_requests=f.log_requests, spec=spec,
                         spec_max=f.spec_max if spec != "off" else 0,
                         tool_format=f.tool_format, prefix_split_last=f.prefix_split_last,
                         chat_format=chat_format_for(f.model))
    srv = Server(front, tok, template, opts, host=f.host, port=f.port)
    sys.stderr.write(f"serving {engine.cfg.name} ({par}, {world} GPUs) on http://{f.host}:{srv.port}/v1\n")
    signal.signal(signal.SIGINT, lambda *_: setattr(srv, "_stop", True))
    signal.signal(signal.SIGTERM, lambda *_: setattr(srv, "_stop", True))
    try:
        srv.serve_forever()
    finally:
        srv.http.stop()
        front.shutdown()
    return 0

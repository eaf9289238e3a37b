"""Small decode workload for kernel profiling: a few layers of a named shape at a given depth.

    python -m b200serve.utils.profile_decode --model dense-27b --layers 4 --depth 4096 --steps 3
    python -m b200serve.utils.profile_decode --model dense-27b --layers 2 --depth 1024 --steps 2 --rows 16 --spec dflash

The KV cache is filled with random values up to ``depth`` (no prompt pass), so a
capture sees only the decode-step kernels.  Runs eagerly (no CUDA graph) so every
launch appears under its own name in a launch list.  ``--spec mtp|dflash``: the steps are
draft-and-verify iterations of a random-init head (``--rows`` - 1 drafts, one verify step of
``--rows`` rows) after a real prompt pass of ``depth`` tokens, which the head ingests.
"""
from __future__ import annotations

import argparse
from dataclasses import replace

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="dense-27b")
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--depth", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--kv-cache", default="bf16")
    ap.add_argument("--graphs", action="store_true")
    ap.add_argument("--nsplit", type=int, default=0, help="KV splits of the decode attention (0: chosen from the KV heads and the depth)")
    ap.add_argument("--time", action="store_true", help="print CUDA-event ms per step")
    ap.add_argument("--spec", default="", help="mtp | dflash: steps are draft-and-verify iterations (drafts of --rows - 1 tokens "
                                                "from a random-init head, one verify step of --rows rows, none accepted)")
    args = ap.parse_args()
    from ..models.config import preset
    from ..models.weights import random_weights
    from ..runtime.engine import Engine, Row
    from ..ops import lib as K
    cfg = replace(preset(args.model), n_layers=args.layers)
    if args.spec:
        return spec_iterations(args, replace(cfg, mtp_layers=1))
    w = random_weights(cfg, device="cuda", seed=0, exact=False)
    eng = Engine(w, max_seqs=1, max_len=args.depth + 256, kv_dtype=args.kv_cache, use_graphs=args.graphs,
                 nsplit_attn=args.nsplit)
    if args.kv_cache == "bf16":
        eng.kv.k.normal_(0, 0.5); eng.kv.v.normal_(0, 0.5)
    eng._ensure_pages(0, args.depth)
    eng.seq_len[0] = args.depth
    m = args.rows
    def step():
        p = eng.seq_len[0]
        return eng.forward_rows([Row(0, p + i, 17 + i) for i in range(m)], advance=False, read=False)
    for _ in range(2):
        step(); eng.truncate(0, args.depth)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step(); eng.truncate(0, args.depth)
    e1.record()
    torch.cuda.synchronize()
    K.check_status()
    if args.time:
        print(f"ms_per_step {e0.elapsed_time(e1) / args.steps:.4f} layers {args.layers} rows {m}")


def spec_iterations(args, cfg):
    """Draft-and-verify iterations of a learned head over the few-layer trunk: a short prompt pass first (the head
    ingests it), then ``--steps`` iterations; eager, so every launch of the draft pass, the candidate kernels and the
    verify step shows under its own name."""
    from ..models.weights import random_weights
    from ..ops import lib as K
    from ..runtime.engine import Engine
    from ..runtime.spec import SpecAdapter
    from ..server.adapter import EngineAdapter
    k = max(1, args.rows - 1)
    w = random_weights(cfg, device="cuda", seed=0, exact=False)
    eng = Engine(w, max_seqs=1, max_len=args.depth + 64 * (args.steps + 4), use_graphs=args.graphs, extra_kv_layers=2)
    ad = SpecAdapter(EngineAdapter(eng), args.spec, k)
    g = torch.Generator().manual_seed(0)
    pending = ad.prefill(0, torch.randint(0, cfg.vocab - 1, (args.depth,), generator=g).tolist())

    def iteration(pending):
        drafts = ad.draft(0, pending, k)
        res = ad.step({0: [pending] + drafts})[0]
        ad.truncate(0, ad.length(0) - len(drafts))
        return res[0]
    for _ in range(2):
        pending = iteration(pending)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        pending = iteration(pending)
    e1.record()
    torch.cuda.synchronize()
    K.check_status()
    if args.time:
        print(f"ms_per_iteration {e0.elapsed_time(e1) / args.steps:.4f} layers {args.layers} spec {args.spec} drafts {k}")


if __name__ == "__main__":
    main()

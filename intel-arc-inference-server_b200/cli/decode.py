"""``b200-decode``: token ids in, token ids out; benchmark and profile modes.

    python -m b200serve.cli.decode <snapshot-or-preset> --ids 1,2,3 --n 32 [--prefill]
    python -m b200serve.cli.decode dense-27b --bench --depth 4096 --tg 128 [--prefill-length 4096]
    python -m b200serve.cli.decode dense-27b --profile --depth 4096 --steps 8

stdout carries only ids or markdown rows; everything else goes to stderr (the reference's rule,
src/cli/stdout_to_stderr.h).  ``--bench`` prints tokens/s, ms/token and the fraction of the measured
HBM bandwidth the step's bytes correspond to (the reference's MBU column, b70_decode.cc:82-90);
``--profile`` times every kernel of a decode step with CUDA events in a separate, instrumented,
eager walk -- never the graph that ``--bench`` times (capture.h:21-50).
"""
from __future__ import annotations

import statistics
import sys

from .flags import DecodeFlags, parse


def _ids(arg):
    if arg.startswith("@"):
        with open(arg[1:]) as f:
            arg = f.read()
    return [int(x) for x in arg.replace("\n", ",").split(",") if x.strip()]


def main(argv=None):
    f = parse(DecodeFlags, argv, "b200-decode", __doc__)
    if not f.model:
        raise SystemExit("give a snapshot directory or a preset name")
    import torch
    from ..ops import lib as K
    from ..runtime.engine import Engine, Row
    from ..utils.bench_kernels import peaks
    from . import common
    common.hardware_gate(1)
    torch.cuda.set_device(0)
    w = common.load_model(f.model, "cuda", f.seed, f.int8_head)
    cfg = w.cfg
    depth = f.depth if (f.bench or f.profile) else 0
    ids = _ids(f.ids) if f.ids else None
    need = max(depth, len(ids or []), f.prefill_length) + (f.tg + 4) * max(1, f.repeats if cfg.n_gdn_layers else 1) + f.n + 64
    eng = Engine(w, max_seqs=1, max_len=need, kv_dtype=f.kv_cache, int8_head=f.int8_head,
                 prefill_backend=f.prefill_backend if f.prefill or f.bench else "rows")
    if ids is not None and not (f.bench or f.profile):
        out = eng.generate(ids, f.n)
        K.check_status()
        print(",".join(str(t) for t in out))
        return
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (max(depth, 16),), generator=g).tolist()
    first = eng.prefill(0, prompt)
    if f.profile:
        return _profile(eng, f, first)
    hbm, _, src = peaks()
    rows = []
    for _ in range(f.repeats):
        if not cfg.n_gdn_layers:    # (a recurrent state is not rewound: a hybrid model's repeats continue the sequence)
            eng.truncate(0, len(prompt))
        eng.decode_begin([0], [first])
        for _ in range(4):
            eng.decode_step(read=False)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(f.tg):
            eng.decode_step(read=False)
        e1.record()
        torch.cuda.synchronize()
        rows.append(e0.elapsed_time(e1) / f.tg)
    K.check_status()
    ms = statistics.median(rows)
    nbytes = cfg.weight_bytes_per_token(1.0 if f.int8_head else 2.0) + cfg.kv_bytes_per_token(f.kv_cache) * depth
    print("| model | depth | tg | ms/token | t/s | GB/token | bandwidth | of HBM copy (" + src + ") |")
    print("|---|---|---|---|---|---|---|---|")
    print(f"| {cfg.name} | {depth} | {f.tg} | {ms:.3f} | {1e3 / ms:.1f} | {nbytes / 1e9:.2f} | "
          f"{nbytes / ms / 1e6:.0f} GB/s | {nbytes / ms / 1e6 / hbm:.2f} |")
    if f.prefill_length:
        pids = torch.randint(0, cfg.vocab, (f.prefill_length,), generator=g).tolist()
        ts = []
        for _ in range(f.repeats + 1):
            eng.reset(0)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.prefill(0, pids, chunk=f.prefill_chunk)
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        pm = statistics.median(ts[1:])
        print(f"| {cfg.name} | prefill {f.prefill_length} | chunk {f.prefill_chunk} | {pm:.1f} ms | "
              f"{f.prefill_length / pm * 1e3:.0f} t/s | | | |")


def _profile(eng, f, first):
    """Per-kernel device time of a decode step: every launch bracketed by CUDA events (eager walk)."""
    import collections
    import torch
    from ..ops import lib as K
    from ..runtime.engine import Row
    times = collections.OrderedDict()
    raw = {}
    names = [n for n in dir(K) if callable(getattr(K, n)) and n in (
        "gemv_w4", "resid_norm", "rope_append", "attn_decode", "head_gemv", "argmax_finish")]
    pending = []

    def wrap(name, fn):
        def inner(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*a, **kw)
            e1.record()
            pending.append((name, e0, e1))
            return r
        return inner
    for n in names:
        raw[n] = getattr(K, n)
        setattr(K, n, wrap(n, raw[n]))
    try:
        eng.use_graphs = False
        pos, tok = eng.seq_len[0], first
        for step in range(f.steps + 1):
            pending.clear()
            tok = eng.forward_rows([Row(0, pos, tok)], advance=False, read=True)[0]
            pos += 1
            torch.cuda.synchronize()
            if step == 0:
                continue
            for name, e0, e1 in pending:
                times.setdefault(name, []).append(e0.elapsed_time(e1) * 1e3)
    finally:
        for n in names:
            setattr(K, n, raw[n])
    print("| kernel family | launches/step | us/step (mean) | share |")
    print("|---|---|---|---|")
    tot = sum(sum(v) for v in times.values()) / f.steps
    for name, v in times.items():
        per = sum(v) / f.steps
        print(f"| {name} | {len(v) // f.steps} | {per:.1f} | {per / tot:.1%} |")
    print(f"| total (events, eager: includes launch gaps) | | {tot:.1f} | |")


if __name__ == "__main__":
    main()

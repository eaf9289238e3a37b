"""Timed regions of ``bench.py``: decode steps and prefill passes through the public Engine API.

The same measurement style as the reference's ``b70-decode --bench``
(src/cli/b70_decode.cc:82-90,131-140): ingest a prompt to the wanted depth, then
time plain decode steps; prefill is timed as whole prompt passes.
"""
from __future__ import annotations

import torch

from ..models.config import preset
from ..models.weights import random_weights
from ..ops import lib as K
from ..runtime.engine import Engine, Row


def _events():
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def run_decode_bench(args, barrier) -> dict:
    cfg = preset(args.model)
    dev = torch.device("cuda", torch.cuda.current_device())
    weights = random_weights(cfg, device=dev, seed=0, exact=False)
    total = args.depth + (max(1, getattr(args, "windows", 5)) + 4) * (args.steps + args.warmup) + 64
    eng = Engine(weights, max_seqs=1, max_len=total, kv_dtype=args.kv_cache, int8_head=args.int8_head,
                 prefill_backend=args.prefill_backend)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab, (args.depth,), generator=g).tolist()
    first = eng.prefill(0, ids)
    # ---- device-timed: graph replays, tokens and positions advance on the device.  ``windows`` timed regions of
    # ``steps`` steps each; the reported time per step is the median window (one hiccup cannot move it)
    windows = max(1, getattr(args, "windows", 5))
    eng.decode_begin([0], [first])
    for _ in range(args.warmup):
        eng.decode_step(read=False)
    win_ms = []
    for _ in range(windows):
        barrier()
        e0, e1 = _events()
        e0.record()
        for _ in range(args.steps):
            eng.decode_step(read=False)
        e1.record()
        barrier()
        win_ms.append(e0.elapsed_time(e1) / args.steps)
    ms = sorted(win_ms)[len(win_ms) // 2]
    launches = eng.launches(1, True) * args.steps
    # ---- end to end: every step the host sends the row (pinned H2D) and reads the token back (D2H)
    tok = eng._read_out(1)[0]
    pos = eng.seq_len[0]
    for _ in range(args.warmup):
        tok = eng.forward_rows([Row(0, pos, tok)], advance=False, read=True)[0]
        pos += 1
    e2e_win = []
    for _ in range(min(3, windows)):
        barrier()
        e0, e1 = _events()
        e0.record()
        for _ in range(args.steps):
            tok = eng.forward_rows([Row(0, pos, tok)], advance=False, read=True)[0]
            pos += 1
        e1.record()
        barrier()
        e2e_win.append(e0.elapsed_time(e1) / args.steps)
    e2e_ms = sorted(e2e_win)[len(e2e_win) // 2]
    w_bytes = cfg.weight_bytes_per_token(1.0 if args.int8_head else 2.0)
    kv_bytes = cfg.kv_bytes_per_token(args.kv_cache) * args.depth
    return {
        "metric": "decode_tokens_per_s", "baseline": 164.0,
        "ms_per_step": ms, "tokens_per_step": 1, "e2e_ms_per_step": e2e_ms,
        "h2d": K.CTRL_WORDS * 4, "d2h": K.CTRL_WORDS * 4, "launches": launches,
        "config": {"model": cfg.name, "global_batch": 1, "seq_len": args.depth, "parallelism": "replica",
                   "kv_cache": args.kv_cache, "lm_head": "int8" if args.int8_head else "bf16",
                   "weights": "W4A16 int4 g64, random init",
                   "l2": f"inputs larger than L2 ({w_bytes / 1e9:.1f} GB of weights per step)",
                   "bytes_per_step": w_bytes + kv_bytes, "windows_ms_per_step": [round(x, 4) for x in win_ms],
                   "launches_per_step": eng.launches(1, True),
                   "achieved_GBps": (w_bytes + kv_bytes) / (ms / 1e3) / 1e9},
    }


def run_prefill_bench(args, barrier, model: str, backend: str, n: int = 0, warm: int = 3, reps: int = 0) -> dict:
    cfg = preset(model)
    dev = torch.device("cuda", torch.cuda.current_device())
    weights = random_weights(cfg, device=dev, seed=0, exact=False)
    n = n or args.prefill_len
    eng = Engine(weights, max_seqs=1, max_len=n + 64, kv_dtype="bf16", prefill_backend=backend, use_graphs=False)
    g = torch.Generator().manual_seed(1)
    ids_t = torch.randint(0, cfg.vocab, (n,), generator=g, dtype=torch.int32).pin_memory()
    ids = ids_t.tolist()
    reps = reps or max(3, min(args.steps, 8))
    for _ in range(warm):
        eng.reset(0)
        eng.prefill(0, ids)
    barrier()
    e0, e1 = _events()
    n0 = K.launch_count
    e0.record()
    for _ in range(reps):
        eng.reset(0)
        eng.prefill(0, ids)       # includes the H2D copy of the ids and the D2H read of the first token
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / reps
    base = 11223.0 if cfg.is_moe else 2800.0
    return {"ms": ms, "tokens": n, "baseline": base, "launches": (K.launch_count - n0),
            "e2e_ms": ms, "h2d": n * 4, "d2h": K.CTRL_WORDS * 4,
            "config": {"model": cfg.name, "global_batch": 1, "seq_len": n,
                       "backend": eng._prefill.backend if eng._prefill is not None else backend,
                       "parallelism": "replica", "l2": "weights larger than L2"}}


def run_spec_bench(args, barrier, iters: int = 12, depth: int = 0, cases=None) -> dict:
    """Draft-and-verify iterations on the 27B shape with FORCED acceptance lengths, so that the step time does
    not depend on what random-init heads happen to propose: an MTP head (1 layer, draft depth 3) and a
    DFlash-style block drafter (2 layers; the pending token and 15 mask rows form one 16-token block whose rows attend
    to one another, 16 candidates per row, picked on the device), each verified in one trunk step of k + 1 rows.  tokens/s = (accepted + 1) / iteration time (draft + verify, host control included)."""
    import dataclasses
    import time
    from ..runtime.spec import SpecAdapter
    from ..server.adapter import EngineAdapter
    cfg = dataclasses.replace(preset(args.model), mtp_layers=1)
    dev = torch.device("cuda", torch.cuda.current_device())
    weights = random_weights(cfg, device=dev, seed=0, exact=False)
    depth = depth or min(args.depth, 4096)     # a real prompt pass of this many tokens comes first (draft heads included)
    out = {"depth": depth}
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab - 1, (depth,), generator=g).tolist()
    for kind, k, accepts, dv in (cases or (("mtp", 3, (0, 3), 0), ("mtp", 3, (3,), 32768), ("dflash", 7, (7,), 0), ("dflash", 15, (0, 3, 7), 0))):
        eng = Engine(weights, max_seqs=1, max_len=depth + 64 * (iters + 4) + 64, extra_kv_layers=2)
        ad = SpecAdapter(EngineAdapter(eng), kind, k, draft_vocab=dv)
        pending = ad.prefill(0, ids)
        for acc in accepts:
            def iteration(pending):
                drafts = ad.draft(0, pending, k)
                res = ad.step({0: [pending] + drafts})[0]
                keep = min(acc, len(drafts))
                if keep < len(drafts):
                    ad.truncate(0, ad.length(0) - (len(drafts) - keep))
                return res[keep]            # the trunk's token after the last kept row
            for _ in range(3):
                pending = iteration(pending)
            barrier()
            t0 = time.perf_counter()
            for _ in range(iters):
                pending = iteration(pending)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / iters
            out[f"{kind}_k{k}{'_dv' + str(dv) if dv else ''}_accept{acc + 1}"] = {"ms_per_iteration": dt * 1e3, "tokens_per_s": (acc + 1) / dt,
                                                  "rows_verified": k + 1}
        del eng, ad
        torch.cuda.empty_cache()
    return out


def run_prefix_bench(args, barrier, prefix_tokens: int = 65536, suffix_tokens: int = 512) -> dict:
    """A request whose first ``prefix_tokens`` positions are already cached: time to the first token cold, with the
    prefix in the device tier (pages adopted by reference), and with it restored from the pinned host tier."""
    import time
    from ..server.prefix import PrefixStore
    cfg = preset(args.model)
    dev = torch.device("cuda", torch.cuda.current_device())
    weights = random_weights(cfg, device=dev, seed=0, exact=False)
    n = prefix_tokens + suffix_tokens
    eng = Engine(weights, max_seqs=2, max_len=n + 64, use_graphs=False, prefill_backend=args.prefill_backend)
    host_gb = eng.kv.k[:, 0].numel() * 2 * 2 * (prefix_tokens // 16) / 2**30 * 1.05
    store = PrefixStore(eng, host_gb=host_gb, block_tokens=2048, device_fraction=0.6)
    g = torch.Generator().manual_seed(3)
    prefix = torch.randint(0, cfg.vocab, (prefix_tokens,), generator=g).tolist()
    out = {"prefix_tokens": prefix_tokens, "suffix_tokens": suffix_tokens, "block_tokens": 2048}

    def request(slot, seed):
        gs = torch.Generator().manual_seed(seed)
        ids = prefix + torch.randint(0, cfg.vocab, (suffix_tokens,), generator=gs).tolist()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        cached = store.begin(slot, ids)
        eng.prefill(slot, ids[cached:])
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        store.after_prefill(slot, ids)
        store.end(slot, ids)
        return cached, dt * 1e3

    cached, ms = request(0, 10)
    out["cold"] = {"cached_tokens": cached, "ttft_ms": ms, "tokens_per_s": n / (ms / 1e3)}
    cached, ms = request(1, 11)           # another slot: the blocks come from the device tier
    out["device_tier_hit"] = {"cached_tokens": cached, "ttft_ms": ms}
    # push every block to the host tier, then a third request restores them over PCIe / C2C
    store.resident.clear()
    eng.reset(0)
    eng.reset(1)
    while store._spill_one():
        pass
    cached, ms = request(0, 12)
    out["host_tier_restore"] = {"cached_tokens": cached, "ttft_ms": ms, "restored_blocks": store.stats["restored_blocks"],
                                "host_store_gib": host_gb}
    K.check_status()
    del eng, store, weights
    return out


def run_hybrid_bench(args, barrier) -> dict:
    """The 27B shape with gated delta-net layers (three before every attention layer): prompt pass (GEMM
    projections + sequential scan) and decode of one request, device-timed like the headline numbers."""
    cfg = preset("hybrid-27b")
    dev = torch.device("cuda", torch.cuda.current_device())
    weights = random_weights(cfg, device=dev, seed=0, exact=False)
    n, steps = args.prefill_len, max(8, min(args.steps, 64))
    eng = Engine(weights, max_seqs=1, max_len=n + 2 * steps + 64, prefill_backend=args.prefill_backend)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab, (n,), generator=g).tolist()
    for _ in range(2):
        eng.reset(0)
        first = eng.prefill(0, ids)
    barrier()
    e0, e1 = _events()
    e0.record()
    eng.reset(0)
    first = eng.prefill(0, ids)
    e1.record()
    barrier()
    pf_ms = e0.elapsed_time(e1)
    eng.decode_begin([0], [first])
    for _ in range(max(3, args.warmup)):
        eng.decode_step(read=False)
    barrier()
    e0, e1 = _events()
    e0.record()
    for _ in range(steps):
        eng.decode_step(read=False)
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1) / steps
    nbytes = cfg.weight_bytes_per_token(2.0) + cfg.kv_bytes_per_token("bf16") * n
    return {"model": cfg.name, "layers": f"{cfg.n_gdn_layers} gated delta-net + {cfg.n_layers - cfg.n_gdn_layers} attention",
            "decode": {"ms_per_step": ms, "tokens_per_s": 1e3 / ms, "depth": n, "steps": steps,
                       "achieved_GBps": nbytes / (ms / 1e3) / 1e9},
            "prefill": {"ms": pf_ms, "tokens": n, "tokens_per_s": n / pf_ms * 1e3,
                        "backend": eng._prefill.backend if eng._prefill is not None else "rows"}}


def run_batch_after_long_prompt(args, barrier, requests: int = 8, prompt: int = 32768, new_tokens: int = 256,
                                kv_dtype: str = "int8") -> dict:
    """The 8-request serving case of the 27B configuration on ONE GPU: every request ingests a ``prompt``-token
    context (int8 KV cache), then all of them decode ``new_tokens`` tokens together, one step of ``requests`` rows per
    token.  Prompt tokens/s over all requests and decode tokens/s of the batch (CUDA events around each part)."""
    cfg = preset(args.model)
    dev = torch.device("cuda", torch.cuda.current_device())
    weights = random_weights(cfg, device=dev, seed=0, exact=False)
    eng = Engine(weights, max_seqs=requests, max_len=prompt + new_tokens + 64, kv_dtype=kv_dtype,
                 prefill_backend="int8" if kv_dtype == "int8" else args.prefill_backend)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (prompt,), generator=g).tolist() for _ in range(requests)]
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    barrier()
    e[0].record()
    toks = [eng.prefill(slot, prompts[slot]) for slot in range(requests)]
    e[1].record()
    from ..runtime.engine import Row
    for _ in range(3):      # capture the 8-row step before the timed part
        rows = [Row(slot, eng.seq_len[slot], toks[slot]) for slot in range(requests)]
        toks = eng.forward_rows(rows)
    torch.cuda.synchronize()
    e[2].record()
    for _ in range(new_tokens - 3):
        rows = [Row(slot, eng.seq_len[slot], toks[slot]) for slot in range(requests)]
        toks = eng.forward_rows(rows)
    e[3].record()
    torch.cuda.synchronize()
    K.check_status()
    pms, dms = e[0].elapsed_time(e[1]), e[2].elapsed_time(e[3])
    steps = new_tokens - 3
    return {"requests": requests, "prompt_tokens_each": prompt, "new_tokens_each": new_tokens, "kv_cache": kv_dtype,
            "prompt_ms": pms, "prompt_tokens_per_s": requests * prompt / (pms / 1e3),
            "decode_ms_per_step": dms / steps, "decode_tokens_per_s_total": requests * steps / (dms / 1e3),
            "note": "every step's rows go host -> device and its tokens device -> host (the engine's public call)"}

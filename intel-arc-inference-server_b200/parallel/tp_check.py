"""Tensor-parallel self-check and timing, run as one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m b200serve.parallel.tp_check --model small-dense --check
    ... -m b200serve.parallel.tp_check --model dense-27b --bench --depth 4096 --steps 32

``--check``: every rank builds the whole (small) model, runs it on its own GPU as the one-GPU
answer, then the group runs the sharded model in both modes; logits of the prompt's last position
and a teacher-forced decode must agree with the one-GPU run within rounding, and all ranks must
hold identical tokens and identical residual bits.  ``--bench``: CUDA-event time of decode steps,
max over ranks, fused wires against the NCCL comparison path.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def widen_for(cfg, world: int):
    """A small preset widened (heads, FFN) so that it divides over ``world`` ranks."""
    if world > 1 and (cfg.n_kv_heads % world or cfg.ffn % (64 * world)):
        import dataclasses
        cfg = dataclasses.replace(cfg, n_kv_heads=max(cfg.n_kv_heads, world), n_q_heads=max(cfg.n_q_heads, 2 * world),
                                  ffn=192 * world)
    return cfg


def self_check(cfg, modes=("fused", "nccl"), prompt_len: int = 40, kv_dtype: str = "bf16") -> dict:
    """The sharded model against the same model on one GPU (every rank computes the one-GPU answer itself): logits of
    the prompt's last position, 12 teacher-forced decode steps, and bit-equal tokens and residual rows on all ranks.
    Returns ``{mode: {...,"ok": bool}}``; call it on every rank of an initialised process group."""
    import torch.distributed as dist
    from ..models.weights import random_weights
    from ..ops import lib as K
    from ..runtime.engine import Engine, Row
    from . import tp as TP
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    report = {}
    full = random_weights(cfg, device=dev, seed=0)
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), generator=g).tolist()
    one = Engine(full, max_seqs=1, max_len=prompt_len + 216, use_graphs=False, kv_dtype=kv_dtype)
    first = one.prefill(0, prompt)
    ref_logits = one.model.buf.logits[one.last_prefill_row].clone()
    ref_toks = [first]
    for _ in range(12):
        ref_toks.append(one.forward_rows([Row(0, one.seq_len[0], ref_toks[-1])])[0])
    shard = TP.shard_weights(full, rank, world, dev)
    per = (cfg.vocab + world - 1) // world
    for mode in modes:
        eng = TP.make_engine(shard, mode=mode, max_seqs=1, max_len=prompt_len + 216, use_graphs=(mode == "fused"),
                             kv_dtype=kv_dtype)
        t0 = eng.prefill(0, prompt)
        lg = eng.model.buf.logits[eng.last_prefill_row]
        want = ref_logits[rank * per: rank * per + lg.numel()]
        err = float((lg - want).abs().max())
        scale = float(ref_logits.abs().max())
        toks = [t0]
        agree = int(t0 == first)
        for i in range(12):   # teacher-forced: feed the one-GPU tokens, compare each arg-max
            t = eng.forward_rows([Row(0, eng.seq_len[0], ref_toks[i])])[0]
            toks.append(t)
            agree += int(t == ref_toks[i + 1])
        tt = torch.tensor(toks, device=dev, dtype=torch.int64)
        all_t = [torch.empty_like(tt) for _ in range(world)]
        rs = eng.model.buf.resid[:1].clone().view(torch.int16).to(torch.int64)
        all_r = [torch.empty_like(rs) for _ in range(world)]
        if world > 1:
            dist.all_gather(all_t, tt)
            dist.all_gather(all_r, rs)
        else:
            all_t, all_r = [tt], [rs]
        same_tok = all(bool((x == all_t[0]).all()) for x in all_t)
        same_res = all(bool((x == all_r[0]).all()) for x in all_r)
        K.check_status()
        good = err < 0.02 * max(scale, 1.0) and agree >= 11 and same_tok and same_res
        report[mode] = {"logit_err": err, "logit_scale": scale, "agree": agree, "of": 13,
                        "ranks_same_tokens": same_tok, "ranks_same_residual": same_res, "ok": good}
        if hasattr(eng, "close"):
            eng.close()
        del eng
    return report


def spec_check(cfg, prompt_len: int = 40, new_tokens: int = 24, k: int = 3, kind: str = "mtp") -> dict:
    """Speculative decoding with an MTP head under tensor parallelism: every rank carries its slice of the head
    (layers sliced like the trunk's, the front held whole) and drafts in lockstep; greedy drafts + verify + accept must
    give the tokens of the same sharded engine decoding plainly, on every rank (the reference's tp_mtp_test.cc).
    ``kind`` "dflash": a block drafter instead -- every rank finds the candidates of its vocabulary slice, the ranks
    merge them, and all must pick the same drafts."""
    import dataclasses
    import torch.distributed as dist
    from ..models.weights import random_weights
    from ..native import host as H
    from ..ops import lib as K
    from ..runtime.spec import SpecAdapter
    from ..server.adapter import EngineAdapter
    from . import tp as TP
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    cfg = dataclasses.replace(cfg, mtp_layers=1)
    full = random_weights(cfg, device=dev, seed=0)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab, (prompt_len,), generator=g).tolist()
    shard = TP.shard_weights(full, rank, world, dev)
    max_len = prompt_len + new_tokens + 64
    plain = TP.make_engine(shard, mode="fused", max_seqs=1, max_len=max_len)
    plain.model.attn_fixed_spans = True       # the spec engine's setting: a row's bits must not depend on its company
    plain.graphs.clear()
    want = plain.generate(prompt, new_tokens)
    if hasattr(plain, "close"):
        plain.close()
    del plain
    eng = TP.make_engine(shard, mode="fused", max_seqs=1, max_len=max_len, extra_kv_layers=2)
    ad = SpecAdapter(EngineAdapter(eng), kind, k)
    pending = ad.prefill(0, prompt)
    got, iters, accepted, same_drafts = [pending], 0, 0, True
    while len(got) < new_tokens:
        drafts = ad.draft(0, pending, k)
        if world > 1:      # every rank proposes the same tokens
            dt = torch.tensor(drafts + [0] * (k - len(drafts)), device=dev, dtype=torch.int64)
            all_d = [torch.empty_like(dt) for _ in range(world)]
            dist.all_gather(all_d, dt)
            same_drafts = same_drafts and all(bool((x == all_d[0]).all()) for x in all_d)
        out = ad.step({0: [pending] + drafts})[0]
        acc, nxt = H.accept_greedy(out, drafts)
        if acc < len(drafts):
            ad.truncate(0, ad.length(0) - (len(drafts) - acc))
        got += drafts[:acc] + [nxt]
        pending = nxt
        iters += 1
        accepted += acc
    K.check_status()
    tt = torch.tensor(got[:new_tokens], device=dev, dtype=torch.int64)
    all_t = [torch.empty_like(tt) for _ in range(world)]
    if world > 1:
        dist.all_gather(all_t, tt)
    else:
        all_t = [tt]
    same = all(bool((x == all_t[0]).all()) for x in all_t)
    good = got[:new_tokens] == want[:new_tokens] and same and same_drafts and ad.stats["drafted"] >= iters
    if hasattr(eng, "close"):
        eng.close()
    return {"kind": kind, "tokens_equal_plain": got[:new_tokens] == want[:new_tokens], "ranks_same_tokens": same,
            "ranks_same_drafts": same_drafts, "iterations": iters,
            "drafted": ad.stats["drafted"], "accepted": accepted, "prompt": prompt_len, "ok": good}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="small-dense")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--depth", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--modes", default="fused,nccl")
    ap.add_argument("--kv-cache", default="bf16", help="bf16 | int8 (the check then runs both engines with an int8 KV cache)")
    ap.add_argument("--prefill", type=int, default=0, help="time prompt passes of this many tokens")
    ap.add_argument("--ops", type=int, default=0, help="time the fused GEMM+collective kernels alone on a chunk of this many rows")
    ap.add_argument("--pp", action="store_true", help="pipeline check: the ranks are stages; tokens must equal the one-GPU run")
    ap.add_argument("--prompt", type=int, default=40, help="prompt length of --check (> 64 takes the GEMM path)")
    ap.add_argument("--spec", action="store_true", help="MTP drafts + verify under tensor parallelism equal plain decoding")
    args = ap.parse_args()

    import torch.distributed as dist
    from ..models.config import preset
    from ..models.weights import random_weights
    from ..ops import lib as K
    from ..runtime.engine import Engine, Row
    from . import tp as TP

    rank, world, local = TP.init_dist()
    dev = torch.device("cuda", local)
    cfg = preset(args.model)
    if args.check:
        cfg = widen_for(cfg, world)   # so that the small preset divides over this many ranks
    ok = True
    report = {"world": world, "model": cfg.name}

    def maxr(x: float) -> float:
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    if args.check:
        chk = self_check(cfg, args.modes.split(","), args.prompt, kv_dtype=args.kv_cache)
        ok = ok and all(v["ok"] for v in chk.values())
        report.update(chk)
    if args.spec:
        for kind in ("mtp", "dflash"):
            sc = spec_check(widen_for(cfg, world), args.prompt, kind=kind)
            ok = ok and sc["ok"]
            report["spec_" + kind] = sc
    if args.pp:
        from . import pp as PP
        full = random_weights(cfg, device=dev, seed=0)
        g = torch.Generator().manual_seed(5)
        prompt = torch.randint(0, cfg.vocab, (args.prompt,), generator=g).tolist()
        # a long prompt takes the tcgen05 prompt kernels on both sides (chunks of 128 so that several are in flight)
        long_prompt = args.prompt > 64
        one = Engine(full, max_seqs=1, max_len=args.prompt + 64, use_graphs=False,
                     prefill_backend="auto" if long_prompt else "rows")
        one.reset(0)
        first = one.prefill(0, prompt, chunk=128 if long_prompt else None)
        one.decode_begin([0], [first])
        want = [first] + [one.decode_step()[0] for _ in range(11)]
        a, b = PP.split_layers(cfg.n_layers, world)[rank]
        eng = PP.PipelineEngine(PP.stage_weights(full, a, b), rank, world, max_seqs=1, max_len=args.prompt + 64)
        eng.reset(0)
        first = eng.prefill(0, prompt, chunk=128 if long_prompt else None)
        eng.decode_begin([0], [first])
        got = [first] + [eng.decode_step()[0] for _ in range(11)]
        K.check_status()
        good = got == want
        ok = ok and good
        report["pp"] = {"stages": world, "layers": [a, b], "tokens_equal": good, "sent_bytes": eng.sent_bytes,
                        "tokens": got, "want": want}
    if args.bench:
        for mode in args.modes.split(","):
            report[f"bench_{mode}"] = TP.bench_decode(cfg, mode, args.depth, args.steps, args.warmup, args.rows)
    if args.prefill:
        for mode in args.modes.split(","):
            report[f"prefill_{mode}"] = TP.bench_prefill(cfg, mode, args.prefill)
    if args.ops:
        import os
        peaks = {}
        path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
        if os.path.exists(path):
            with open(path) as f:
                peaks = json.load(f)
        report["fused_ops"] = TP.bench_fused_ops(cfg, args.ops, peaks=peaks)
    if rank == 0:
        print(json.dumps(report))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())

"""Expert-parallel self-check and timing, one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        -m b200serve.parallel.ep_check --model small-moe --check
    ... -m b200serve.parallel.ep_check --model moe-35b-a3b --prefill 4096

``--check``: every rank holds the whole small model, runs a prompt on one GPU as the answer, then the group
runs the same prompt with the experts spread over the ranks (fused wires, then the NCCL comparison); logits
must agree within rounding.  ``--prefill N``: every rank ingests its own N-token prompt (data-parallel
attention, expert-parallel MoE); tokens/s is the whole group's, time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch


def self_check(cfg, modes=("fused", "nccl"), n_tokens: int = 300) -> dict:
    """The model with its experts spread over the ranks against the same model on one GPU: every rank holds the whole
    (small) model, runs a prompt alone as the answer, then the group runs the same prompt in each mode; logits must
    agree within rounding and the next token must be the same.  Returns ``{mode: {..., "ok": bool}}``."""
    import torch.distributed as dist
    from ..models.weights import random_weights
    from ..ops import lib as K
    from ..runtime.engine import Engine
    from ..runtime.prefill import PrefillRunner
    from . import ep as EP
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dev = torch.device("cuda", torch.cuda.current_device())
    report = {}
    full = random_weights(cfg, device=dev, seed=4)
    g = torch.Generator().manual_seed(12)
    ids = torch.randint(0, cfg.vocab, (n_tokens,), generator=g).tolist()
    one = Engine(full, max_seqs=1, max_len=1024, use_graphs=False)
    t_ref = PrefillRunner(one, max_chunk=512).run(0, ids)
    ref = one.model.buf.logits[0].clone()
    shard = EP.ep_shard_weights(full, rank, world)
    for mode in modes:
        eng = Engine(shard, max_seqs=1, max_len=1024, use_graphs=False)
        runner = PrefillRunner(eng, max_chunk=512)
        runner.ep = EP.EpMoe(cfg, 512, mode=mode)
        t = runner.run(0, ids)
        K.check_status()
        err = float((eng.model.buf.logits[0] - ref).abs().max())
        good = err < 0.02 * float(ref.abs().max()) and t == t_ref
        report[mode] = {"logit_err": err, "logit_scale": float(ref.abs().max()), "token": t, "want": t_ref, "ok": good}
        if world > 1:
            dist.barrier()
        runner.ep.close()
    if "fused" in modes:
        report["decode_rows_fused"] = check_rows(cfg, full, shard, ids[:64])
    return report


def check_rows(cfg, full, shard, ids, steps: int = 6) -> dict:
    """Decode steps with the experts spread over the ranks against the same model on one GPU.  Every rank runs its OWN
    request (the prompt rotated by its rank), so the ranks send each other different rows; each compares its tokens and
    last logits with a one-GPU engine run of the same request."""
    import torch.distributed as dist
    from ..ops import lib as K
    from ..runtime.engine import Engine
    from . import ep as EP
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    mine = ids[rank:] + ids[:rank]
    # both engines ingest the prompt through row steps (up to max_rows positions per step), so the sharded one's
    # prompt goes through the row form of the exchange too
    from ..runtime.engine import Row
    one = Engine(full, max_seqs=1, max_len=256, use_graphs=False, prefill_backend="rows")
    eng = Engine(shard, max_seqs=1, max_len=256, use_graphs=False, prefill_backend="rows")
    ep = EP.attach_rows(eng, eng.max_rows)
    tok, mine_tok = one.prefill(0, mine), eng.prefill(0, mine)
    want, got = [tok], [mine_tok]
    scale = float(one.model.buf.logits[0].abs().max())
    err = float((eng.model.buf.logits[eng.last_prefill_row] - one.model.buf.logits[one.last_prefill_row]).abs().max())
    for _ in range(steps - 1):      # teacher-forced with the one-GPU tokens: every step's logits are comparable
        r = one.forward_rows([Row(0, one.seq_len[0], tok)])[0]
        g = eng.forward_rows([Row(0, eng.seq_len[0], tok)])[0]
        err = max(err, float((eng.model.buf.logits[0] - one.model.buf.logits[0]).abs().max()))
        want.append(r)
        got.append(g)
        tok = r
    K.check_status()
    agree = sum(int(a == b) for a, b in zip(got, want))
    good = err < 0.02 * scale and agree >= steps - 1       # the return rows are bf16: a near-tie may flip
    t = torch.tensor([1 if good else 0], device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
    ep.close()
    return {"tokens": got, "want": want, "agree": agree, "of": steps, "logit_err": err, "logit_scale": scale, "ok": bool(int(t))}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="small-moe")
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--prefill", type=int, default=0)
    ap.add_argument("--modes", default="fused,nccl")
    args = ap.parse_args()
    import torch.distributed as dist
    from ..models.config import preset
    from ..models.weights import random_weights
    from ..ops import lib as K
    from ..runtime.engine import Engine
    from ..runtime.prefill import PrefillRunner
    from . import ep as EP
    from . import tp as TP

    rank, world, local = TP.init_dist()
    dev = torch.device("cuda", local)
    cfg = preset(args.model)
    report = {"world": world, "model": cfg.name}
    ok = True
    if args.check:
        chk = self_check(cfg, args.modes.split(","))
        ok = ok and all(v["ok"] for v in chk.values())
        report.update(chk)
    if args.prefill:
        report.update(EP.bench_prefill(cfg, args.prefill, args.modes.split(",")))
    if rank == 0:
        print(json.dumps(report))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())

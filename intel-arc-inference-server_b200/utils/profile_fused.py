"""The fused tensor-parallel prompt layer and the fused expert-parallel block as a group of ONE rank, for a launch
list on one GPU:

    python -m b200serve.utils.profile_fused --what tp --tokens 512
    python -m b200serve.utils.profile_fused --what ep --tokens 512

With a single rank every "peer" store lands in the GPU's own buffers, so the kernels that run are exactly the ones a
multi-GPU group runs (GEMM -> reduce-scatter push, owner fold + norm + all-gather push, all-gather -> GEMM wait;
counts push, plan, dispatch, grouped GEMMs with arrival waits and the return epilogue, flag / wait, combine) -- and a
profiler that must not wrap a multi-rank job can still list them.  No collective library is loaded on these paths.
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--what", default="tp", help="tp | ep | ep-rows")
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--passes", type=int, default=2)
    args = ap.parse_args()
    from ..models.config import preset
    from ..models.weights import random_weights
    from ..ops import lib as K
    from ..runtime.engine import Engine
    from ..runtime.prefill import PrefillRunner
    g = torch.Generator().manual_seed(11)
    if args.what == "tp":
        from ..parallel.tp_prefill import TpPrefillRunner
        cfg = preset("small-dense")
        eng = Engine(random_weights(cfg, device="cuda", seed=3), max_seqs=1, max_len=args.tokens + 64, use_graphs=False)
        ids = torch.randint(0, cfg.vocab, (args.tokens,), generator=g).tolist()
        runner = TpPrefillRunner(eng, max_chunk=512)
        for _ in range(args.passes):
            eng.reset(0)
            tok = runner.run(0, ids)
        runner.close()
    elif args.what == "ep":
        from ..parallel.ep import EpMoe
        cfg = preset("small-moe")
        eng = Engine(random_weights(cfg, device="cuda", seed=4), max_seqs=1, max_len=args.tokens + 64, use_graphs=False)
        ids = torch.randint(0, cfg.vocab, (args.tokens,), generator=g).tolist()
        runner = PrefillRunner(eng, max_chunk=512)
        runner.ep = EpMoe(cfg, 512, mode="fused")
        for _ in range(args.passes):
            eng.reset(0)
            tok = runner.run(0, ids)
        runner.ep.close()
    else:
        from ..parallel.ep import attach_rows
        cfg = preset("small-moe")
        eng = Engine(random_weights(cfg, device="cuda", seed=4), max_seqs=1, max_len=256, use_graphs=False,
                     prefill_backend="rows")
        ep = attach_rows(eng, eng.max_rows)
        ids = torch.randint(0, cfg.vocab, (40,), generator=g).tolist()
        tok = eng.generate(ids, 4)[-1]
        ep.close()
    torch.cuda.synchronize()
    K.check_status()
    print("last token", tok)


if __name__ == "__main__":
    main()

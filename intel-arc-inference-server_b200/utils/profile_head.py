"""The lm_head GEMV + arg-max candidates alone, for a profiler capture on a small case:

    python -m b200serve.utils.profile_head --rows 16 --vocab 151936 --hidden 5120 --time

bf16 weights of a 27B-shape head (1.56 GB: larger than L2), ``--rows`` activation rows, a few launches.
"""
from __future__ import annotations

import argparse

import torch


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=16)
    ap.add_argument("--vocab", type=int, default=151936)
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--int8", action="store_true", help="an int8 head with one scale per row (the FMA form)")
    ap.add_argument("--time", action="store_true", help="CUDA-event microseconds per launch (graph of 10 launches)")
    args = ap.parse_args()
    from ..ops import lib as K
    n, h, m = args.vocab, args.hidden, args.rows
    w = (torch.randn(n, h, device="cuda") * 0.02).to(torch.bfloat16)
    x = torch.randn(m, h, device="cuda").to(torch.bfloat16)
    sc = None
    if args.int8:
        sc = w.float().abs().amax(1) / 127
        w = torch.round(w.float() / sc[:, None]).to(torch.int8)
    ncand = K.head_ncand(n)
    out = torch.zeros(m, n, device="cuda")
    cv = torch.zeros(m * ncand, device="cuda")
    ci = torch.zeros(m * ncand, dtype=torch.int32, device="cuda")
    for _ in range(args.launches):
        K.head_gemv(w, x, out, m, n, h, cv, ci, wscale=sc)
    torch.cuda.synchronize()
    K.check_status()
    if args.time:
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for _ in range(10):
                K.head_gemv(w, x, out, m, n, h, cv, ci, wscale=sc)
        gr.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        gr.replay()
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 100
        print(f"rows {m}: {us:.1f} us per launch, {n * h * w.element_size() / us / 1e6:.2f} TB/s of weights")


if __name__ == "__main__":
    main()

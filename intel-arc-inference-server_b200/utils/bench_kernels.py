"""Kernel micro-benchmarks with CUDA events: achieved bandwidth / FLOP rate per shape.

    python -m b200serve.utils.bench_kernels gemv            # W4A16 weight-streaming kernel, 27B shapes
    python -m b200serve.utils.bench_kernels gemm            # tcgen05 GEMMs, 27B prefill shapes

Weights rotate through enough copies to exceed the 126 MB L2 between launches, so
every launch streams from HBM.  Fractions are of the measured peaks in
``MEASURED_PEAKS.json`` when that file is present beside the repository root.
"""
from __future__ import annotations

import json
import os
import sys

import torch

from ..ops import lib as K
from ..utils import quant as Q


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def time_ms(fn, iters=20, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def bench_gemv(ms_list=(1, 4, 8, 16, 64), only=None, iters_mult=4, graph=False):
    hbm, _, src = peaks()
    shapes = [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120), ("down", 5120, 17408)]
    for name, n, k in shapes:
        if only and name != only:
            continue
        nbytes = (n // 128) * (k // 64) * Q.BLOCK_BYTES
        copies = max(2, int(400e6 // nbytes) + 1)
        ws = [Q.random_w4b(n, k, "cuda", i) for i in range(copies)]
        s = K.gemv_splits(n, k)
        for m in ms_list:
            x = torch.randn(m, k, device="cuda").to(torch.bfloat16)
            out = torch.zeros(s, m, n, device="cuda")
            it = [0]

            fed = os.environ.get("B2_BENCH_PREQUANT", "0") == "1"   # time the GEMV alone on pre-quantised rows
            if fed:
                xq = torch.zeros(m * (k // 64) * 128, dtype=torch.uint8, device="cuda")
                gs = torch.zeros(64 * (k // 64) * 2, dtype=torch.int32, device="cuda")
                K.quant_x(x, m, k, xq, gs)

            def fn():
                if fed:
                    K.gemv_w4_fused(ws[it[0] % copies], xq, out, m, n, k, s, x_mode=3, norm_ssq=gs)
                else:
                    K.gemv_w4(ws[it[0] % copies], x, out, m, n, k, s)
                it[0] += 1
            ms = time_ms(fn, iters=max(2, iters_mult * copies))
            if graph:
                # the same launches inside a CUDA graph: no host launch cost between kernels
                n_in = 4 * copies
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for _ in range(n_in):
                        fn()
                ms = time_ms(g.replay, iters=5) / n_in
            gbs = nbytes / ms / 1e6
            print(f"gemv_w4 {name:8s} N={n:6d} K={k:6d} M={m:3d} S={s:2d}  {ms * 1e3:8.2f} us  {gbs:8.1f} GB/s  "
                  f"{gbs / hbm:5.2f} of {src} HBM copy bandwidth")
        del ws
    K.check_status()


def bench_gemm():
    _, tf, src = peaks()
    from ..ops import gemm as G
    for name, n, k in [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120), ("down", 5120, 17408)]:
        for m in (4096,):
            a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
            nb = max(2, int(400e6 // (n * k * 2)) + 1)
            bs = [(torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(nb)]
            c = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
            it = [0]

            def fn():
                G.gemm_bf16(a, bs[it[0] % nb], c)
                it[0] += 1
            ms = time_ms(fn, iters=3 * nb)
            fl = 2.0 * m * n * k / ms / 1e9
            ref = time_ms(lambda: torch.matmul(a, bs[0].t(), out=c), iters=3 * nb)
            print(f"gemm_tc bf16 {name:8s} M={m} N={n} K={k}: {ms:7.3f} ms {fl:7.1f} TFLOP/s "
                  f"{fl / tf:5.2f} of {src} cuBLAS burst; torch.matmul {ref:7.3f} ms")
            a8 = torch.randint(-127, 127, (m, k), device="cuda", dtype=torch.int8)
            b8 = torch.randint(-127, 127, (n, k), device="cuda", dtype=torch.int8)
            sa, sb = torch.rand(m, device="cuda"), torch.rand(n, device="cuda")
            ms8 = time_ms(lambda: G.gemm_i8(a8, b8, sa, sb, c), iters=6)
            print(f"gemm_tc int8 {name:8s} M={m} N={n} K={k}: {ms8:7.3f} ms {2.0 * m * n * k / ms8 / 1e9:7.1f} TOP/s")
            del bs
    K.check_status()


if __name__ == "__main__":
    what = sys.argv[1] if len(sys.argv) > 1 else "gemv"
    if what == "gemv-one":      # one shape, one M, few launches: the target of an ncu capture
        bench_gemv((int(sys.argv[3]),), only=sys.argv[2], iters_mult=1)
    elif what == "prefill-one":  # two layers of the 27B shape over a 2048-token prompt: GEMM and attention captures
        from dataclasses import replace
        from ..models.config import preset
        from ..models.weights import random_weights
        from ..runtime.engine import Engine
        cfg = replace(preset("dense-27b"), n_layers=2)
        ntok = int(sys.argv[2]) if len(sys.argv) > 2 else 2048
        backend = sys.argv[3] if len(sys.argv) > 3 else "bf16-resident"     # or int8 | w4
        eng = Engine(random_weights(cfg, device="cuda", seed=0, exact=False), max_seqs=1, max_len=ntok + 64, use_graphs=False,
                     prefill_backend=backend)
        ids = torch.randint(0, cfg.vocab, (ntok,)).tolist()
        for _ in range(2):
            eng.reset(0)
            eng.prefill(0, ids)
        torch.cuda.synchronize()
        K.check_status()
    elif what == "fused-one":   # the fused collective kernels as a group of one rank (every "peer" buffer is local)
        from dataclasses import replace
        from ..models.config import preset
        from ..models.weights import random_weights
        from ..parallel.ep import EpMoe
        from ..parallel.tp_prefill import TpPrefillRunner
        from ..runtime.engine import Engine
        from ..runtime.prefill import PrefillRunner
        cfg = replace(preset("dense-27b"), n_layers=2)
        eng = Engine(random_weights(cfg, device="cuda", seed=0, exact=False), max_seqs=1, max_len=2112, use_graphs=False,
                     prefill_backend="bf16-resident")
        ids = torch.randint(0, cfg.vocab, (2048,)).tolist()
        runner = TpPrefillRunner(eng, max_chunk=2048)
        for _ in range(2):
            eng.reset(0)
            runner.run(0, ids)
        torch.cuda.synchronize()
        K.check_status()
        mcfg = replace(preset("moe-35b-a3b"), n_layers=2)
        meng = Engine(random_weights(mcfg, device="cuda", seed=0, exact=False), max_seqs=1, max_len=2112, use_graphs=False,
                      prefill_backend="bf16-resident")
        mrun = PrefillRunner(meng, max_chunk=2048)
        mrun.ep = EpMoe(mcfg, 2048)
        for _ in range(2):
            meng.reset(0)
            mrun.run(0, ids)
        torch.cuda.synchronize()
        K.check_status()
    elif what == "sampler-one":  # the device sampler on a few rows of 27B-vocabulary logits (temperature, top-k, top-p)
        m, n = (int(sys.argv[2]) if len(sys.argv) > 2 else 8), 151936
        logits = torch.randn(m, n, device="cuda") * 3
        f32, i32 = torch.float32, torch.int32
        temp = torch.full((m,), 0.8, dtype=f32, device="cuda")
        top_k = torch.full((m,), 40, dtype=i32, device="cuda")
        top_p = torch.full((m,), 0.95, dtype=f32, device="cuda")
        seed = torch.arange(m, dtype=torch.int64, device="cuda") + 1234
        tok, status = torch.zeros(m, dtype=i32, device="cuda"), torch.zeros(m, dtype=i32, device="cuda")
        ms = time_ms(lambda: K.sample_rows(logits, m, n, temp, top_k, top_p, seed, tok, status), iters=5)
        print(f"sample_rows {m} rows x {n} logits: {ms * 1e3:.1f} us per launch; tokens {tok.tolist()} status {status.tolist()}")
        K.check_status()
    elif what == "gemv-graph":  # back-to-back launches inside a CUDA graph
        bench_gemv((1, 4, 8), graph=True)
    else:
        {"gemv": bench_gemv, "gemm": bench_gemm}[what]()

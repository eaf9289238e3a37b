"""The allocation-free decode-attention entry point, called through its exported C symbol.

Embedders that may not allocate device memory (a plug-in under a framework that owns the whole GPU
pool, a latency-bound serving thread that must stay off cudaMalloc's locks, a C caller without an
allocator) use ``b2_attn_decode_static``: the split-KV scratch lives in a fixed device array inside
the library.  Its output must equal the regular entry point's, on two calls in a row (the second
call finds the first call's leftovers in the shared array), and it must refuse sizes beyond the
array.  Collected last on purpose: a run that stops at the first failure has run everything else.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, m, n_q, n_kv, d, ctx, nsplit):
    from b200serve.ops import lib as K
    torch.manual_seed(seed)
    max_blocks = (ctx + 15) // 16 + 2
    num_pages = max_blocks + 4
    table = torch.zeros(2, max_blocks, dtype=torch.int32)
    table[1, : max_blocks - 2] = torch.randperm(num_pages - 1)[: max_blocks - 2].to(torch.int32) + 1
    table = table.cuda()
    kc = (torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    q = torch.randn(m, n_q * d, device="cuda").to(torch.bfloat16)
    ctrl = torch.zeros(K.CTRL_WORDS, dtype=torch.int32)
    for i in range(m):
        ctrl[K.CTRL_ROW_REQ + i] = 1
        ctrl[K.CTRL_ROW_POS + i] = ctx - m + i
    return K, q, kc, vc, table, ctrl.cuda(), max_blocks


@pytest.mark.parametrize("m,n_q,n_kv,d,ctx,nsplit", [(1, 40, 8, 128, 700, 16), (3, 4, 2, 64, 90, 4), (4, 16, 4, 128, 333, 7)])
def test_static_entry_matches_regular_entry_twice(m, n_q, n_kv, d, ctx, nsplit):
    K, q, kc, vc, table, ctrl, max_blocks = _case(m * 100 + n_q, m, n_q, n_kv, d, ctx, nsplit)
    scale = 1.0 / math.sqrt(d)
    ref = torch.zeros(m, n_q * d, dtype=torch.bfloat16, device="cuda")
    o_part = torch.zeros(m * n_q * nsplit * d, device="cuda")
    ml = torch.zeros(m * n_q * nsplit * 2, device="cuda")
    K.attn_decode(q, kc, vc, table, ctrl, o_part, ml, ref, m, n_q, n_kv, d, nsplit, max_blocks, scale)
    fn = K.lib().b2_attn_decode_static            # the exported C symbol
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        out = torch.full((m, n_q * d), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = fn(p(q), p(kc), p(vc), p(None), p(None), p(table), p(ctrl), p(out), m, n_q, n_kv, d, nsplit, max_blocks,
                ctypes.c_float(scale), 0, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        # same kernels, same order of operations: the tolerance of the attention tests, in practice bit-equal
        assert (out.float() - ref.float()).abs().max() <= 0.02 * ref.float().abs().max() + 1e-3
        assert torch.equal(out, ref), f"call {call}"
        # a different problem in between leaves other contents in the shared array
        K2, q2, kc2, vc2, t2, c2, mb2 = _case(999 + call, 2, 8, 2, 128, 50, 3)
        o2 = torch.zeros(2, 8 * 128, dtype=torch.bfloat16, device="cuda")
        assert fn(p(q2), p(kc2), p(vc2), p(None), p(None), p(t2), p(c2), p(o2), 2, 8, 2, 128, 3, mb2,
                  ctypes.c_float(scale), 0, stream) == 0
    K.check_status()


def test_static_entry_refuses_sizes_beyond_its_array():
    K, q, kc, vc, table, ctrl, max_blocks = _case(5, 1, 8, 2, 128, 40, 2)
    fn = K.lib().b2_attn_decode_static
    fn.restype = ctypes.c_int
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())
    out = torch.zeros(8, 8 * 128, dtype=torch.bfloat16, device="cuda")
    args = lambda m, n_q, nsplit, d: (p(q), p(kc), p(vc), p(None), p(None), p(table), p(ctrl), p(out), m, n_q, 2, d,
                                       nsplit, max_blocks, ctypes.c_float(0.1), 0, ctypes.c_void_p(0))
    assert fn(*args(5, 8, 2, 128)) == -10          # too many rows
    assert fn(*args(1, 128, 2, 128)) == -10        # too many heads
    assert fn(*args(1, 8, 17, 128)) == -10         # too many splits
    assert fn(*args(1, 8, 2, 256)) == -10          # head size without a kernel
    torch.cuda.synchronize()

"""Decode-path kernels against plain PyTorch fp32 references of the same op (GPU)."""
import math

import pytest
import torch

from b200serve.models.oracle import apply_rope, rope_tables
from b200serve.models.weights import deinterleave16
from b200serve.utils import quant as Q

pytestmark = pytest.mark.gpu


def K():
    from b200serve.ops import lib
    return lib


def _ctrl(rows):
    k = K()
    c = torch.zeros(k.CTRL_WORDS, dtype=torch.int32)
    c[k.CTRL_N_ROWS] = len(rows)
    for i, (req, pos, tok) in enumerate(rows):
        c[k.CTRL_ROW_REQ + i], c[k.CTRL_ROW_POS + i], c[k.CTRL_CUR_TOKEN + i] = req, pos, tok
    return c.cuda()


@pytest.mark.parametrize("m,n,k", [(1, 256, 256), (1, 5120, 5120), (3, 1408, 256), (8, 512, 704),
                                     (13, 640, 1024), (33, 384, 2048), (64, 256, 512), (2, 200, 192)])
def test_gemv_w4_matches_fp32(m, n, k):
    k_ = K()
    torch.manual_seed(m * 1000 + n)
    w = torch.randn(n, k) * 0.02
    q, s = Q.quantize_rtn(w)
    w4b = Q.to_w4b(q, s).cuda()
    wd = Q.dequant(q, s)
    x = (torch.randn(m, k)).to(torch.bfloat16)
    splits = k_.gemv_splits(n, k)
    out = torch.full((splits, m, n), float("nan"), device="cuda")
    k_.gemv_w4(w4b, x.cuda(), out, m, n, k, splits)
    torch.cuda.synchronize()
    k_.check_status()
    got = out.sum(0).cpu()
    ref = x.float() @ wd.t()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max() <= 2e-3 * ref.abs().max() + 1e-4


@pytest.mark.parametrize("m", [1, 4])
def test_gemv_w4_outlier_activations(m):
    """A few activations hundreds of times larger than the rest (the massive-activation channels of real models): the
    kernel re-quantises each 64-k group of a row to 15-bit integers against the GROUP's maximum, so an outlier may cost
    precision only inside its own group.  Checked per output against the fp32 product of the same bf16 inputs, with a
    tolerance scaled by each row's own |x| . |w| bound rather than by the largest output."""
    k_ = K()
    torch.manual_seed(11 + m)
    n, k = 768, 2048
    w = torch.randn(n, k) * 0.02
    q, s = Q.quantize_rtn(w)
    w4b = Q.to_w4b(q, s).cuda()
    wd = Q.dequant(q, s)
    x = torch.randn(m, k)
    x[:, 5] = 300.0          # one massive channel in group 0
    x[:, 1031] = -450.0      # another in group 16
    x[0, 64:128] = 0.0       # an all-zero group
    x = x.to(torch.bfloat16)
    splits = k_.gemv_splits(n, k)
    out = torch.full((splits, m, n), float("nan"), device="cuda")
    k_.gemv_w4(w4b, x.cuda(), out, m, n, k, splits)
    torch.cuda.synchronize()
    k_.check_status()
    got = out.sum(0).cpu()
    ref = x.float() @ wd.t()
    assert torch.isfinite(got).all()
    # error budget per group: |w| . (group max |x|) * 64 / 2^14 (half a quantisation step of every element)
    xg = x.float().abs().view(m, k // 64, 64).amax(dim=2)                       # [m][groups]
    wg = wd.abs().view(n, k // 64, 64).sum(dim=2)                               # [n][groups]
    bound = (xg @ wg.t()) / 16383.0 * 0.5 + 1e-5 * ref.abs()                    # [m][n]
    assert ((got - ref).abs() <= bound + 1e-4).all(), float(((got - ref).abs() / (bound + 1e-4)).max())
    # and the groups without an outlier keep their own precision: zero the outlier channels, the rest must agree tightly
    x2 = x.clone()
    x2[:, 5] = 0
    x2[:, 1031] = 0
    out2 = torch.zeros(splits, m, n, device="cuda")
    k_.gemv_w4(w4b, x2.cuda(), out2, m, n, k, splits)
    ref2 = x2.float() @ wd.t()
    assert (out2.sum(0).cpu() - ref2).abs().max() <= 2e-3 * ref2.abs().max() + 1e-4


def test_gemv_w4_rows_do_not_depend_on_m():
    """Property R: a row's bits are the same whether it runs alone or among other rows."""
    k_ = K()
    torch.manual_seed(7)
    n, k = 512, 1024
    w4b = Q.random_w4b(n, k, "cuda", 3)
    x = torch.randn(40, k, device="cuda").to(torch.bfloat16)
    s = k_.gemv_splits(n, k)
    outs = {}
    for m in (1, 5, 8, 9, 17, 40):
        o = torch.zeros(s, m, n, device="cuda")
        k_.gemv_w4(w4b, x[:m].contiguous(), o, m, n, k, s)
        outs[m] = o.sum(0)
    torch.cuda.synchronize()
    for m in (5, 8, 9, 17, 40):
        assert torch.equal(outs[m][0], outs[1][0])
        assert torch.equal(outs[40][:m], outs[m])


def test_gemv_w4_silu_mul_fold_input():
    k_ = K()
    torch.manual_seed(11)
    m, i_dim, n = 4, 704, 256
    s_in = 3
    gu = torch.randn(s_in, m, 2 * i_dim) * 0.5
    w = torch.randn(n, i_dim) * 0.02
    q, s = Q.quantize_rtn(w)
    w4b = Q.to_w4b(q, s).cuda()
    splits = k_.gemv_splits(n, i_dim)
    out = torch.zeros(splits, m, n, device="cuda")
    k_.gemv_w4(w4b, gu.cuda(), out, m, n, i_dim, splits, x_mode=1, s_in=s_in, x_slice=m * 2 * i_dim)
    torch.cuda.synchronize()
    g, u = deinterleave16(gu.sum(0))
    act = (torch.nn.functional.silu(g) * u).to(torch.bfloat16).float()
    ref = act @ Q.dequant(q, s).t()
    got = out.sum(0).cpu()
    assert (got - ref).abs().max() <= 3e-3 * ref.abs().max() + 1e-4


def test_resid_norm_embed_and_fold():
    k_ = K()
    torch.manual_seed(5)
    m, h, vocab = 5, 5120, 100
    embed = (torch.randn(vocab, h) * 0.02).to(torch.bfloat16).cuda()
    w = (1 + 0.1 * torch.randn(h)).cuda()
    toks = [3, 99, 0, 42, 7]
    ctrl = _ctrl([(0, i, t) for i, t in enumerate(toks)])
    resid = torch.zeros(m, h, dtype=torch.bfloat16, device="cuda")
    x = torch.zeros_like(resid)
    k_.resid_norm(0, m, h, w, 1e-6, resid, x, embed=embed, ctrl=ctrl, vocab=vocab)
    r_ref = embed[toks].float()
    x_ref = r_ref * torch.rsqrt(r_ref.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert torch.equal(resid, embed[toks])
    assert (x.float() - x_ref).abs().max() < 2e-2 * x_ref.abs().max()
    # fold: resid + sum of 3 slices
    part = torch.randn(3, m, h, device="cuda") * 0.05
    resid2 = torch.zeros_like(resid)
    k_.resid_norm(1, m, h, w, 1e-6, resid2, x, resid_in=resid, part=part, part_slice=m * h, splits=3)
    r2 = (resid.float() + part[0] + part[1] + part[2]).to(torch.bfloat16)
    assert torch.equal(resid2, r2)
    x2 = r2.float() * torch.rsqrt(r2.float().pow(2).mean(-1, keepdim=True) + 1e-6) * w
    assert (x.float() - x2).abs().max() < 1e-2 * x2.abs().max()
    k_.check_status()


@pytest.mark.parametrize("kv_int8", [False, True])
@pytest.mark.parametrize("n_q,n_kv,d", [(4, 2, 64), (40, 8, 128), (16, 4, 128)])
def test_rope_append_and_attention(n_q, n_kv, d, kv_int8):
    """rope_append writes q and the paged cache; attn_decode + merge reproduce softmax attention."""
    k_ = K()
    torch.manual_seed(n_q + d)
    ctx, m = 77, 3                       # 3 verify rows at positions ctx-3 .. ctx-1 of request 1
    max_blocks, num_pages = 8, 32
    qkv_dim = (n_q + 2 * n_kv) * d
    cos, sin = rope_tables(d, 1e6, 256)
    cos, sin = cos.cuda(), sin.cuda()
    # scattered pages for request 1
    table = torch.zeros(2, max_blocks, dtype=torch.int32)
    pages = [5, 9, 2, 17, 30]
    table[1, :5] = torch.tensor(pages, dtype=torch.int32)
    table = table.cuda()
    dt = torch.int8 if kv_int8 else torch.bfloat16
    kc = torch.zeros(num_pages, n_kv, 16, d, dtype=dt, device="cuda")
    vc = torch.zeros_like(kc)
    ks = torch.zeros(num_pages, n_kv, 16, device="cuda") if kv_int8 else None
    vs = torch.zeros(num_pages, n_kv, 16, device="cuda") if kv_int8 else None
    all_qkv = torch.randn(ctx, qkv_dim)
    q_out = torch.zeros(64, n_q * d, dtype=torch.bfloat16, device="cuda")
    # append in chunks of up to 64 rows, 2 split-K slices each
    for c0 in range(0, ctx, 64):
        rows = list(range(c0, min(ctx, c0 + 64)))
        sl = torch.stack([all_qkv[rows] * 0.25, all_qkv[rows] * 0.75]).cuda().contiguous()
        ctrl = _ctrl([(1, p, 0) for p in rows])
        k_.rope_append(sl, len(rows) * qkv_dim, 2, len(rows), ctrl, table, max_blocks, cos, sin, n_q, n_kv, d,
                       q_out, kc, vc, ks, vs, kv_int8)
    torch.cuda.synchronize()
    pos = torch.arange(ctx)
    q_ref = apply_rope(all_qkv[:, : n_q * d].reshape(ctx, n_q, d), pos, 1e6)
    k_ref = apply_rope(all_qkv[:, n_q * d: (n_q + n_kv) * d].reshape(ctx, n_kv, d), pos, 1e6)
    v_ref = all_qkv[:, (n_q + n_kv) * d:].reshape(ctx, n_kv, d)
    # cache contents
    def gather(cache, scale):
        out = torch.zeros(ctx, n_kv, d)
        for p in range(ctx):
            pg = pages[p // 16]
            row = cache[pg, :, p % 16, :].float().cpu()
            if scale is not None:
                row = row * scale[pg, :, p % 16].cpu()[:, None]
            out[p] = row
        return out
    tol = 0.02 if kv_int8 else 0.01
    assert (gather(kc, ks) - k_ref).abs().max() < tol * k_ref.abs().max()
    assert (gather(vc, vs) - v_ref).abs().max() < tol * v_ref.abs().max()
    # attention for the last m rows (their q was written by the last rope_append call)
    last_rows = list(range(ctx - m, ctx))
    nrows_last = ctx - (ctx - 1) // 64 * 64
    qsel = q_out[nrows_last - m: nrows_last].contiguous()
    assert (qsel.float().cpu().reshape(m, n_q, d) - q_ref[last_rows]).abs().max() < 0.02 * q_ref.abs().max()
    ctrl = _ctrl([(1, p, 0) for p in last_rows])
    nsplit = 4
    o_part = torch.zeros(m * n_q * nsplit * d, device="cuda")
    ml = torch.zeros(m * n_q * nsplit * 2, device="cuda")
    out = torch.zeros(m, n_q * d, dtype=torch.bfloat16, device="cuda")
    k_.attn_decode(qsel, kc, vc, table, ctrl, o_part, ml, out, m, n_q, n_kv, d, nsplit, max_blocks,
                   1.0 / math.sqrt(d), ks, vs, kv_int8)
    torch.cuda.synchronize()
    k_.check_status()
    g = n_q // n_kv
    kk = k_ref.repeat_interleave(g, dim=1)
    vv = v_ref.repeat_interleave(g, dim=1)
    ref = torch.zeros(m, n_q, d)
    for i, p in enumerate(last_rows):
        sc = torch.einsum("hd,shd->hs", q_ref[p], kk[: p + 1]) / math.sqrt(d)
        ref[i] = torch.einsum("hs,shd->hd", torch.softmax(sc, -1), vv[: p + 1])
    got = out.float().cpu().reshape(m, n_q, d)
    assert (got - ref).abs().max() < (0.04 if kv_int8 else 0.02) * ref.abs().max() + 1e-3


def test_head_logits_do_not_depend_on_the_rows_that_share_the_pass():
    """A row's logits are the same bits alone, among 8 rows and among 19 (two passes): verify rows reproduce
    single-row decoding through near-ties."""
    k_ = K()
    torch.manual_seed(21)
    n, kdim = 1500, 1024
    w = (torch.randn(n, kdim) * 0.05).to(torch.bfloat16).cuda()
    x = torch.randn(19, kdim).to(torch.bfloat16).cuda()
    ncand = k_.head_ncand(n)
    outs = {}
    for m in (1, 8, 19):
        out = torch.zeros(m, n, device="cuda")
        cv = torch.zeros(m * ncand, device="cuda")
        ci = torch.zeros(m * ncand, dtype=torch.int32, device="cuda")
        k_.head_gemv(w, x[:m].contiguous(), out, m, n, kdim, cv, ci)
        outs[m] = out
    torch.cuda.synchronize()
    k_.check_status()
    assert torch.equal(outs[1][0], outs[8][0]) and torch.equal(outs[8], outs[19][:8])
    ref = x.float() @ w.float().t()
    assert (outs[19] - ref).abs().max() < 2e-3 * ref.abs().max()


@pytest.mark.parametrize("int8,m", [(False, 6), (True, 6), (False, 1), (False, 16), (False, 19)])
def test_head_gemv_and_argmax(int8, m):
    k_ = K()
    torch.manual_seed(9)
    n, kdim = 1000, 512
    w = (torch.randn(n, kdim) * 0.05).to(torch.bfloat16)
    x = torch.randn(m, kdim).to(torch.bfloat16)
    # force a tie between ids 17 and 600 on row 0: identical weight rows
    w[600] = w[17]
    ncand = k_.head_ncand(n)
    out = torch.zeros(m, n, device="cuda")
    cv = torch.zeros(m * ncand, device="cuda")
    ci = torch.zeros(m * ncand, dtype=torch.int32, device="cuda")
    if int8:
        sc = w.float().abs().amax(1) / 127
        w8 = torch.round(w.float() / sc[:, None]).to(torch.int8)
        k_.head_gemv(w8.cuda(), x.cuda(), out, m, n, kdim, cv, ci, wscale=sc.cuda())
        ref = x.float() @ (w8.float() * sc[:, None]).t()
    else:
        k_.head_gemv(w.cuda(), x.cuda(), out, m, n, kdim, cv, ci)
        ref = x.float() @ w.float().t()
    ctrl = _ctrl([(0, 10 + i, 0) for i in range(m)])
    k_.argmax_finish(cv, ci, ncand, m, ctrl, True)
    torch.cuda.synchronize()
    k_.check_status()
    got = out.cpu()
    assert (got - ref).abs().max() < 2e-3 * ref.abs().max()
    c = ctrl.cpu()
    toks = c[k_.CTRL_OUT_TOKEN: k_.CTRL_OUT_TOKEN + m]
    # device arg-max of its own logits, ties to the lower id
    mx = got.max(dim=1, keepdim=True).values
    idx = torch.where(got == mx, torch.arange(n)[None, :], torch.tensor(n)).min(dim=1).values
    assert toks.tolist() == idx.tolist()
    assert got[0, 17] == got[0, 600]
    assert c[k_.CTRL_CUR_TOKEN: k_.CTRL_CUR_TOKEN + m].tolist() == idx.tolist()
    assert c[k_.CTRL_ROW_POS: k_.CTRL_ROW_POS + m].tolist() == [11 + i for i in range(m)]


def test_attn_decode_fused_merge_equals_separate_merge():
    k_ = K()
    torch.manual_seed(21)
    n_q, n_kv, d, ctx, m, nsplit = 40, 8, 128, 1500, 2, 16
    max_blocks = (ctx + 15) // 16 + 1
    num_pages = max_blocks + 2
    table = torch.zeros(1, max_blocks, dtype=torch.int32)
    table[0, : max_blocks - 1] = torch.randperm(num_pages - 1)[: max_blocks - 1].to(torch.int32) + 1
    table = table.cuda()
    kc = (torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    q = torch.randn(m, n_q * d, device="cuda").to(torch.bfloat16)
    ctrl = _ctrl([(0, ctx - m + i, 0) for i in range(m)])
    o_part = torch.zeros(m * n_q * nsplit * d, device="cuda")
    ml = torch.zeros(m * n_q * nsplit * 2, device="cuda")
    ref = torch.zeros(m, n_q * d, dtype=torch.bfloat16, device="cuda")
    k_.attn_decode(q, kc, vc, table, ctrl, o_part, ml, ref, m, n_q, n_kv, d, nsplit, max_blocks, d ** -0.5)
    tickets = torch.zeros(m * n_kv, dtype=torch.int32, device="cuda")
    for _ in range(3):          # the counters return to zero by themselves
        out = torch.full_like(ref, float("nan"))
        k_.attn_decode(q, kc, vc, table, ctrl, o_part, ml, out, m, n_q, n_kv, d, nsplit, max_blocks, d ** -0.5,
                       tickets=tickets)
        torch.cuda.synchronize()
        # same sums, different association of the final division: equal to rounding
        assert (out.float() - ref.float()).abs().max() <= 2e-2 * ref.float().abs().max()
        assert int(tickets.abs().sum()) == 0
    k_.check_status()


@pytest.mark.parametrize("m", [1, 5, 20])
def test_gemv_fused_fold_and_norm(m):
    """o-projection style GEMV that folds into the residual, then a GEMV that normalises while staging."""
    k_ = K()
    torch.manual_seed(31 + m)
    h, kin, n2 = 1024, 512, 768
    w1 = torch.randn(h, kin) * 0.02
    q1, s1 = Q.quantize_rtn(w1)
    w2 = torch.randn(n2, h) * 0.02
    q2, s2 = Q.quantize_rtn(w2)
    a = torch.randn(m, kin).to(torch.bfloat16)
    resid = torch.randn(m, h).to(torch.bfloat16)
    nw = (1 + 0.1 * torch.randn(h))
    sp1, sp2 = k_.gemv_splits(h, kin), k_.gemv_splits(n2, h)
    part1 = torch.zeros(sp1, m, h, device="cuda")
    tickets = torch.zeros(h // 128, dtype=torch.int32, device="cuda")
    ssq = torch.zeros(m, h // 128, device="cuda")
    r_dev = resid.cuda().clone()
    for rep in range(2):        # tickets reset themselves; the second pass folds again on top
        k_.gemv_w4_fused(Q.to_w4b(q1, s1).cuda(), a.cuda(), part1, m, h, kin, sp1, fold_tickets=tickets,
                         fold_resid=r_dev, fold_ssq=ssq)
    torch.cuda.synchronize()
    y = a.float() @ Q.dequant(q1, s1).t()
    r1 = (resid.float() + y).to(torch.bfloat16)
    r2 = (r1.float() + y).to(torch.bfloat16)
    assert (r_dev.float().cpu() - r2.float()).abs().max() <= 0.02 * r2.float().abs().max()
    got_ssq = ssq.sum(1).cpu()
    assert torch.allclose(got_ssq, r_dev.float().cpu().pow(2).sum(1), rtol=1e-4)
    assert int(tickets.abs().sum()) == 0
    part2 = torch.zeros(sp2, m, n2, device="cuda")
    k_.gemv_w4_fused(Q.to_w4b(q2, s2).cuda(), r_dev, part2, m, n2, h, sp2, x_mode=2, norm_w=nw.cuda(), norm_ssq=ssq,
                     norm_eps=1e-6)
    torch.cuda.synchronize()
    k_.check_status()
    rf = r_dev.float().cpu()
    xn = (rf * torch.rsqrt(rf.pow(2).mean(-1, keepdim=True) + 1e-6) * nw).to(torch.bfloat16).float()
    ref = xn @ Q.dequant(q2, s2).t()
    assert (part2.sum(0).cpu() - ref).abs().max() <= 5e-3 * ref.abs().max() + 1e-4


@pytest.mark.gpu
@pytest.mark.parametrize("m", [3, 8, 20])
def test_prequantised_rows_give_the_same_bits_as_in_kernel_staging(m):
    """quant_x + x_mode 3 is the GEMV's own prologue run once per row: the partial sums must be bit-identical."""
    from b200serve.ops import lib as K
    from b200serve.utils import quant as Q
    torch.manual_seed(m)
    n, k = 384, 1024
    w4b = Q.random_w4b(n, k, "cuda", seed=3)
    x = (torch.randn(m, k, device="cuda") * 0.7).to(torch.bfloat16)
    s = K.gemv_splits(n, k)
    a = torch.zeros(s * m * n, dtype=torch.float32, device="cuda")
    b = torch.zeros_like(a)
    K.gemv_w4(w4b, x, a, m, n, k, s)
    xq = torch.zeros(m * (k // 64) * 128, dtype=torch.uint8, device="cuda")
    gs = torch.zeros(K.quant_slots(m) * (k // 64) * 2, dtype=torch.int32, device="cuda")   # 8 token slots per row tile
    K.quant_x(x, m, k, xq, gs)
    K.gemv_w4_fused(w4b, xq, b, m, n, k, s, x_mode=3, norm_ssq=gs)
    torch.cuda.synchronize()
    K.check_status()
    assert torch.equal(a, b)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,rows,ctx,nsplit", [(40, 8, [(0, 8)], 1500, 16), (16, 4, [(0, 3), (1, 1), (0, 2)], 700, 8),
                                                       (8, 2, [(0, 1)], 4096, 32), (5, 1, [(1, 8), (0, 5)], 333, 4),
                                                       (8, 2, [(0, 4), (1, 1)], 4000, 4)])   # 8 batches per split: prefetch path
def test_attn_rows_matches_per_row_kernel(n_q, n_kv, rows, ctx, nsplit):
    """The tensor-core multi-row kernel against the per-row kernel (itself checked against fp32): groups of
    consecutive rows of one request, several requests in one step, ragged contexts, several splits."""
    k_ = K()
    torch.manual_seed(ctx)
    d = 128
    max_blocks = (ctx + 15) // 16 + 2
    num_pages = 2 * max_blocks + 2
    table = torch.zeros(2, max_blocks, dtype=torch.int32)
    perm = torch.randperm(num_pages - 1) + 1
    table[0] = perm[:max_blocks].to(torch.int32)
    table[1] = perm[max_blocks: 2 * max_blocks].to(torch.int32)
    table = table.cuda()
    kc = (torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    vc = (torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5).to(torch.bfloat16)
    spec = []
    for req, n in rows:                      # each group's rows sit at consecutive positions ending at ctx - 1
        base = ctx - n - 7 * req
        spec += [(req, base + i, 0) for i in range(n)]
    m = len(spec)
    q = torch.randn(m, n_q * d, device="cuda").to(torch.bfloat16)
    ctrl = _ctrl(spec)
    o_part = torch.zeros(m * n_q * nsplit * d, device="cuda")
    ml = torch.zeros(m * n_q * nsplit * 2, device="cuda")
    ref = torch.zeros(m, n_q * d, dtype=torch.bfloat16, device="cuda")
    k_.attn_decode(q, kc, vc, table, ctrl, o_part, ml, ref, m, n_q, n_kv, d, nsplit, max_blocks, d ** -0.5)
    tickets = torch.zeros(m * n_kv, dtype=torch.int32, device="cuda")
    for rep in range(3):
        out = torch.full_like(ref, float("nan"))
        o_part.fill_(float("nan"))
        k_.attn_rows(q, kc, vc, table, ctrl, o_part, ml, out, tickets if rep < 2 else None, m, n_q, n_kv, d, nsplit,
                     max_blocks, d ** -0.5)
        torch.cuda.synchronize()
        k_.check_status()
        assert not torch.isnan(out.float()).any()
        err = (out.float() - ref.float()).abs().max()
        assert err <= 2e-2 * ref.float().abs().max() + 2e-3, float(err)
        assert int(tickets.abs().sum()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("window,fixed", [(40, False), (300, False), (300, True), (5000, False)])
def test_attn_rows_sliding_window_matches_fp32(window, fixed):
    """Sliding-window layers: every row attends to its last ``window`` positions; pages before the first row's
    window are not read.  Compared with an fp32 softmax over the gathered pages."""
    k_ = K()
    torch.manual_seed(window)
    n_q, n_kv, d, ctx, nsplit = 8, 2, 128, 1100, 6
    max_blocks = (ctx + 15) // 16 + 2
    num_pages = 2 * max_blocks + 2
    table = torch.zeros(2, max_blocks, dtype=torch.int32)
    perm = torch.randperm(num_pages - 1) + 1
    table[0] = perm[:max_blocks].to(torch.int32)
    table[1] = perm[max_blocks: 2 * max_blocks].to(torch.int32)
    kc = (torch.randn(num_pages, n_kv, 16, d) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(num_pages, n_kv, 16, d) * 0.5).to(torch.bfloat16)
    spec = [(0, ctx - 5 + i, 0) for i in range(5)] + [(1, 17, 0)] + [(1, 600 + i, 0) for i in range(3)]
    m = len(spec)
    q = torch.randn(m, n_q * d).to(torch.bfloat16)
    ref = torch.zeros(m, n_q, d)
    for i, (req, pos, _) in enumerate(spec):
        lo = max(0, pos + 1 - window)
        keys = torch.arange(lo, pos + 1)
        pg, sl = table[req][keys // 16].long(), keys % 16
        for h in range(n_q):
            kk, vv = kc[pg, h // (n_q // n_kv), sl].float(), vc[pg, h // (n_q // n_kv), sl].float()
            p = torch.softmax(kk @ q[i, h * d:(h + 1) * d].float() * d ** -0.5, dim=0)
            ref[i, h] = p @ vv
    ctrl = _ctrl(spec)
    o_part = torch.full((m * n_q * nsplit * d,), float("nan"), device="cuda")
    ml = torch.zeros(m * n_q * nsplit * 2, device="cuda")
    out = torch.full((m, n_q * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    k_.attn_rows(q.cuda(), kc.cuda(), vc.cuda(), table.cuda(), ctrl, o_part, ml, out, None, m, n_q, n_kv, d, nsplit,
                 max_blocks, d ** -0.5, span_pages=(max_blocks + nsplit - 1) // nsplit if fixed else 0, window=window)
    torch.cuda.synchronize()
    k_.check_status()
    err = (out.float().cpu().view(m, n_q, d) - ref).abs().max()
    assert not torch.isnan(out.float()).any()
    assert err <= 2e-2 * ref.abs().max() + 2e-3, float(err)


@pytest.mark.gpu
def test_attn_rows_int8_kv_matches_per_row_kernel():
    k_ = K()
    torch.manual_seed(77)
    n_q, n_kv, d, ctx, nsplit = 16, 4, 128, 900, 2      # 4 batches of keys per split: the prefetch path
    max_blocks = (ctx + 15) // 16 + 2
    num_pages = max_blocks + 2
    table = (torch.randperm(num_pages - 1)[:max_blocks] + 1).to(torch.int32).view(1, -1).cuda()
    kf = torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5
    vf = torch.randn(num_pages, n_kv, 16, d, device="cuda") * 0.5
    ks = (kf.abs().amax(dim=-1) / 127).contiguous()
    vs = (vf.abs().amax(dim=-1) / 127).contiguous()
    k8 = torch.round(kf / ks[..., None]).clamp(-127, 127).to(torch.int8).contiguous()
    v8 = torch.round(vf / vs[..., None]).clamp(-127, 127).to(torch.int8).contiguous()
    spec = [(0, ctx - 5 + i, 0) for i in range(5)]
    m = len(spec)
    q = torch.randn(m, n_q * d, device="cuda").to(torch.bfloat16)
    ctrl = _ctrl(spec)
    o_part = torch.zeros(m * n_q * nsplit * d, device="cuda")
    ml = torch.zeros(m * n_q * nsplit * 2, device="cuda")
    ref = torch.zeros(m, n_q * d, dtype=torch.bfloat16, device="cuda")
    k_.attn_decode(q, k8, v8, table, ctrl, o_part, ml, ref, m, n_q, n_kv, d, nsplit, max_blocks, d ** -0.5, ks, vs, True)
    out = torch.full_like(ref, float("nan"))
    k_.attn_rows(q, k8, v8, table, ctrl, o_part, ml, out, None, m, n_q, n_kv, d, nsplit, max_blocks, d ** -0.5,
                 k_scale=ks, v_scale=vs, kv_int8=True)
    torch.cuda.synchronize()
    k_.check_status()
    err = (out.float() - ref.float()).abs().max()
    assert err <= 2e-2 * ref.float().abs().max() + 2e-3, float(err)
    # the same rows launched as ONE request's group (a CTA column per group of rows instead of one per row): same bits
    out1 = torch.full_like(ref, float("nan"))
    k_.attn_rows(q, k8, v8, table, ctrl, o_part, ml, out1, None, m, n_q, n_kv, d, nsplit, max_blocks, d ** -0.5,
                 k_scale=ks, v_scale=vs, kv_int8=True, one_request=True)
    torch.cuda.synchronize()
    k_.check_status()
    assert torch.equal(out1, out)


@pytest.mark.gpu
def test_gdn_conv_and_step_match_fp32():
    """Gated delta-net kernels against the same recurrence in fp32 torch: several rows of two slots in one step
    (rows of a slot see each other's state), split-K partials folded by the convolution kernel."""
    import torch.nn.functional as F
    k_ = K()
    torch.manual_seed(11)
    n_k, n_v, dh, splits, slots = 2, 4, 128, 3, 3
    kd, vd = n_k * dh, n_v * dh
    cc, n = 2 * kd + vd, 2 * kd + 2 * vd + 2 * n_v
    spec = [(2, 5, 0), (2, 6, 0), (0, 9, 0), (2, 7, 0), (0, 10, 0)]
    m = len(spec)
    part = torch.randn(splits, m, n) * 0.7
    conv_w = torch.randn(cc, 4) * 0.5
    conv_state = torch.randn(slots, cc, 3)
    state = torch.randn(slots, n_v, dh, dh) * 0.1
    a_log, dt_bias, norm_w = torch.log(torch.rand(n_v) * 4 + 0.5), torch.randn(n_v) * 0.5, 1 + 0.1 * torch.randn(dh)
    eps = 1e-6
    # reference
    proj = part.sum(0)
    conv_r, st_r = conv_state.clone(), state.clone()
    ref = torch.zeros(m, vd)
    for i, (slot, _, _) in enumerate(spec):
        hist = torch.cat([conv_r[slot], proj[i, :cc, None]], dim=1)
        y = F.silu((hist * conv_w).sum(1))
        conv_r[slot] = hist[:, 1:]
        q, k, v = y[:kd].view(n_k, dh), y[kd:2 * kd].view(n_k, dh), y[2 * kd:].view(n_v, dh)
        z = proj[i, cc:cc + vd].view(n_v, dh)
        b, a = proj[i, cc + vd:cc + vd + n_v], proj[i, cc + vd + n_v:]
        q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dh ** -0.5
        k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        q, k = q.repeat_interleave(n_v // n_k, 0), k.repeat_interleave(n_v // n_k, 0)
        S = st_r[slot] * torch.exp(-torch.exp(a_log) * F.softplus(a + dt_bias))[:, None, None]
        delta = (v - torch.einsum("hij,hi->hj", S, k)) * torch.sigmoid(b)[:, None]
        S = S + torch.einsum("hi,hj->hij", k, delta)
        st_r[slot] = S
        o = torch.einsum("hij,hi->hj", S, q)
        ref[i] = (o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * norm_w * F.silu(z)).reshape(vd)
    # device
    ctrl = _ctrl(spec)
    d = lambda t: t.cuda().contiguous()
    act = torch.zeros(m, n, device="cuda")
    conv_d, st_d = d(conv_state), d(state)
    out = torch.zeros(m, vd, dtype=torch.bfloat16, device="cuda")
    k_.gdn_conv(d(part), splits, m, n, cc, ctrl, d(conv_w), conv_d, act)
    k_.gdn_step(act, m, n, n_k, n_v, dh, ctrl, d(a_log), d(dt_bias), d(norm_w), eps, st_d, out)
    torch.cuda.synchronize()
    k_.check_status()
    assert (conv_d.cpu() - conv_r).abs().max() < 1e-5
    assert (st_d.cpu() - st_r).abs().max() < 2e-3 * st_r.abs().max()
    assert (st_d.cpu()[1] - state[1]).abs().max() == 0          # a slot without rows keeps its state
    assert (out.float().cpu() - ref).abs().max() < 0.02 * ref.abs().max() + 1e-3
    # the prompt-chunk form (normalisation and gates in parallel over the rows, one scan, gated norm in parallel):
    # the same rows as ONE slot's chunk give what the step kernel gives for them
    ctrl1 = _ctrl([(1, i, 0) for i in range(m)])
    conv_a, conv_b, st_a, st_b = d(conv_state), d(conv_state), d(state), d(state)
    act_a, act_b = torch.zeros(m, n, device="cuda"), torch.zeros(m, n, device="cuda")
    out_a, out_b = torch.zeros_like(out), torch.zeros_like(out)
    k_.gdn_conv(d(part), splits, m, n, cc, ctrl1, d(conv_w), conv_a, act_a)
    k_.gdn_step(act_a, m, n, n_k, n_v, dh, ctrl1, d(a_log), d(dt_bias), d(norm_w), eps, st_a, out_a)
    k_.gdn_conv(d(part), splits, m, n, cc, None, d(conv_w), conv_b, act_b, slot=1)
    k_.gdn_chunk(act_b, m, n, n_k, n_v, dh, 1, d(a_log), d(dt_bias), d(norm_w), eps, st_b, out_b)
    torch.cuda.synchronize()
    k_.check_status()
    assert torch.equal(conv_a, conv_b)
    assert (st_a - st_b).abs().max() < 1e-4 * st_a.abs().max()
    assert (out_a.float() - out_b.float()).abs().max() < 0.01 * out_a.float().abs().max() + 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("m,seed", [(200, 3), (64, 4), (1000, 5)])
def test_gdn_chunked_scan_on_tensor_cores_matches_recurrence(m, seed):
    """The chunked (WY) form of the gated delta rule -- triangular solve per 64-row chunk, state walked chunk by chunk
    with tensor-core products -- against the row-by-row recurrence in float64 torch, and against the sequential scan
    kernel: read-out rows, final state; a partial last chunk and a non-zero starting state included."""
    import torch.nn.functional as F
    k_ = K()
    torch.manual_seed(seed)
    n_k, n_v, dh = 2, 4, 128
    kd, vd = n_k * dh, n_v * dh
    n = 2 * kd + 2 * vd + 2 * n_v
    dev = "cuda"
    act0 = torch.randn(m, n, device=dev) * 0.8          # what gdn_conv leaves: q | k | v | z | b | a
    act0[:, 2 * kd + 2 * vd + n_v:] = torch.randn(m, n_v, device=dev) * 1.5 - 1.0     # a: decay factors from ~0.3 to ~1
    state0 = torch.randn(2, n_v, dh, dh, device=dev) * 0.1
    a_log = torch.log(torch.rand(n_v, device=dev) * 2 + 0.2)
    dt_bias, norm_w = torch.randn(n_v, device=dev) * 0.5, 1 + 0.1 * torch.randn(dh, device=dev)
    eps = 1e-6
    # float64 reference, row by row
    f = act0.double()
    q, k = f[:, :kd].view(m, n_k, dh), f[:, kd:2 * kd].view(m, n_k, dh)
    v, z = f[:, 2 * kd:2 * kd + vd].view(m, n_v, dh), f[:, 2 * kd + vd:2 * kd + 2 * vd].view(m, n_v, dh)
    b, a = f[:, 2 * kd + 2 * vd:2 * kd + 2 * vd + n_v], f[:, 2 * kd + 2 * vd + n_v:]
    q = q * torch.rsqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dh ** -0.5
    k = k * torch.rsqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(n_v // n_k, 1), k.repeat_interleave(n_v // n_k, 1)
    decay = torch.exp(-torch.exp(a_log.double()) * F.softplus(a + dt_bias.double()))
    beta = torch.sigmoid(b)
    S = state0[1].double().clone()
    o_ref = torch.zeros(m, n_v, dh, dtype=torch.float64, device=dev)
    for i in range(m):
        S = S * decay[i][:, None, None]
        delta = (v[i] - torch.einsum("hij,hi->hj", S, k[i])) * beta[i][:, None]
        S = S + torch.einsum("hi,hj->hij", k[i], delta)
        o_ref[i] = torch.einsum("hij,hi->hj", S, q[i])
    ref = (o_ref * torch.rsqrt((o_ref * o_ref).mean(-1, keepdim=True) + eps) * norm_w.double() * F.silu(z)).reshape(m, vd)
    # the two kernels
    outs, states, raws = [], [], []
    for wy in (False, True):
        act, st = act0.clone(), state0.clone()
        out = torch.zeros(m, vd, dtype=torch.bfloat16, device=dev)
        if wy:
            ws = torch.zeros(((m + 63) // 64) * n_v * k_.gdn_wy_block_bytes(), dtype=torch.uint8, device=dev)
            k_.gdn_chunk_wy(act, m, n, n_k, n_v, dh, 1, a_log, dt_bias, norm_w, eps, st, out, ws)
        else:
            k_.gdn_chunk(act, m, n, n_k, n_v, dh, 1, a_log, dt_bias, norm_w, eps, st, out)
        torch.cuda.synchronize()
        k_.check_status()
        outs.append(out.float())
        states.append(st)
        raws.append(act[:, 2 * kd:2 * kd + vd].clone())
    o_scale = float(o_ref.abs().max())
    for name, raw, st, out in (("scan", raws[0], states[0], outs[0]), ("wy", raws[1], states[1], outs[1])):
        assert torch.equal(st[0], state0[0]), name                                  # the other slot is untouched
        e_o = float((raw.double().view(m, n_v, dh) - o_ref).abs().max())
        e_s = float((st[1].double() - S).abs().max())
        assert e_o < (2e-5 if name == "scan" else 4e-3) * o_scale + 1e-6, (name, e_o, o_scale)
        assert e_s < (2e-5 if name == "scan" else 4e-3) * float(S.abs().max()), (name, e_s)
        assert float((out.double() - ref).abs().max()) < 0.02 * float(ref.abs().max()) + 1e-3, name


@pytest.mark.parametrize("m,nsplit", [(4, 8), (13, 37)])
def test_attention_merge_writes_the_same_quantised_rows_as_the_quantiser(m, nsplit):
    """The merge's optional second output is quant_x of its own bf16 rows, bit for bit (limbs, scales, sums)."""
    k_ = K()
    torch.manual_seed(5 + m)
    n_q, d = 10, 128
    o_part = torch.randn(m * n_q * nsplit * d, device="cuda")
    ml = torch.empty(m * n_q * nsplit, 2, device="cuda")
    ml[:, 0] = torch.randn(m * n_q * nsplit, device="cuda") * 3
    ml[:, 1] = torch.rand(m * n_q * nsplit, device="cuda") + 0.5
    ml[5, 0] = float("-inf")                  # a split without keys
    kdim = n_q * d
    slots = k_.quant_slots(m)

    def bufs():
        return (torch.zeros(m * (kdim // 64) * 128, dtype=torch.uint8, device="cuda"),
                torch.zeros(slots * (kdim // 64) * 2, dtype=torch.int32, device="cuda"))
    out_a = torch.zeros(m, kdim, dtype=torch.bfloat16, device="cuda")
    out_b = torch.zeros_like(out_a)
    xq_a, gs_a = bufs()
    xq_b, gs_b = bufs()
    L, P, S = k_.lib(), k_._p, k_._stream
    assert L.b2_attn_merge(P(o_part), P(ml), P(out_a), m, n_q, nsplit, d, S()) == 0
    k_.quant_x(out_a, m, kdim, xq_a, gs_a)
    assert L.b2_attn_merge_quant(P(o_part), P(ml), P(out_b), m, n_q, nsplit, d, P(xq_b), P(gs_b), slots, S()) == 0
    torch.cuda.synchronize()
    k_.check_status()
    assert torch.equal(out_a, out_b)
    assert torch.equal(xq_a, xq_b)
    g_a = gs_a.view(kdim // 64, slots, 2)[:, :m]
    g_b = gs_b.view(kdim // 64, slots, 2)[:, :m]
    assert torch.equal(g_a, g_b)

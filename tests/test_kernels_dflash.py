"""The block drafter's candidate kernels against plain PyTorch / numpy references (GPU)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def D():
    from b200serve.ops import dflash
    return dflash


def K():
    from b200serve.ops import lib
    return lib


def _ref_topk(row, used, k, table=None, mult=1.0, cap=0.0):
    """Larger value first, equal values by the lower index, NaN never wins."""
    idx = [i for i in range(min(len(row), used)) if not math.isnan(row[i])]
    idx.sort(key=lambda i: (-row[i], i))
    out = []
    for i in idx[:k]:
        v = np.float32(row[i]) * np.float32(mult)
        if cap > 0:
            v = np.float32(cap) * np.tanh(v / np.float32(cap), dtype=np.float32)
        out.append((table[i] if table is not None else i, float(v)))
    while len(out) < k:
        out.append((D().NO_IDX, -math.inf))
    return out


@pytest.mark.parametrize("n,used,k,rows", [(151936, 151800, 16, 3), (4096, 4096, 16, 3), (1000, 7, 16, 3), (32768, 32768, 4, 3),
                                           (248320, 248320, 16, 15), (40000, 39000, 16, 70)])
def test_topk_order_ties_nan_and_padding(n, used, k, rows):
    torch.manual_seed(n + k)
    x = torch.randn(rows, n)
    x[0, 5] = x[0, 900 % n] = 7.5          # a tie at the top: the lower index first
    x[1, 3] = float("nan")
    x[2] = torch.round(x[2] * 2) / 2       # many ties
    cand = torch.zeros(rows, k, dtype=torch.int32, device="cuda")
    val = torch.zeros(rows, k, device="cuda")
    D().topk(x.cuda(), rows, n, used, k, cand, val)
    torch.cuda.synchronize()
    K().check_status()
    for r in range(rows):
        want = _ref_topk(x[r].tolist(), used, k)
        got = list(zip((cand[r].cpu().numpy().astype(np.int64) & 0x7FFFFFFF).tolist(), val[r].cpu().tolist()))
        assert [g[0] for g in got] == [w[0] for w in want], (r, got[:4], want[:4])
        for (gi, gv), (wi, wv) in zip(got, want):
            assert gv == wv or (math.isinf(wv) and math.isinf(gv))


def test_topk_through_a_draft_vocabulary_with_multiplier_and_softcap():
    torch.manual_seed(1)
    n, k = 32768, 16
    table = torch.sort(torch.randperm(150000)[:n]).values.to(torch.int32)
    x = torch.randn(2, n) * 3
    cand = torch.zeros(2, k, dtype=torch.int32, device="cuda")
    val = torch.zeros(2, k, device="cuda")
    D().topk(x.cuda(), 2, n, n, k, cand, val, id_table=table.cuda(), out_mult=0.5, softcap=2.0)
    torch.cuda.synchronize()
    for r in range(2):
        want = _ref_topk(x[r].tolist(), n, k, table.tolist(), 0.5, 2.0)
        assert cand[r].cpu().tolist() == [w[0] for w in want]
        assert np.allclose(val[r].cpu().numpy(), [w[1] for w in want], rtol=1e-5, atol=1e-6)


def test_rerank_scores_candidates_exactly_and_orders_them():
    torch.manual_seed(2)
    vocab, h, rows, c, k = 5000, 1024, 4, 64, 16
    head = (torch.randn(vocab, h) * 0.05).to(torch.bfloat16).cuda()
    x = torch.randn(rows, h).to(torch.bfloat16).cuda()
    ids = torch.stack([torch.randperm(vocab)[:c] for _ in range(rows)]).to(torch.int32)
    ids[1, 5] = D().NO_IDX           # an absent candidate
    ids[2, 7] = vocab + 10           # beyond the used head rows: never a candidate
    cand = torch.zeros(rows, k, dtype=torch.int32, device="cuda")
    val = torch.zeros(rows, k, device="cuda")
    D().rerank(head, x, rows, vocab, ids.cuda(), c, k, cand, val)
    torch.cuda.synchronize()
    K().check_status()
    ref = x.float() @ head.float().t()                        # [rows][vocab]
    for r in range(rows):
        valid = [int(i) for i in ids[r].tolist() if 0 <= i < vocab]
        order = sorted(valid, key=lambda i: (-float(ref[r, i]), i))[:k]
        got = cand[r].cpu().tolist()
        # the same candidates in the same order (a pair closer than fp32 summation noise may swap)
        for a, b in zip(got, order):
            assert a == b or abs(float(ref[r, a] - ref[r, b])) < 1e-4 * float(ref[r].abs().max())
        want_v = torch.tensor([float(ref[r, i]) for i in got])
        assert torch.allclose(val[r].cpu(), want_v, rtol=1e-4, atol=1e-5)


def test_select_argmax_and_keyed_gumbel_is_reproducible():
    torch.manual_seed(3)
    rows, k = 7, 16
    cand = torch.stack([torch.randperm(100000)[:k] for _ in range(rows)]).to(torch.int32)
    score = torch.randn(rows, k)
    score[0, 3] = score[0, 9] = 5.0                 # tie: the better-ranked candidate (lower index) wins
    cand[1, 4:] = D().NO_IDX                        # a short row
    ids = torch.zeros(rows, dtype=torch.int32, device="cuda")
    chosen = torch.zeros(rows, dtype=torch.int32, device="cuda")
    D().select(cand.cuda(), score.cuda(), rows, k, 0.0, 1234, ids, chosen, pos0=500)
    torch.cuda.synchronize()
    for r in range(rows):
        valid = [c for c in range(k) if int(cand[r, c]) != D().NO_IDX]
        want = min(valid, key=lambda c: (-float(score[r, c]), c))
        assert int(chosen[r]) == want and int(ids[r]) == int(cand[r, want])
    # temperature > 0: arg-max of score / T + noise(seed, position, id); the host twin predicts the pick
    T, seed, pos0 = 0.8, 99, 4096
    picks = []
    for _ in range(2):
        D().select(cand.cuda(), score.cuda(), rows, k, T, seed, ids, chosen, pos0=pos0)
        torch.cuda.synchronize()
        picks.append(chosen.cpu().tolist())
    assert picks[0] == picks[1]
    for r in range(rows):
        vals = []
        for c in range(k):
            if int(cand[r, c]) == D().NO_IDX:
                continue
            vals.append((float(np.float32(score[r, c]) / np.float32(T)) + D().gumbel_of(seed, pos0 + r, int(cand[r, c])), c))
        best = max(vals, key=lambda t: (t[0], -t[1]))
        second = sorted(vals, key=lambda t: -t[0])[1][0] if len(vals) > 1 else -1e9
        if best[0] - second > 1e-4:        # not a near-tie in fp32
            assert picks[0][r] == best[1]
    # another seed or another position moves the noise
    D().select(cand.cuda(), score.cuda() * 0, rows, k, 1.0, seed + 1, ids, chosen, pos0=pos0)
    torch.cuda.synchronize()
    other = chosen.cpu().tolist()
    D().select(cand.cuda(), score.cuda() * 0, rows, k, 1.0, seed, ids, chosen, pos0=pos0)
    torch.cuda.synchronize()
    assert other != chosen.cpu().tolist()


@pytest.mark.parametrize("causal_rows", [0, 2])
def test_block_rows_attend_to_the_whole_block(causal_rows):
    """Rows flagged as block rows (window = -1) see every position up to the block's last one; the rows before them stay
    causal -- against fp32 softmax attention with that mask."""
    k_ = K()
    torch.manual_seed(4)
    n_q, n_kv, d, rows, ctx0, nsplit = 8, 2, 128, 6, 70, 4
    gqa = n_q // n_kv
    pages = (ctx0 + rows + 15) // 16 + 1
    kc = (torch.randn(pages, n_kv, 16, d) * 0.5).to(torch.bfloat16).cuda()
    vc = (torch.randn(pages, n_kv, 16, d) * 0.5).to(torch.bfloat16).cuda()
    q = torch.randn(rows, n_q * d).to(torch.bfloat16).cuda()
    bt = torch.arange(pages, dtype=torch.int32).view(1, -1).cuda()
    ctrl = torch.zeros(k_.CTRL_WORDS, dtype=torch.int32)
    ctrl[k_.CTRL_N_ROWS] = rows
    for i in range(rows):
        ctrl[k_.CTRL_ROW_REQ + i], ctrl[k_.CTRL_ROW_POS + i] = 0, ctx0 + i
        ctrl[k_.CTRL_ROW_BLOCK + i] = 1 if i >= causal_rows else 0
    ctrl = ctrl.cuda()
    o_part = torch.zeros(rows * n_q * nsplit * d, device="cuda")
    ml = torch.zeros(rows * n_q * nsplit * 2, device="cuda")
    out = torch.zeros(rows, n_q * d, dtype=torch.bfloat16, device="cuda")
    k_.attn_rows(q, kc, vc, bt, ctrl, o_part, ml, out, None, rows, n_q, n_kv, d, nsplit, pages, d ** -0.5, window=-1)
    torch.cuda.synchronize()
    k_.check_status()
    total = ctx0 + rows
    kf = kc.float().permute(1, 0, 2, 3).reshape(n_kv, pages * 16, d)[:, :total]
    vf = vc.float().permute(1, 0, 2, 3).reshape(n_kv, pages * 16, d)[:, :total]
    qf = q.float().view(rows, n_q, d)
    seen = torch.tensor([total if i >= causal_rows else ctx0 + i + 1 for i in range(rows)], device="cuda")
    mask = torch.arange(total, device="cuda")[None, :] < seen[:, None]
    ref = torch.zeros(rows, n_q, d, device="cuda")
    for h in range(n_q):
        s = (qf[:, h] @ kf[h // gqa].t()) * d ** -0.5
        s = s.masked_fill(~mask, float("-inf"))
        ref[:, h] = torch.softmax(s, dim=-1) @ vf[h // gqa]
    assert (out.float().view(rows, n_q, d) - ref).abs().max() < 2e-2 * ref.abs().max() + 2e-3

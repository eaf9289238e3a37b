"""Int4 formats: GPTQ pack / unpack, W4B repack round trip, dequant equivalence."""
import torch

from b200serve.utils import quant as Q


def test_gptq_pack_roundtrip():
    g = torch.Generator().manual_seed(1)
    q = torch.randint(0, 16, (128, 24), generator=g, dtype=torch.uint8)
    qw = Q.pack_gptq(q)
    assert qw.dtype == torch.int32 and qw.shape == (16, 24)
    assert torch.equal(Q.unpack_gptq(qw), q)
    # nibble i of word (r, n) is k = 8 r + i
    w = int(qw[3, 5]) & 0xFFFFFFFF
    for i in range(8):
        assert (w >> (4 * i)) & 15 == int(q[8 * 3 + i, 5])


def test_qzeros_symmetric_constant():
    z = Q.make_qzeros(128, 64)
    assert z.shape == (2, 8) and (z == 0x77777777).all()


def test_rtn_quant_error_bound():
    g = torch.Generator().manual_seed(2)
    w = torch.randn(96, 256, generator=g) * 0.02
    q, s = Q.quantize_rtn(w)
    wd = Q.dequant(q, s)
    # error of round-to-nearest is at most half a step (fp16 scale rounding adds a little)
    step = s.float().repeat_interleave(64, dim=0).t()
    assert ((wd - w).abs() <= 0.5 * step * 1.01 + 1e-7).all()


def test_w4b_roundtrip_with_padding():
    g = torch.Generator().manual_seed(3)
    for n, k in ((200, 128), (128, 64), (384, 704)):
        w = torch.randn(n, k, generator=g) * 0.02
        q, s = Q.quantize_rtn(w)
        blk = Q.to_w4b(q, s)
        assert blk.shape == ((n + 127) // 128, k // 64, Q.BLOCK_BYTES)
        q2, s2 = Q.from_w4b(blk, n)
        assert torch.equal(q2, q) and torch.equal(s2, s)
        assert torch.equal(Q.dequant_w4b(blk, n), Q.dequant(q, s))


def test_w4b_nibble_positions_match_mma_fragment():
    """Word c of lane l in tile j must hold the rows / k the kernel's mask-and-shift expects."""
    k, n = 64, 128
    q = (torch.arange(k)[:, None] * 0 + torch.arange(n)[None, :]) % 16          # value = row % 16
    kq = (torch.arange(k)[:, None] % 16 + 0 * torch.arange(n)[None, :])         # value = k % 16
    s = torch.ones(1, n, dtype=torch.float16)
    brow = Q.to_w4b(q.to(torch.uint8), s)[0, 0, :4096].view(torch.int32).reshape(8, 32, 4)
    bk = Q.to_w4b(kq.to(torch.uint8), s)[0, 0, :4096].view(torch.int32).reshape(8, 32, 4)
    for j in (0, 5):
        for lane in (0, 7, 31):
            g_, t = lane // 4, lane % 4
            for c in range(4):
                wr = int(brow[j, lane, c]) & 0xFFFFFFFF
                wk = int(bk[j, lane, c]) & 0xFFFFFFFF
                row = 16 * j + g_ + 8 * (c & 1)
                assert all(((wr >> (4 * p)) & 15) == row % 16 for p in range(8))
                lo = wk & 0x0F0F0F0F              # a0 / a1 of the 32-k step: k = 4t + b
                hi = (wk >> 4) & 0x0F0F0F0F       # a2 / a3: k = 16 + 4t + b
                for b in range(4):
                    assert (lo >> (8 * b)) & 0xFF == (32 * (c >> 1) + 4 * t + b) % 16
                    assert (hi >> (8 * b)) & 0xFF == (32 * (c >> 1) + 16 + 4 * t + b) % 16


def test_random_w4b_statistics():
    r = Q.random_w4b(200, 256, "cpu", seed=0)
    w = Q.dequant_w4b(r, 200)
    assert w.shape == (200, 256)
    assert 0.015 < float(w.std()) < 0.025


def test_group128_expansion():
    s = torch.arange(6, dtype=torch.float16).reshape(2, 3)
    e = Q.expand_group128(s)
    assert e.shape == (4, 3) and torch.equal(e[0], e[1]) and torch.equal(e[2], e[3])

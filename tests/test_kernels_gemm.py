"""tcgen05 GEMMs against fp32 PyTorch references (GPU)."""
import pytest
import torch

from b200serve.utils import quant as Q

pytestmark = pytest.mark.gpu


def G():
    from b200serve.ops import gemm
    return gemm


def K():
    from b200serve.ops import lib
    return lib


def _rowwise_close(got, ref, cos_min=0.9995, tile=32, tile_tol=0.03):
    """Per-row cosine and per-32-column-piece error against the piece's own scale: a wrong piece of small values does
    not hide behind the tensor's largest element."""
    cos = torch.nn.functional.cosine_similarity(got.float(), ref.float(), dim=1)
    assert float(cos.min()) > cos_min, float(cos.min())
    m, n = ref.shape
    n32 = n // tile * tile
    g = got.float()[:, :n32].reshape(m, n32 // tile, tile)
    r = ref.float()[:, :n32].reshape(m, n32 // tile, tile)
    scale = r.abs().amax(dim=2).clamp_min(float(ref.abs().mean()))
    assert float(((g - r).abs().amax(dim=2) / scale).max()) < tile_tol


@pytest.mark.parametrize("m,n,k,bn", [(128, 256, 64, 256), (128, 128, 64, 128), (256, 512, 256, 256),
                                      (200, 384, 192, 128), (4096, 1024, 512, 256), (77, 264, 128, 0),
                                      (1000, 5120, 1024, 0)])
def test_gemm_bf16(m, n, k, bn):
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    G().gemm_bf16(a, b, c, bn=bn)
    torch.cuda.synchronize()
    K().check_status()
    ref = a.float() @ b.float().t()
    assert torch.isfinite(c.float()).all()
    assert (c.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    _rowwise_close(c, ref)      # every 32-column piece against its own scale, every row's direction


def test_gemm_bf16_epilogues():
    g = G()
    torch.manual_seed(3)
    m, n, k = 300, 512, 256
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    c32 = torch.zeros(m, n, device="cuda")
    g.gemm_bf16(a, b, c32, epi=g.EPI_F32)
    assert (c32 - ref).abs().max() <= 2e-3 * ref.abs().max()
    # SiLU(gate) * up with gate / up alternating in runs of 16 columns
    cs = torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda")
    g.gemm_bf16(a, b, cs, epi=g.EPI_SILU_MUL)
    v = ref.reshape(m, n // 32, 2, 16)
    want = (torch.nn.functional.silu(v[:, :, 0]) * v[:, :, 1]).reshape(m, n // 2)
    assert (cs.float() - want).abs().max() <= 1e-2 * want.abs().max() + 1e-3
    _rowwise_close(cs, want, tile=16, tile_tol=0.05)
    # residual add, in place
    r = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    want = (r.float() + ref)
    g.gemm_bf16(a, b, r, epi=g.EPI_RESID_ADD, resid=r)
    torch.cuda.synchronize()
    K().check_status()
    assert (r.float() - want).abs().max() <= 1e-2 * want.abs().max()
    _rowwise_close(r, want)


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (333, 640, 512), (2048, 1024, 1024)])
def test_gemm_i8(m, n, k):
    g = G()
    torch.manual_seed(m)
    a8 = torch.randint(-127, 128, (m, k), device="cuda", dtype=torch.int8)
    b8 = torch.randint(-127, 128, (n, k), device="cuda", dtype=torch.int8)
    sa = torch.rand(m, device="cuda") * 0.01 + 0.001
    sb = torch.rand(n, device="cuda") * 0.01 + 0.001
    c = torch.zeros(m, n, device="cuda")
    g.gemm_i8(a8, b8, sa, sb, c, epi=g.EPI_F32)
    torch.cuda.synchronize()
    K().check_status()
    ref = (a8.double() @ b8.double().t()) * sa.double()[:, None] * sb.double()[None, :]
    assert (c.double() - ref).abs().max() <= 1e-5 * ref.abs().max()


def test_dequant_w4b_matches_host():
    g = G()
    torch.manual_seed(5)
    n, k = 384, 256
    w = torch.randn(n, k) * 0.02
    q, s = Q.quantize_rtn(w)
    out = g.dequant_w4b(Q.to_w4b(q, s).cuda(), n, k)
    ref = Q.dequant(q, s).to(torch.bfloat16)
    assert torch.equal(out.cpu(), ref)


def test_quant_rows_i8():
    g = G()
    x = (torch.randn(50, 512, device="cuda") * 3).to(torch.bfloat16)
    q, s = g.quant_rows_i8(x)
    ref_s = x.float().abs().amax(1) / 127
    assert torch.allclose(s, ref_s, rtol=1e-6)
    assert (q.float() * s[:, None] - x.float()).abs().max() <= 0.51 * s.max()


def test_gemm_grouped():
    """Expert-sorted rows, a device table of 128-row blocks, per-expert weights."""
    g = G()
    torch.manual_seed(8)
    e, n, k = 4, 256, 128
    counts = [130, 0, 77, 256]
    b = (torch.randn(e, n, k, device="cuda") * 0.05).to(torch.bfloat16)
    # rows of each expert start on a 128-row boundary (padded layout)
    blk_e, blk_r0, blk_n = [], [], []
    row = 0
    for ex, cnt in enumerate(counts):
        for j in range(0, cnt, 128):
            blk_e.append(ex); blk_r0.append(row + j); blk_n.append(min(128, cnt - j))
        row += (cnt + 127) // 128 * 128
    total = row
    a = torch.randn(total, k, device="cuda").to(torch.bfloat16)
    c = torch.zeros(total, n, dtype=torch.bfloat16, device="cuda")
    max_blk = 16
    pad = lambda v: torch.tensor(v + [0] * (max_blk - len(v)), dtype=torch.int32, device="cuda")
    blocks = (pad(blk_e), pad(blk_r0), pad(blk_n), torch.tensor([len(blk_e)], dtype=torch.int32, device="cuda"), max_blk)
    g.gemm_grouped_bf16(a, b, c, blocks)
    torch.cuda.synchronize()
    K().check_status()
    for ex, r0, rn in zip(blk_e, blk_r0, blk_n):
        ref = a[r0:r0 + rn].float() @ b[ex].float().t()
        assert (c[r0:r0 + rn].float() - ref).abs().max() <= 1e-2 * ref.abs().max()
        _rowwise_close(c[r0:r0 + rn], ref)
    # rows beyond a block's valid count are not written
    assert (c[130:256] == 0).all()


@pytest.mark.parametrize("m,n,k,bn", [(128, 256, 64, 256), (128, 128, 128, 128), (300, 512, 256, 256),
                                      (200, 384, 192, 128), (4096, 1024, 512, 0), (77, 264, 128, 0),
                                      (1000, 5120, 1024, 0), (512, 1408, 512, 256)])
def test_gemm_w4_reads_int4_and_matches_the_dequantised_gemm(m, n, k, bn):
    """The GEMM that expands W4B blocks in shared memory against (a) the bf16 GEMM over the dequantised weight:
    the same bits, both accumulate the same bf16 operands in the same order; (b) fp32 matmul, per row and per piece."""
    g = G()
    torch.manual_seed(m + n + k)
    w4b = Q.random_w4b(n, k, "cuda", seed=n + k)
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    wb = g.dequant_w4b(w4b, n, k)
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    g.gemm_w4(a, w4b, n, k, c, bn=bn)
    c2 = torch.empty_like(c)
    g.gemm_bf16(a, wb, c2, bn=bn)
    torch.cuda.synchronize()
    K().check_status()
    assert torch.isfinite(c.float()).all()
    assert torch.equal(c, c2)
    _rowwise_close(c, a.float() @ wb.float().t())


def test_gemm_w4_epilogues_and_grouped_form():
    g = G()
    torch.manual_seed(9)
    m, n, k = 300, 512, 256
    w4b = Q.random_w4b(n, k, "cuda", seed=1)
    wb = g.dequant_w4b(w4b, n, k)
    a = torch.randn(m, k, device="cuda").to(torch.bfloat16)
    ref = a.float() @ wb.float().t()
    cs = torch.zeros(m, n // 2, dtype=torch.bfloat16, device="cuda")
    g.gemm_w4(a, w4b, n, k, cs, epi=g.EPI_SILU_MUL)
    v = ref.reshape(m, n // 32, 2, 16)
    _rowwise_close(cs, (torch.nn.functional.silu(v[:, :, 0]) * v[:, :, 1]).reshape(m, n // 2), tile=16, tile_tol=0.05)
    r = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    want = r.float() + ref
    g.gemm_w4(a, w4b, n, k, r, epi=g.EPI_RESID_ADD, resid=r)
    _rowwise_close(r, want)
    # grouped: three experts, blocks of uneven row counts, one launch
    e = 3
    ws = torch.stack([Q.random_w4b(n, k, "cuda", seed=10 + i) for i in range(e)])
    rows = [130, 0, 77]
    blk_e, blk_r0, blk_n, row = [], [], [], 0
    for ei, cnt in enumerate(rows):
        for b0 in range(0, cnt, 128):
            blk_e.append(ei); blk_r0.append(row + b0); blk_n.append(min(128, cnt - b0))
        row += (cnt + 127) // 128 * 128
    i32 = dict(dtype=torch.int32, device="cuda")
    blocks = (torch.tensor(blk_e, **i32), torch.tensor(blk_r0, **i32), torch.tensor(blk_n, **i32),
              torch.tensor([len(blk_e)], **i32), len(blk_e) + 2)
    xs = torch.randn(row, k, device="cuda").to(torch.bfloat16)
    y = torch.zeros(row, n, dtype=torch.bfloat16, device="cuda")
    g.gemm_w4(xs, ws, n, k, y, blocks=blocks, n_experts=e)
    torch.cuda.synchronize()
    K().check_status()
    for ei, r0, cnt in zip(blk_e, blk_r0, blk_n):
        wref = g.dequant_w4b(ws[ei], n, k).float()
        _rowwise_close(y[r0: r0 + cnt], xs[r0: r0 + cnt].float() @ wref.t())

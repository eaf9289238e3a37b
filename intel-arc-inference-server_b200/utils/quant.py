"""Int4 weight formats: the GPTQ checkpoint layout and the kernel ("W4B") layout.

Checkpoint layout (what the loader reads; the reference documents the same
contract in docs/02-formats.md:47-59 and docs/13-loader.md:95-166):

* ``qweight`` int32 ``[K/8][N]``; nibble ``i`` of word ``(r, n)`` is the stored
  value ``q`` of input channel ``k = 8 r + i``; the weight is ``(q - 8) * scale``.
* ``scales`` fp16 ``[K/64][N]`` (one per group of 64 input channels).
* ``qzeros`` int32 ``[K/64][N/8]``, every word ``0x77777777`` (symmetric).

Kernel layout "W4B" (what the sm_100a kernels stream): the matrix is cut in
blocks of 128 output rows x 64 input channels (one quantisation group).  A
block is ``4352`` bytes: ``4096`` bytes of nibbles followed by the block's 128
fp16 scales.  Blocks are stored ``[N/128][K/64]`` so a CTA that owns 128 output
rows reads one contiguous stream along K.  Inside a block the nibbles are
ordered for the A operand of the warp-level 8-bit ``mma.m16n8k32``: tile ``j``
(16 rows) owns 512 bytes, lane ``l`` owns 16 bytes = words ``c = 0..3``; with
``g = l / 4``, ``t = l % 4`` word ``c`` holds row ``16 j + g + 8 (c & 1)`` and the
32-k step ``c >> 1`` of the group.  Byte ``b`` of the word holds ``k = 32 (c >> 1) +
4 t + b`` in its low nibble and ``k + 16`` in its high nibble, so a mask with
``0x0F0F0F0F`` of the word and of the word shifted by 4 yields the operand
registers (unsigned bytes 0..15) directly.  The 16 scales of a tile are
stored as pairs ``(row g, row g + 8)`` so a lane reads its two scales as one
32-bit word: position ``2 (r % 8) + r / 8`` holds the scale of tile row ``r``.
"""
from __future__ import annotations

import torch

GROUP = 64
BLOCK_N = 128
BLOCK_BYTES = 4352
BLOCK_W_BYTES = 4096


def quantize_rtn(w: torch.Tensor, group: int = GROUP):
    """Round-to-nearest symmetric int4. ``w`` is ``[N][K]`` (out, in) fp32.

    Returns ``q`` uint8 ``[K][N]`` in 0..15 and ``scales`` fp16 ``[K/group][N]``.
    Same rule as the reference's host quantiser (loader/rtn.h:36-59): the scale
    of a group is max|w| / 7, values clamp to [-8, 7].
    """
    n, k = w.shape
    assert k % group == 0
    wg = w.float().t().reshape(k // group, group, n)
    amax = wg.abs().amax(dim=1)
    scale = (amax / 7.0).clamp_min(1e-8).half()
    q = torch.round(wg / scale.float().unsqueeze(1)).clamp_(-8, 7) + 8
    return q.reshape(k, n).to(torch.uint8), scale


def pack_gptq(q: torch.Tensor) -> torch.Tensor:
    """``q`` uint8 ``[K][N]`` -> qweight int32 ``[K/8][N]``."""
    k, n = q.shape
    q32 = q.to(torch.int64).reshape(k // 8, 8, n)
    word = torch.zeros(k // 8, n, dtype=torch.int64, device=q.device)
    for i in range(8):
        word |= q32[:, i, :] << (4 * i)
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word)
    return word.to(torch.int32)


def unpack_gptq(qweight: torch.Tensor) -> torch.Tensor:
    """qweight int32 ``[K/8][N]`` -> ``q`` uint8 ``[K][N]``."""
    r, n = qweight.shape
    w = qweight.to(torch.int64) & 0xFFFFFFFF
    out = torch.stack([(w >> (4 * i)) & 0xF for i in range(8)], dim=1)
    return out.reshape(r * 8, n).to(torch.uint8)


def make_qzeros(k: int, n: int, group: int = GROUP, device="cpu") -> torch.Tensor:
    return torch.full((k // group, n // 8), 0x77777777, dtype=torch.int32, device=device)


def dequant(q: torch.Tensor, scales: torch.Tensor, group: int = GROUP) -> torch.Tensor:
    """fp32 ``[N][K]`` weight from ``q`` ``[K][N]`` and ``scales`` ``[K/group][N]``."""
    k, n = q.shape
    s = scales.float().repeat_interleave(group, dim=0)
    return ((q.float() - 8.0) * s).t().contiguous()


def expand_group128(scales: torch.Tensor) -> torch.Tensor:
    """Group-128 scales ``[K/128][N]`` -> group-64 ``[K/64][N]`` (each row twice).

    The reference accepts g128 checkpoints the same way (loader/quant.h:33-200).
    """
    return scales.repeat_interleave(2, dim=0)


# Nibble position p (bits 4p .. 4p+3) of W4B word c of lane (g, t) holds row g + 8 (c & 1) and
# k = 32 (c >> 1) + 4 t + _NIB_KOFF[p]: the low nibbles of the word's four bytes are k 4t .. 4t+3 of
# the 32-k step, the high nibbles k 16+4t .. 16+4t+3 -- so ``w & 0x0F0F0F0F`` and
# ``(w >> 4) & 0x0F0F0F0F`` are the a0/a1 and a2/a3 registers of ``mma.m16n8k32`` (8-bit operands).
_NIB_KOFF = (0, 16, 1, 17, 2, 18, 3, 19)


def _scale_perm(device):
    """``perm[pos]`` = row (0..127) of the block whose scale is stored at position ``pos``."""
    pos = torch.arange(BLOCK_N, device=device)
    j, p_ = pos // 16, pos % 16
    return j * 16 + (p_ // 2) + 8 * (p_ % 2)


def to_w4b(q: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Repack ``q`` ``[K][N]``, ``scales`` ``[K/64][N]`` into W4B bytes.

    Returns uint8 ``[N/128][K/64][4352]``.  N is zero-padded to a multiple of 128
    (padded rows get q = 8, scale = 0, i.e. weight 0).
    """
    k, n = q.shape
    assert k % GROUP == 0
    npad = (n + BLOCK_N - 1) // BLOCK_N * BLOCK_N
    dev = q.device
    if npad != n:
        q = torch.cat([q, torch.full((k, npad - n), 8, dtype=q.dtype, device=dev)], dim=1)
        scales = torch.cat([scales, torch.zeros(scales.shape[0], npad - n, dtype=scales.dtype, device=dev)], dim=1)
    nb, kg = npad // BLOCK_N, k // GROUP
    # index tensors for one block: word (j, lane, c), nibble p -> (row, k)
    j = torch.arange(8, device=dev).view(8, 1, 1, 1)
    lane = torch.arange(32, device=dev).view(1, 32, 1, 1)
    c = torch.arange(4, device=dev).view(1, 1, 4, 1)
    p = torch.arange(8, device=dev).view(1, 1, 1, 8)
    g, t = lane // 4, lane % 4
    row = 16 * j + g + 8 * (c & 1) + 0 * p                      # [8,32,4,8]
    kk = 32 * (c >> 1) + 4 * t + torch.tensor(_NIB_KOFF, device=dev).view(1, 1, 1, 8) + 0 * j
    row = row.expand(8, 32, 4, 8).reshape(-1)
    kk = kk.expand(8, 32, 4, 8).reshape(-1)
    qb = q.reshape(kg, GROUP, nb, BLOCK_N).permute(2, 0, 1, 3)   # [nb][kg][64 k][128 n]
    nibs = qb[:, :, kk, row].to(torch.int32).reshape(nb, kg, 8 * 32 * 4, 8)
    lo = nibs[..., 0] | (nibs[..., 1] << 4) | (nibs[..., 2] << 8) | (nibs[..., 3] << 12)
    hi = nibs[..., 4] | (nibs[..., 5] << 4) | (nibs[..., 6] << 8) | (nibs[..., 7] << 12)
    wb = torch.stack([lo & 0xFF, lo >> 8, hi & 0xFF, hi >> 8], dim=-1).to(torch.uint8)
    wb = wb.reshape(nb, kg, BLOCK_W_BYTES)
    sb = scales.reshape(kg, nb, BLOCK_N).permute(1, 0, 2)[..., _scale_perm(dev)].contiguous().view(torch.uint8)
    sb = sb.reshape(nb, kg, BLOCK_N * 2)
    return torch.cat([wb, sb], dim=-1).contiguous()


def from_w4b(w4b: torch.Tensor, n: int):
    """Inverse of :func:`to_w4b` (used by tests and by the CPU fallback)."""
    nb, kg, _ = w4b.shape
    dev = w4b.device
    wb = w4b[..., :BLOCK_W_BYTES].reshape(nb, kg, 8 * 32 * 4, 4).to(torch.int32)
    lo = wb[..., 0] | (wb[..., 1] << 8)
    hi = wb[..., 2] | (wb[..., 3] << 8)
    nibs = torch.stack([lo & 15, (lo >> 4) & 15, (lo >> 8) & 15, (lo >> 12) & 15,
                        hi & 15, (hi >> 4) & 15, (hi >> 8) & 15, (hi >> 12) & 15], dim=-1)
    j = torch.arange(8, device=dev).view(8, 1, 1, 1)
    lane = torch.arange(32, device=dev).view(1, 32, 1, 1)
    c = torch.arange(4, device=dev).view(1, 1, 4, 1)
    g, t = lane // 4, lane % 4
    row = (16 * j + g + 8 * (c & 1)).expand(8, 32, 4, 8).reshape(-1)
    kk = 32 * (c >> 1) + 4 * t + torch.tensor(_NIB_KOFF, device=dev).view(1, 1, 1, 8) + 0 * j
    kk = kk.expand(8, 32, 4, 8).reshape(-1)
    qb = torch.zeros(nb, kg, GROUP, BLOCK_N, dtype=torch.uint8, device=dev)
    qb[:, :, kk, row] = nibs.reshape(nb, kg, -1).to(torch.uint8)
    q = qb.permute(1, 2, 0, 3).reshape(kg * GROUP, nb * BLOCK_N)[:, :n].contiguous()
    sb = w4b[..., BLOCK_W_BYTES:].contiguous().view(torch.float16).reshape(nb, kg, BLOCK_N)
    sb = sb[..., torch.argsort(_scale_perm(dev))]
    scales = sb.permute(1, 0, 2).reshape(kg, nb * BLOCK_N)[:, :n].contiguous()
    return q, scales


def random_w4b(n: int, k: int, device, seed: int, std: float = 0.02) -> torch.Tensor:
    """Random-init W4B weight made directly on ``device`` (no fp32 master copy).

    Nibbles are uniform in 0..15 (std of ``q-8`` is 4.61), scales are chosen so the
    dequantised weights have standard deviation ``std``; used for the full-size
    benchmark shapes where quantising an fp32 matrix would take minutes.
    """
    npad = (n + BLOCK_N - 1) // BLOCK_N * BLOCK_N
    nb, kg = npad // BLOCK_N, k // GROUP
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = torch.empty(nb, kg, BLOCK_BYTES, dtype=torch.uint8, device=device)
    out[..., :BLOCK_W_BYTES] = torch.randint(0, 256, (nb, kg, BLOCK_W_BYTES), dtype=torch.uint8,
                                             device=device, generator=gen)
    s = (std / 4.61) * (0.75 + 0.5 * torch.rand(nb, kg, BLOCK_N, device=device, generator=gen))
    out[..., BLOCK_W_BYTES:] = s.half().view(torch.uint8).reshape(nb, kg, BLOCK_N * 2)
    if npad != n:
        # padded rows: zero their scales
        sc = out[..., BLOCK_W_BYTES:].view(torch.float16).reshape(nb, kg, BLOCK_N)
        rows = (torch.arange(nb, device=device)[:, None] * BLOCK_N + _scale_perm(device)[None, :]).reshape(nb, 1, BLOCK_N)
        sc.masked_fill_(rows >= n, 0.0)
    return out


def dequant_w4b(w4b: torch.Tensor, n: int) -> torch.Tensor:
    """fp32 ``[N][K]`` weight of a W4B tensor."""
    q, s = from_w4b(w4b, n)
    return dequant(q, s)

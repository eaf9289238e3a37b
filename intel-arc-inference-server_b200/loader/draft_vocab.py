"""Reduced draft vocabulary: the draft head scores only V' of the V output ids.

A draft token only has to be a good guess; scoring 32k instead of 152k rows of the lm_head makes a draft pass
several times cheaper, and the verify step still scores the full vocabulary, so the output is unchanged.  The
rule for V' follows the reference's (src/loader/draft_vocab.h:52-96): the forced ids (added / special tokens and
the EOS ids) always belong; then the ids of a ranked list (most frequent first) in order; then the lowest ids,
until the size is reached.  The result is sorted, so equal logits resolve to the lower id as in the full head.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import torch


def build_draft_vocab(vocab: int, size: int, forced: Iterable[int] = (), ranked: Optional[Sequence[int]] = None) -> List[int]:
    if size <= 0 or size >= vocab:
        return list(range(vocab))
    chosen = []
    seen = set()

    def take(i: int):
        if 0 <= i < vocab and i not in seen and len(chosen) < size:
            seen.add(i)
            chosen.append(i)

    forced = sorted(set(int(i) for i in forced))
    if len(forced) > size:
        raise ValueError(f"draft vocabulary of {size} cannot hold the {len(forced)} forced ids")
    for i in forced:
        take(i)
    for i in (ranked or ()):
        take(int(i))
    i = 0
    while len(chosen) < size and i < vocab:
        take(i)
        i += 1
    return sorted(chosen)


def read_ranked_ids(path: str) -> List[int]:
    """One id per line (or whitespace-separated), most useful first; lines starting with # are skipped."""
    out: List[int] = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line or line.startswith("#"):
                continue
            out += [int(t) for t in line.replace(",", " ").split()]
    return out


def int8_rows(w: torch.Tensor, rows_per_pass: int = 16384):
    """``w`` [n][k] as (int8 rows, fp32 scale per row), symmetric, the row's largest magnitude at 127."""
    q = torch.empty(w.shape, dtype=torch.int8, device=w.device)
    sc = torch.empty(w.shape[0], dtype=torch.float32, device=w.device)
    for r0 in range(0, w.shape[0], rows_per_pass):
        wf = w[r0: r0 + rows_per_pass].float()
        s = wf.abs().amax(dim=1).clamp_min(1e-12) / 127.0
        q[r0: r0 + rows_per_pass] = torch.round(wf / s[:, None]).clamp_(-127, 127).to(torch.int8)
        sc[r0: r0 + rows_per_pass] = s
    return q.contiguous(), sc.contiguous()


class DraftVocab:
    """The gathered head rows and the map from a position in V' back to the token id."""

    def __init__(self, lm_head: torch.Tensor, ids: Sequence[int], int8: bool = False):
        """``int8``: keep the gathered rows as int8 with one scale per row -- a candidate head at half the bytes, whose
        best candidates a block drafter then scores exactly against the bf16 rows (the reference's candidate head is
        an int4 / 2-bit copy of its int8 head: src/loader/dflash_loader.h:24-75)."""
        self.ids = torch.as_tensor(list(ids), dtype=torch.int64, device=lm_head.device)
        self.head = lm_head.index_select(0, self.ids).contiguous()
        self.head_i8 = None
        self.exact_rows = not int8      # the logits of ``head`` are the target head's own
        if int8:
            self.head_i8 = int8_rows(self.head)
            self.head = None
        self.ids32 = self.ids.to(torch.int32)
        self.size = int(self.ids.numel())

    def to_token(self, pos: int) -> int:
        return int(self.ids[pos])

"""Speculative decoding with a learned draft head: MTP chain or DFlash-style block drafter.

Both heads read the trunk's hidden state: the input of position ``p`` is
``fc([norm_e(embed(x_p)) ‖ norm_h(h_{p-1})])`` followed by the head's own decoder layers (their KV
lives in extra layers of the engine's page pool, same block tables), the head's norm and the shared
lm_head -- the reference's MTP head (src/runtime/capture.cc build_draft / build_verify,
src/kernels/prefill/pf_mtp_front.cl) and its DFlash drafter (src/kernels/dflash/*.cl).

One iteration (``SpecAdapter.step`` then ``draft``):
  verify   the pending token and the drafts run as rows of one trunk step (M = k + 1);
  accept   the server applies the accept rule and truncates the rejected rows;
  catch-up the head runs the accepted positions with the trunk's TRUE hidden states, which fills
           its KV and yields the first new draft;
  draft    MTP: k - 1 more single rows chained on the head's own hidden state;
           DFlash: the remaining drafts are mask rows of the SAME forward pass (one block).
Rows the head wrote beyond the accepted length are overwritten by the next catch-up.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..models.config import dflash_drafter
from ..models.weights import MtpWeights, QLinear, _norm_weight, _rand_layer
from ..ops import dflash as DF
from ..ops import gemm as G
from ..ops import lib as K
from .engine import Engine, Row


def random_drafter(cfg, device, seed: int = 7, layers: int = 2) -> MtpWeights:
    """Random-init DFlash-shape drafter: ``layers`` W4A16 decoder layers at the trunk's width plus the front."""
    dcfg = dflash_drafter(cfg)
    h = cfg.hidden
    fc = QLinear.random(h, 2 * h, device, seed * 1000 + 777, 0.02)
    return MtpWeights(_norm_weight(h, device), _norm_weight(h, device), fc,
                      [_rand_layer(dcfg, device, seed * 1000 + 800 + i, False, 0.02) for i in range(layers)],
                      _norm_weight(h, device))


DF_CANDIDATES = 16      # candidates a block drafter's row keeps (the sparse q of the sampled accept rule)


def _rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps) * w


class DraftHead:
    def __init__(self, engine: Engine, head: MtpWeights, kind: str = "mtp", kv_layer0: Optional[int] = None,
                 mask_token: Optional[int] = None, draft_vocab=None):
        self.eng, self.head, self.kind = engine, head, kind
        self.dv = draft_vocab        # loader.draft_vocab.DraftVocab or None: score a subset of the lm_head
        if draft_vocab is not None:
            dev = engine.device
            nc = K.head_ncand(draft_vocab.size)
            self.dv_logits = torch.zeros(engine.max_rows, draft_vocab.size, dtype=torch.float32, device=dev)
            self.dv_cand_val = torch.zeros(engine.max_rows * nc, dtype=torch.float32, device=dev)
            self.dv_cand_idx = torch.zeros(engine.max_rows * nc, dtype=torch.int32, device=dev)
            self.dv_ncand = nc
        cfg = engine.cfg
        self.kv0 = cfg.n_layers if kv_layer0 is None else kv_layer0
        if engine.kv.n_layers < self.kv0 + len(head.layers):
            raise ValueError("the engine's KV cache has no layers for the draft head (extra_kv_layers)")
        if mask_token is None:
            mask_token = getattr(head, "mask_token", None)
        self.mask_token = cfg.vocab - 1 if mask_token is None else mask_token
        dev = engine.device
        self.xcat = torch.zeros(engine.max_rows, 2 * cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.hid_in = torch.zeros(engine.max_rows, cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.zero_rows = torch.zeros(engine.max_rows, cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.draft_list = torch.zeros(64, dtype=torch.int32, device=dev)     # arg-maxes of chained rows, in order
        self.draft_n = torch.zeros(1, dtype=torch.int64, device=dev)
        # block drafter: per row the 16 best candidates of the (draft-vocabulary) head, then the same candidates
        # re-scored exactly against the target's lm_head rows, best first; the pick among them
        nk = DF_CANDIDATES
        self.df_cand0 = torch.zeros(engine.max_rows, nk, dtype=torch.int32, device=dev)
        self.df_val0 = torch.zeros(engine.max_rows, nk, dtype=torch.float32, device=dev)
        self.df_cand = torch.zeros(engine.max_rows, nk, dtype=torch.int32, device=dev)
        self.df_val = torch.zeros(engine.max_rows, nk, dtype=torch.float32, device=dev)
        self.df_chosen = torch.zeros(engine.max_rows, dtype=torch.int32, device=dev)
        self.df_host = None          # pinned (candidates, scores) of the last pass, read on demand
        self.fused_layers = os.environ.get("B2_HEAD_FUSED", "1") == "1"    # 0: the head's layers walk unfused
        self.graphs = {}
        self.prev_last: Dict[int, torch.Tensor] = {}    # last hidden of the previous prompt chunk, per slot
        engine.on_chunk_hidden = self._ingest_chunk
        self.rows_run = 0

    # ------------------------------------------------------------------ decode-time rows (M <= max_rows)
    def _enqueue(self, n: int, chain: bool, block: bool = False):
        """The head's forward pass for ``n`` rows as device work only (no host read, so it can be captured): tokens
        and positions come from the control block, hidden inputs from ``hid_in``.  ``chain``: leave the control block
        and ``hid_in`` ready for ONE more row that follows the last one -- its token is this pass's arg-max, its
        hidden input this pass's own hidden state -- and append the arg-max to the device-side draft list."""
        eng, m, head = self.eng, self.eng.model, self.head
        cfg, b = eng.cfg, m.buf
        h = cfg.hidden
        K.draft_front(m.w.embed, eng.ctrl, cfg.vocab, self.hid_in, head.pre_norm_embed, head.pre_norm_hidden,
                      cfg.rms_eps, n, h, self.xcat, b.flag)
        dense = all(lw.gate_up is not None and lw.gdn is None for lw in head.layers)
        m.block_rows = block         # rows flagged in the control block attend to the whole block (no causal mask)
        try:
            if m.fused and dense and h % 128 == 0 and self.fused_layers:
                # the front's GEMV folds its split-K slices onto zero rows and leaves the rows' sums of squares: the
                # head's layers then run as the trunk's do (six launches each, tensor-parallel folds included); the
                # front itself is held whole by every rank
                b.resid[:n].copy_(self.zero_rows[:n])
                m._gemv_fused("head_fc", head.fc, self.xcat, n, fold=True, tp_fold=False)
                pend = m.layers_walk(head.layers, n, eng.ctrl, eng.block_table, eng.max_blocks, eng.kv,
                                     first_from_embed=False, kv_layer0=self.kv0, resid_ready=True)
            else:
                part, s = m._gemv("head_fc", head.fc, self.xcat, n)
                # residual stream of the head = the fc output (the split-K slices folded onto zero rows)
                K.resid_norm(1, n, h, head.norm, cfg.rms_eps, b.resid, None, resid_in=self.zero_rows, part=part,
                             part_slice=n * h, splits=s)
                pend = m.layers_walk(head.layers, n, eng.ctrl, eng.block_table, eng.max_blocks, eng.kv,
                                     first_from_embed=False, kv_layer0=self.kv0)
        finally:
            m.block_rows = False
        if self.kind == "dflash":
            return self._candidates(n, pend)
        if self.dv is None:
            m.head(n, pend, eng.ctrl, False, final_norm=head.norm)
        else:
            # reduced draft vocabulary: fold + norm as the head does, then only V' rows of the lm_head; the arg-max
            # is a position in V', mapped to a token id through the id table (on the device)
            K.resid_norm(1, n, h, head.norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, part=pend[0],
                         part_slice=n * h, splits=pend[1])
            K.head_gemv(self.dv.head, b.x, self.dv_logits, n, self.dv.size, h, self.dv_cand_val, self.dv_cand_idx)
            K.argmax_finish(self.dv_cand_val, self.dv_cand_idx, self.dv_ncand, n, eng.ctrl, False)
            out = eng.ctrl[K.CTRL_OUT_TOKEN: K.CTRL_OUT_TOKEN + n]
            out.copy_(torch.index_select(self.dv.ids32, 0, out.to(torch.int64)))
        if chain:
            c = eng.ctrl
            last = n - 1
            c[K.CTRL_CUR_TOKEN: K.CTRL_CUR_TOKEN + 1] = c[K.CTRL_OUT_TOKEN + last: K.CTRL_OUT_TOKEN + last + 1]
            c[K.CTRL_ROW_POS: K.CTRL_ROW_POS + 1] = c[K.CTRL_ROW_POS + last: K.CTRL_ROW_POS + last + 1] + 1
            c[K.CTRL_ROW_REQ: K.CTRL_ROW_REQ + 1] = c[K.CTRL_ROW_REQ + last: K.CTRL_ROW_REQ + last + 1]
            self.hid_in[0:1].copy_(b.resid[last: last + 1])
            self.draft_list.index_copy_(0, self.draft_n, c[K.CTRL_OUT_TOKEN + last: K.CTRL_OUT_TOKEN + last + 1])
            self.draft_n += 1

    def _candidates(self, n: int, pend):
        """A block drafter's head (src/kernels/dflash/df_topk.cl, df_candidate.cl, df_rerank.cl in the reference): fold +
        norm, logits of the draft vocabulary (or of the whole head), the 16 best per row, and -- when those logits are
        not the target's own bf16 head rows -- the same candidates scored exactly against them and put in order."""
        eng, m, head = self.eng, self.eng.model, self.head
        cfg, b = eng.cfg, m.buf
        h = cfg.hidden
        K.resid_norm(1, n, h, head.norm, cfg.rms_eps, b.resid, b.x, resid_in=b.resid, part=pend[0],
                     part_slice=n * h, splits=pend[1])
        exact = True
        if self.dv is not None:
            if self.dv.head_i8 is not None:
                w8, sc = self.dv.head_i8
                K.head_gemv(w8, b.x, self.dv_logits, n, self.dv.size, h, self.dv_cand_val, self.dv_cand_idx, wscale=sc)
            else:
                K.head_gemv(self.dv.head, b.x, self.dv_logits, n, self.dv.size, h, self.dv_cand_val, self.dv_cand_idx)
            DF.topk(self.dv_logits, n, self.dv.size, self.dv.size, DF_CANDIDATES, self.df_cand0, self.df_val0,
                    id_table=self.dv.ids32)
            exact = self.dv.exact_rows
        else:
            nv = m.head_rows
            if m.int8_head:
                w8, sc = m.w.lm_head_i8
                K.head_gemv(w8, b.x, b.logits, n, nv, h, b.cand_val, b.cand_idx, wscale=sc)
                exact = False
            else:
                K.head_gemv(m.w.lm_head, b.x, b.logits, n, nv, h, b.cand_val, b.cand_idx)
            DF.topk(b.logits, n, nv, nv, DF_CANDIDATES, self.df_cand0, self.df_val0)
        if m.tp is not None or m.nccl is not None:
            return          # a vocabulary slice per rank: the ranks' candidates are merged after the pass (_merge_ranks)
        if exact:
            self.df_cand[:n].copy_(self.df_cand0[:n])
            self.df_val[:n].copy_(self.df_val0[:n])
        else:
            DF.rerank(m.w.lm_head, b.x, n, m.head_rows, self.df_cand0, DF_CANDIDATES, DF_CANDIDATES, self.df_cand, self.df_val)

    def _merge_ranks(self, n: int):
        """Tensor parallelism: every rank holds the 16 best of its vocabulary slice; the ranks exchange them (one small
        all-gather) and each keeps the 16 best of all, larger score first and the lower id among equals -- the same
        list on every rank (the reference merges its two halves' candidates on the host:
        src/runtime/dflash/tp_dflash_drafter.h)."""
        import torch.distributed as dist
        m = self.eng.model
        world = m.tp.world if m.tp is not None else m.nccl[1]
        group = getattr(m.tp, "group", None) if m.tp is not None else m.nccl[2]
        off = m.vocab_offset if m.tp is not None else m.vocab_offset_nccl
        ids = self.df_cand0[:n].to(torch.int64)
        ids = torch.where(ids == DF.NO_IDX, ids, ids + off)
        mine = torch.stack([ids, self.df_val0[:n].view(torch.int32).to(torch.int64)], dim=0).contiguous()     # [2][n][16]
        every = torch.empty((world,) + tuple(mine.shape), dtype=torch.int64, device=mine.device)
        dist.all_gather_into_tensor(every, mine, group=group)
        all_ids = every[:, 0].permute(1, 0, 2).reshape(n, -1)
        all_val = every[:, 1].permute(1, 0, 2).reshape(n, -1).to(torch.int32).view(torch.float32)
        by_id = torch.sort(all_ids, dim=1, stable=True)
        val = torch.gather(all_val, 1, by_id.indices)
        by_val = torch.sort(val, dim=1, descending=True, stable=True)       # equal scores stay in id order
        self.df_val[:n].copy_(by_val.values[:, :DF_CANDIDATES])
        self.df_cand[:n].copy_(torch.gather(by_id.values, 1, by_val.indices)[:, :DF_CANDIDATES].to(torch.int32))

    def _pick(self, row0: int, n: int, temperature: float, seed: int):
        """One token per row out of its candidates into the control block's output words: the best one, or at a
        temperature the Gumbel-arg-max whose noise depends on (seed, position, token) only -- a draw from
        softmax(scores / T) over the candidates, the q of the sparse accept rule (src/kernels/dflash/df_select.cl)."""
        c = self.eng.ctrl
        DF.select(self.df_cand[row0:], self.df_val[row0:], n, DF_CANDIDATES, temperature, seed,
                  c[K.CTRL_OUT_TOKEN + row0:], self.df_chosen[row0:], ctrl=c[row0:])

    def _run(self, n: int, chain: bool, block: bool = False):
        """Replays (capturing it first) the head's pass for ``n`` rows; eager when the engine runs without graphs."""
        eng = self.eng
        if not eng.use_graphs:
            return self._enqueue(n, chain, block)
        key = (n, chain, block)
        g = self.graphs.get(key)
        if g is None:
            saved = (eng.ctrl.clone(), self.hid_in.clone(), self.draft_n.clone(), self.draft_list.clone())
            self._enqueue(n, chain, block)   # warm-up outside capture: function attributes, scratch allocation
            torch.cuda.current_stream().synchronize()
            for dst, src in zip((eng.ctrl, self.hid_in, self.draft_n, self.draft_list), saved):
                dst.copy_(src)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self._enqueue(n, chain, block)
            for dst, src in zip((eng.ctrl, self.hid_in, self.draft_n, self.draft_list), saved):
                dst.copy_(src)               # KV rows written by the warm-up and the capture are rewritten by the replay
            self.graphs[key] = g
        g.replay()

    def rows(self, rows: Sequence[Row], hidden: torch.Tensor, chain: int = -1, picks=None) -> List[int]:
        """Runs head rows (token, position) with ``hidden[i]`` = hidden state of the position before row i; the head's
        own hidden states stay in ``engine.model.buf.resid``.  ``chain`` < 0: returns each row's token.  ``chain``
        >= 0: the last row's arg-max is the first draft and ``chain`` more single rows follow ON THE DEVICE, each taking
        the arg-max and the hidden state of the row before it (the MTP chain); returns the ``chain + 1`` drafts.
        Either way the host reads the device once.  A block drafter picks each row's token among its candidates:
        ``picks`` lists (first row, rows, temperature, seed) per request (default: the best candidate of every row)."""
        eng = self.eng
        n = len(rows)
        upto: Dict[int, int] = {}
        for r in rows:
            upto[r.slot] = max(upto.get(r.slot, 0), r.pos + 1 + max(chain, 0))
        for slot, end in upto.items():
            eng._ensure_pages(slot, min(end, eng.max_len))
        eng._write_rows(rows)
        self.hid_in[:n].copy_(hidden[:n])
        if chain < 0:
            self._run(n, False, any(r.block for r in rows))
            if self.kind == "dflash":
                if eng.model.tp is not None or eng.model.nccl is not None:
                    self._merge_ranks(n)
                for row0, cnt, temperature, seed in (picks or [(0, n, 0.0, 0)]):
                    self._pick(row0, cnt, temperature, seed)
                self.df_host = None
            self.rows_run += n
            return eng._read_out(n)
        self.draft_n.zero_()
        self._run(n, True)
        for _ in range(chain):
            self._run(1, True)
        self.rows_run += n + chain
        drafts = self.draft_list[: chain + 1].tolist()      # the one read: it also orders the host after the passes
        eng.check_failed("draft")
        return [int(t) for t in drafts]

    def candidates(self, row0: int, n: int):
        """(ids [n][16], scores [n][16]) of rows ``row0 .. row0 + n - 1`` of the last block pass, on the host: the
        support and the logits of the q that ``picks`` drew from (absent candidates: id 0x7fffffff, score -inf)."""
        if self.df_host is None:
            self.df_host = (self.df_cand.cpu().numpy(), self.df_val.cpu().numpy())
        c, v = self.df_host
        return c[row0: row0 + n].astype(np.uint32), v[row0: row0 + n]

    # ------------------------------------------------------------------ prompt ingestion
    def _ingest_chunk(self, runner, slot: int, ids: Sequence[int], pos0: int, resid: torch.Tensor):
        """Fills the head's KV for a prompt chunk: position p takes (h_{p-1}, x_p)."""
        eng, cfg, head = self.eng, self.eng.cfg, self.head
        c, h = len(ids), cfg.hidden
        prev = self.prev_last.get(slot) if pos0 > 0 else None
        hid = torch.empty(c, h, dtype=torch.bfloat16, device=eng.device)
        hid[1:] = resid[: c - 1]
        hid[0] = prev if prev is not None else 0
        self.prev_last[slot] = resid[c - 1].clone()
        if runner is None or c <= eng.max_rows:
            b = eng.model.buf
            saved = b.logits[:c].clone() if c <= eng.max_rows else None   # the caller may still sample from these rows
            for c0 in range(0, c, eng.max_rows):
                part = list(ids[c0: c0 + eng.max_rows])
                self.rows([Row(slot, pos0 + c0 + i, int(t)) for i, t in enumerate(part)], hid[c0: c0 + len(part)])
            if saved is not None:
                b.logits[:c].copy_(saved)
            return
        # GEMM path: the runner's buffers are free again (its layers are done); residual rows are overwritten
        ids_dev = runner.ids_dev[:c]
        e = _rmsnorm(torch.index_select(eng.model.w.embed, 0, ids_dev), head.pre_norm_embed, cfg.rms_eps)
        hh = _rmsnorm(hid, head.pre_norm_hidden, cfg.rms_eps)
        xcat = torch.cat([e, hh], dim=1).to(torch.bfloat16)
        keep = resid[c - 1].clone()
        runner.linear(head.fc, xcat, resid, G.EPI_BF16)
        for i, lw in enumerate(head.layers):
            runner.layer(lw, self.kv0 + i, slot, c, pos0, resid, runner.x[:c])
        resid[c - 1].copy_(keep)          # the caller reads the trunk's last row afterwards

    def last_prompt_hidden(self, slot: int) -> torch.Tensor:
        return self.prev_last[slot]


class SpecAdapter:
    """EngineIface with ``draft``: wraps an ``EngineAdapter`` and a draft head."""

    def __init__(self, inner, spec: str = "mtp", spec_max: int = 3, draft_model=None, draft_vocab: int = 0,
                 draft_vocab_ids: Optional[str] = None, candidate_head_int8: bool = False):
        self.inner = inner
        self.e: Engine = inner.e
        self.spec, self.k_max = spec, spec_max
        if self.e.cfg.is_moe:
            # never validated: the one run of a draft head over a mixture-of-experts trunk ended in an illegal memory
            # access, so the combination is refused until its cause is found
            raise NotImplementedError("draft heads (--spec mtp / dflash) are not available for mixture-of-experts models; "
                                      "use --spec lookup or --spec off")
        w = self.e.model.w
        if spec == "mtp":
            if w.mtp is None:
                raise ValueError("--spec mtp needs a checkpoint with an MTP head")
            head, kind = w.mtp, "mtp"
        else:
            if isinstance(draft_model, str):      # a drafter snapshot (--draft-model); sliced under tensor parallelism
                from ..loader.loader import load_drafter
                tpw = self.e.model.tp
                draft_model = load_drafter(draft_model, self.e.device,
                                           tp=(tpw.rank, tpw.world) if tpw is not None else (0, 1))
            head = draft_model if isinstance(draft_model, MtpWeights) else random_drafter(self.e.cfg, self.e.device)
            kind = "dflash"
        dv = None
        sharded = self.e.model.tp is not None or self.e.model.nccl is not None
        if draft_vocab and draft_vocab < self.e.cfg.vocab and sharded:
            raise ValueError("a reduced draft vocabulary is not sliced for tensor parallelism")
        if draft_vocab and draft_vocab < self.e.cfg.vocab:
            from ..loader.draft_vocab import DraftVocab, build_draft_vocab, read_ranked_ids
            ranked = read_ranked_ids(draft_vocab_ids) if draft_vocab_ids else None
            dv = DraftVocab(w.lm_head, build_draft_vocab(self.e.cfg.vocab, draft_vocab, inner.eos_ids, ranked),
                            int8=candidate_head_int8 and kind == "dflash")
        self.head = DraftHead(self.e, head, kind, draft_vocab=dv)
        self.e.model.attn_fixed_spans = True     # verify rows must reproduce single-row decoding bit for bit
        self.e.graphs.clear()
        self.vocab_size, self.max_len, self.max_seqs, self.eos_ids = inner.vocab_size, inner.max_len, inner.max_seqs, inner.eos_ids
        self.hid: Dict[int, torch.Tensor] = {}     # hidden rows of the slot's last trunk step
        self.base: Dict[int, int] = {}             # position of its first row
        self.toks: Dict[int, List[int]] = {}       # its row tokens
        self.stats = {"drafted": 0, "iterations": 0}
        self.q: Dict[int, tuple] = {}              # sparse q of the last sampled block drafts, per slot

    # ---- pass-through
    def reset(self, slot):
        self.inner.reset(slot)
        self.hid.pop(slot, None)

    def length(self, slot): return self.inner.length(slot)
    def truncate(self, slot, length): self.inner.truncate(slot, length)
    def kv_form(self): return self.inner.kv_form()
    def logits(self, slot, row=0): return self.inner.logits(slot, row)

    def sample(self, *args, **kw):
        fn = getattr(self.inner, "sample", None)
        return fn(*args, **kw) if fn is not None else None

    def prefill(self, slot, ids):
        tok = self.inner.prefill(slot, ids)
        n = self.e.seq_len[slot]
        self.hid[slot] = self.head.last_prompt_hidden(slot).view(1, -1)
        self.base[slot] = n - 1
        self.toks[slot] = [int(ids[-1])]
        return tok

    def step(self, rows: Dict[int, List[int]]):
        bases = {slot: self.e.seq_len[slot] for slot in rows}
        out = self.inner.step(rows)
        resid = self.e.model.buf.resid
        for slot, span in self.inner._rows_of.items():
            self.hid[slot] = resid[span.start: span.stop].clone()
            self.base[slot] = bases[slot]
            self.toks[slot] = list(rows[slot])
        return out

    # ---- drafting
    def _plan(self, slot: int, pending: int, k: int):
        """The head rows that catch up with the accepted positions of ``slot`` and the hidden state each one takes."""
        if k <= 0 or slot not in self.hid:
            return None
        k = min(k, self.k_max, self.e.max_len - self.e.seq_len[slot] - 2)
        if k <= 0:
            return None
        length = self.e.seq_len[slot]
        base, hid, toks = self.base[slot], self.hid[slot], self.toks[slot]
        r = length - base                       # trunk rows that were kept: positions base .. length - 1
        if r < 1 or r > hid.shape[0]:
            return None
        # catch-up rows: position base + 1 + j takes the hidden state of position base + j
        row_toks = [toks[j + 1] for j in range(r - 1)] + [int(pending)]
        rows = [Row(slot, base + 1 + j, t) for j, t in enumerate(row_toks)]
        return k, r, rows, hid[:r]

    def draft(self, slot: int, pending: int, k: int, temperature: float = 0.0, seed: int = 0) -> List[int]:
        """Up to ``k`` draft tokens that follow ``pending`` (the token at position ``length(slot)``).  A block drafter
        at a ``temperature`` draws each draft from softmax(scores / T) over the row's candidates (``draft_q``)."""
        return self.draft_many({slot: (pending, k, temperature, seed)}).get(slot, [])

    def draft_many(self, reqs: Dict[int, tuple]) -> Dict[int, List[int]]:
        """Drafts for several slots: ``reqs[slot] = (pending, k[, temperature, seed])``.  The block drafter serves all
        of them in passes of up to ``max_rows`` rows (a request's rows form a group of the attention kernel, its block
        rows -- the pending token and the mask rows -- see one another); the MTP chain runs slot by slot."""
        out: Dict[int, List[int]] = {}
        self.q = {}
        if self.head.kind != "dflash":
            for slot, rq in reqs.items():
                plan = self._plan(slot, rq[0], rq[1])
                if plan is None:
                    continue
                k, r, rows, hidden = plan
                saved_len = self.e.seq_len[slot]
                # the catch-up rows, then k - 1 rows chained on the device (token and hidden state of the row before)
                out[slot] = self.head.rows(rows, hidden, chain=k - 1)
                self.e.seq_len[slot] = saved_len        # the head's rows are not part of the sequence
                self.stats["drafted"] += len(out[slot])
                self.stats["iterations"] += 1
            return out
        batch, used = [], 0

        def flush():
            nonlocal batch, used
            if not batch:
                return
            rows = [x for b in batch for x in b[2]]
            hidden = torch.cat([b[3] for b in batch], dim=0)
            picks, row0 = [], 0
            for slot, r, rws, _, temperature, seed in batch:
                picks.append((row0 + r - 1, len(rws) - r + 1, temperature, seed))
                row0 += len(rws)
            saved = {b[0]: self.e.seq_len[b[0]] for b in batch}
            toks = self.head.rows(rows, hidden, picks=picks)
            sampled = any(b[4] > 0 for b in batch)
            row0 = 0
            for slot, r, rws, _, temperature, seed in batch:
                out[slot] = [int(t) for t in toks[row0 + r - 1: row0 + len(rws)]]
                if sampled and temperature > 0:
                    self.q[slot] = self.head.candidates(row0 + r - 1, len(rws) - r + 1)
                self.e.seq_len[slot] = saved[slot]
                self.stats["drafted"] += len(out[slot])
                self.stats["iterations"] += 1
                row0 += len(rws)
            batch, used = [], 0

        for slot, rq in reqs.items():
            plan = self._plan(slot, rq[0], rq[1])
            if plan is None:
                continue
            k, r, rows, hidden = plan
            temperature, seed = (rq[2], rq[3]) if len(rq) >= 4 else (0.0, 0)
            extra = max(0, min(k - 1, self.e.max_rows - r))
            if used + r + extra > self.e.max_rows:
                flush()
            length = self.e.seq_len[slot]
            rows[-1].block = 1 if extra else 0          # the block: the pending token's row and the mask rows
            rows = rows + [Row(slot, length + 1 + j, self.head.mask_token, 1) for j in range(extra)]
            if extra:
                hidden = torch.cat([hidden, hidden[r - 1: r].expand(extra, -1)], dim=0)
            batch.append((slot, r, rows, hidden, float(temperature), int(seed)))
            used += len(rows)
        flush()
        return out

    def draft_q(self, slot: int):
        """(candidate ids [k][16], scores [k][16]) the last sampled drafts of ``slot`` were drawn from, or None."""
        return self.q.get(slot)

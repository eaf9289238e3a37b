"""Checkpoint loader: HF safetensors (GPTQ / AutoRound W4A16, group 64) -> ``ModelWeights``.

Steps, as in the reference's loader (src/loader/loader.cc:308 load_linear, :460 load_small, :521
load_mtp, :954 load_impl; docs/13-loader.md): resolve the name view (``model.language_model.``
prefix stripped, ``model.visual.*`` skipped, ``mtp.*`` optional), check the quantisation config and
each linear's invariants, fuse (q‖k‖v concatenated, gate‖up interleaved in runs of 16), repack into
the kernel layout on the target device, convert norms to fp32, and cross-check the bytes a decode
step reads ("W") against the descriptor's arithmetic.  Tensor parallel: ``tp=(rank, world)`` takes
the rank's column slice of qkv / gate‖up / lm_head (whole heads, whole interleave runs) and its row
slice (input channels) of o / down straight from the checkpoint tensors (loader.cc:882-886).
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import Dict, List, Optional, Tuple

import torch

from ..models.config import ModelConfig
from ..models.weights import ExpertWeights, LayerWeights, ModelWeights, MtpWeights, QLinear, interleave16
from ..utils import quant as Q
from ..utils.safetensors_io import SafetensorsSet
from .quant_config import QuantConfig, QuantError, assert_quant_invariants
from .snapshot import resolve_snapshot


class NameView:
    """Checkpoint names as the loader sees them: wrapper prefixes stripped, vision towers skipped."""

    def __init__(self, st: SafetensorsSet, copy: bool = True):
        self.st = st
        self.copy = copy   # False when every tensor is moved to a device before the set is dropped
        self.map: Dict[str, str] = {}
        for n in st.names():
            v = n
            if v.startswith("model.visual.") or v.startswith("visual."):
                continue
            if v.startswith("model.language_model."):
                v = "model." + v[len("model.language_model."):]
            elif v.startswith("language_model."):
                v = v[len("language_model."):]
            self.map[v] = n

    def has(self, name):
        return name in self.map

    def get(self, name) -> torch.Tensor:
        if name not in self.map:
            raise KeyError(f"checkpoint has no tensor {name}")
        return self.st.get(self.map[name], self.copy)

    def shape(self, name):
        return self.st.shape(self.map[name])

    def dtype(self, name) -> str:
        return self.st.dtype(self.map[name])


class _LinearSrc:
    """One quantised (or bf16) linear of the checkpoint: ``q`` uint8 [K][N] + scales, or a dense weight."""

    def __init__(self, view: NameView, prefix: str, qc: QuantConfig):
        self.prefix = prefix
        if view.has(prefix + ".qweight"):
            qw = view.get(prefix + ".qweight")
            sc = view.get(prefix + ".scales")
            qz = view.get(prefix + ".qzeros") if view.has(prefix + ".qzeros") else None
            gi = view.get(prefix + ".g_idx") if view.has(prefix + ".g_idx") else None
            assert_quant_invariants(prefix, qw, sc, qz, gi, qc.group_size)
            self.q = Q.unpack_gptq(qw)                      # [K][N]
            self.scales = sc if qc.group_size == 64 else Q.expand_group128(sc)
            self.dense = None
        elif view.has(prefix + ".weight"):
            # an excluded module or an unquantised drafter (bf16, or int8 with one scale per output row): quantise on
            # the host (RTN)
            self.dense = view.get(prefix + ".weight").float()
            if view.has(prefix + ".weight_scale"):
                self.dense = self.dense * view.get(prefix + ".weight_scale").float().reshape(-1, 1)
            self.q, self.scales = Q.quantize_rtn(self.dense)
        else:
            raise KeyError(f"checkpoint has neither {prefix}.qweight nor {prefix}.weight")

    @property
    def n(self):
        return self.q.shape[1]

    @property
    def k(self):
        return self.q.shape[0]


def _cols(src: _LinearSrc, lo: int, hi: int):
    return src.q[:, lo:hi], src.scales[:, lo:hi]


def _fuse_cols(parts: List[Tuple[torch.Tensor, torch.Tensor]]):
    return torch.cat([p[0] for p in parts], dim=1), torch.cat([p[1] for p in parts], dim=1)


def _interleave_cols(gate, up):
    """Column-wise interleave16 of two (q, scales) pairs."""
    out = []
    for a, b in zip(gate, up):
        r, n = a.shape
        out.append(torch.stack([a.reshape(r, n // 16, 16), b.reshape(r, n // 16, 16)], dim=2).reshape(r, 2 * n))
    return out[0], out[1]


def _ql(q, scales, device) -> QLinear:
    return QLinear(Q.to_w4b(q.to(device), scales.to(device)), q.shape[1], q.shape[0])


def _load_layer(view: NameView, cfg: ModelConfig, prefix: str, qc: QuantConfig, device, tp) -> LayerWeights:
    rank, world = tp
    hd = cfg.head_dim
    if view.has(prefix + ".linear_attn.A_log"):
        return _load_gdn_layer(view, cfg, prefix, qc, device, tp)
    q_s = _LinearSrc(view, prefix + ".self_attn.q_proj", qc)
    k_s = _LinearSrc(view, prefix + ".self_attn.k_proj", qc)
    v_s = _LinearSrc(view, prefix + ".self_attn.v_proj", qc)
    o_s = _LinearSrc(view, prefix + ".self_attn.o_proj", qc)
    if cfg.n_kv_heads % world or cfg.n_q_heads % world:
        raise ValueError(f"tensor parallel {world} does not divide {cfg.n_q_heads} q / {cfg.n_kv_heads} kv heads")
    qh, kh = cfg.n_q_heads // world, cfg.n_kv_heads // world
    qkv = _fuse_cols([_cols(q_s, rank * qh * hd, (rank + 1) * qh * hd), _cols(k_s, rank * kh * hd, (rank + 1) * kh * hd),
                      _cols(v_s, rank * kh * hd, (rank + 1) * kh * hd)])
    # row-parallel o: this rank's input channels (its heads' outputs)
    o_rows = slice(rank * qh * hd, (rank + 1) * qh * hd)
    o_q, o_sc = o_s.q[o_rows], o_s.scales[o_rows.start // 64: o_rows.stop // 64]
    lw = LayerWeights(
        input_norm=view.get(prefix + ".input_layernorm.weight").float().to(device),
        post_norm=view.get(prefix + ".post_attention_layernorm.weight").float().to(device),
        qkv=_ql(*qkv, device), o=_ql(o_q, o_sc, device))
    _load_ffn(lw, view, cfg, prefix, qc, device, tp)
    return lw


def _load_gdn_layer(view: NameView, cfg: ModelConfig, prefix: str, qc: QuantConfig, device, tp) -> LayerWeights:
    """A gated delta-net layer: ``linear_attn.in_proj_qkvz`` (columns [ q | k | v | z ], heads in order) and the
    gate projection are fused into one projection; ``conv1d.weight`` is [channels][1][4].  The gate projection comes
    as one ``in_proj_ba`` ([ b | a ]) or as two tensors ``in_proj_b`` and ``in_proj_a``, int4 or unquantised (exports
    differ: some exclude a / b from quantisation, some quantise them like every other linear); an unquantised one is
    quantised on the host.  Every GDN layer of a checkpoint must use the form and the kind of the first one -- a later
    layer in the other form is refused by name (the reference's rule: src/loader/ab.h:13-21)."""
    from ..models.weights import GdnWeights
    if tp[1] != 1:
        raise ValueError("gated delta-net layers are not sliced for tensor parallelism")
    p = prefix + ".linear_attn"
    qkvz = _LinearSrc(view, p + ".in_proj_qkvz", qc)
    split = not (view.has(p + ".in_proj_ba.qweight") or view.has(p + ".in_proj_ba.weight"))
    first_name = p + (".in_proj_b" if split else ".in_proj_ba")
    form = ("split" if split else "fused", "int4" if view.has(first_name + ".qweight") else "dense")
    seen = getattr(view, "_gdn_gate_form", None)
    if seen is None:
        view._gdn_gate_form = (form, p)
    elif seen[0] != form:
        raise ValueError(f"{p}: gate projection is {form[0]} / {form[1]}, but {seen[1]} has it {seen[0][0]} / {seen[0][1]}: "
                         "a checkpoint keeps one form for all gated delta-net layers")
    if split:
        pb, pa = _LinearSrc(view, p + ".in_proj_b", qc), _LinearSrc(view, p + ".in_proj_a", qc)
        if pb.n != cfg.gdn_v_heads or pa.n != cfg.gdn_v_heads:
            raise ValueError(f"{p}: in_proj_b / in_proj_a have {pb.n} / {pa.n} columns, expected {cfg.gdn_v_heads} each")
        ba_cols = _fuse_cols([_cols(pb, 0, pb.n), _cols(pa, 0, pa.n)])
        ba_n = pb.n + pa.n
    else:
        ba = _LinearSrc(view, p + ".in_proj_ba", qc)
        ba_cols, ba_n = _cols(ba, 0, ba.n), ba.n
    if qkvz.n != 2 * cfg.gdn_key_dim + 2 * cfg.gdn_value_dim or ba_n != 2 * cfg.gdn_v_heads:
        raise ValueError(f"{p}: projection widths {qkvz.n} / {ba_n} do not match the configured heads")
    out = _LinearSrc(view, p + ".out_proj", qc)
    conv = view.get(p + ".conv1d.weight").float().reshape(cfg.gdn_conv_channels, 4)
    lw = LayerWeights(
        input_norm=view.get(prefix + ".input_layernorm.weight").float().to(device),
        post_norm=view.get(prefix + ".post_attention_layernorm.weight").float().to(device), qkv=None, o=None)
    lw.gdn = GdnWeights(
        in_proj=_ql(*_fuse_cols([_cols(qkvz, 0, qkvz.n), ba_cols]), device),
        conv_w=conv.contiguous().to(device), a_log=view.get(p + ".A_log").float().to(device),
        dt_bias=view.get(p + ".dt_bias").float().to(device), norm_w=view.get(p + ".norm.weight").float().to(device),
        out_proj=_ql(out.q, out.scales, device))
    _load_ffn(lw, view, cfg, prefix, qc, device, tp)
    return lw


def _load_ffn(lw: LayerWeights, view: NameView, cfg: ModelConfig, prefix: str, qc: QuantConfig, device, tp):
    rank, world = tp

    def has_linear(name):
        return view.has(name + ".qweight") or view.has(name + ".weight")

    def mlp(p, ffn, fused=None):
        """``fused``: the per-expert form the layer uses (decided from expert 0, required of every expert): separate
        ``gate_proj`` / ``up_proj``, or one ``gate_up_proj`` whose first half of output columns is gate (the
        reference reads both: src/loader/moe.h:29-57)."""
        is_fused = has_linear(f"{p}.gate_up_proj")
        if fused is not None and is_fused != fused:
            raise ValueError(f"{p}: mixed expert forms in one layer (gate_up_proj next to gate_proj / up_proj)")
        d = _LinearSrc(view, f"{p}.down_proj", qc)
        if is_fused:
            both = _LinearSrc(view, f"{p}.gate_up_proj", qc)
            if both.n != 2 * ffn:
                raise ValueError(f"{p}.gate_up_proj: {both.n} output columns, expected {2 * ffn}")
            g = u = None
            gc = lambda lo, hi: _cols(both, lo, hi)
            uc = lambda lo, hi: _cols(both, ffn + lo, ffn + hi)
        else:
            g, u = (_LinearSrc(view, f"{p}.{n}_proj", qc) for n in ("gate", "up"))
            gc = lambda lo, hi: _cols(g, lo, hi)
            uc = lambda lo, hi: _cols(u, lo, hi)
        if ffn % (16 * world):
            raise ValueError(f"tensor parallel {world} does not divide FFN {ffn} into runs of 16")
        lo, hi = rank * ffn // world, (rank + 1) * ffn // world
        gu = _interleave_cols(gc(lo, hi), uc(lo, hi))
        if (lo % 64) or (hi % 64):
            raise ValueError(f"tensor parallel {world}: FFN slice {lo}:{hi} is not a whole number of groups")
        return _ql(*gu, device), _ql(d.q[lo:hi], d.scales[lo // 64: hi // 64], device)

    if cfg.is_moe:
        lw.router = view.get(prefix + ".mlp.gate.weight").to(torch.bfloat16).to(device)
        lw.experts = []
        fused = has_linear(f"{prefix}.mlp.experts.0.gate_up_proj")
        for e in range(cfg.n_experts):
            gu, dn = mlp(f"{prefix}.mlp.experts.{e}", cfg.expert_ffn, fused)
            lw.experts.append(ExpertWeights(gu, dn))
        lw.experts_gate_up_w4b = torch.stack([x.gate_up.w4b for x in lw.experts]).contiguous()
        lw.experts_down_w4b = torch.stack([x.down.w4b for x in lw.experts]).contiguous()
        if cfg.shared_ffn:
            gu, dn = mlp(f"{prefix}.mlp.shared_expert", cfg.shared_ffn)
            lw.shared = ExpertWeights(gu, dn)
            if view.has(prefix + ".mlp.shared_expert_gate.weight"):
                lw.shared_gate = view.get(prefix + ".mlp.shared_expert_gate.weight").to(torch.bfloat16).to(device)
    else:
        lw.gate_up, lw.down = mlp(prefix + ".mlp", cfg.ffn)


def load(snapshot: str, device="cuda", mtp: bool = True, int8_head: bool = False, tp: Tuple[int, int] = (0, 1),
         report=sys.stderr) -> ModelWeights:
    t0 = time.time()
    snap = resolve_snapshot(snapshot)
    with open(os.path.join(snap, "config.json")) as f:
        hf = json.load(f)
    if "text_config" in hf:
        hf = {**hf["text_config"], "quantization_config": hf.get("quantization_config", hf["text_config"].get("quantization_config"))}
    cfg = ModelConfig.from_hf_config(hf)
    qc = QuantConfig.parse(hf)
    st = SafetensorsSet(snap)
    view = NameView(st, copy=torch.device(device).type == "cpu")
    rank, world = tp
    embed = view.get("model.embed_tokens.weight").to(torch.bfloat16).to(device)
    head_name = "lm_head.weight" if view.has("lm_head.weight") else "model.embed_tokens.weight"   # tied embeddings
    head = view.get(head_name).to(torch.bfloat16)
    if world > 1:   # vocabulary-parallel head
        per = (cfg.vocab + world - 1) // world
        head = head[rank * per: min(cfg.vocab, (rank + 1) * per)]
    head = head.to(device).contiguous()
    layers = [_load_layer(view, cfg, f"model.layers.{i}", qc, device, tp) for i in range(cfg.n_layers)]
    w = ModelWeights(cfg, embed, head, view.get("model.norm.weight").float().to(device), layers)
    if mtp and cfg.mtp_layers and (view.has("mtp.fc.qweight") or view.has("mtp.fc.weight")):
        fc = _LinearSrc(view, "mtp.fc", qc)
        w.mtp = MtpWeights(view.get("mtp.pre_fc_norm_embedding.weight").float().to(device),
                           view.get("mtp.pre_fc_norm_hidden.weight").float().to(device),
                           _ql(fc.q, fc.scales, device),
                           [_load_layer(view, cfg, f"mtp.layers.{i}", qc, device, tp)
                            for i in range(cfg.mtp_layers)],
                           view.get("mtp.norm.weight").float().to(device))
    if int8_head:
        wf = w.lm_head.float()
        sc = wf.abs().amax(dim=1).clamp_min(1e-8) / 127.0
        w.lm_head_i8 = (torch.round(wf / sc[:, None]).clamp_(-127, 127).to(torch.int8).contiguous(), sc.contiguous())
    if report is not None:
        want = cfg.weight_bytes_per_token(1.0 if int8_head else 2.0) / world
        got = sum(l.qkv.nbytes + l.o.nbytes + (l.gate_up.nbytes + l.down.nbytes if l.gate_up is not None else 0)
                  for l in layers) + w.lm_head.numel() * (1 if int8_head else 2)
        line = (f"load: {cfg.name} {qc.method} g{qc.group_size} from {snap}: {w.nbytes() / 1e9:.3f} GB resident, "
                f"{time.time() - t0:.1f} s")
        if not cfg.is_moe:
            line += f", W = {got / 1e9:.3f} GB / token (descriptor {want / 1e9:.3f})"
            if abs(got - want) > 0.02 * want:
                raise QuantError(f"bytes per token {got} differ from the descriptor's {want:.0f} by more than 2 %")
        report.write(line + "\n")
    return w


def _drafter_linears(cfg: ModelConfig, prefix: str, n_layers: int):
    """(name, out features, in features) of every linear a draft head's snapshot must hold."""
    h = cfg.hidden
    out = [(prefix + "fc", h, 2 * h)]
    for i in range(n_layers):
        p = f"{prefix}layers.{i}"
        out += [(p + ".self_attn.q_proj", cfg.q_dim, h), (p + ".self_attn.k_proj", cfg.kv_dim, h),
                (p + ".self_attn.v_proj", cfg.kv_dim, h), (p + ".self_attn.o_proj", h, cfg.q_dim),
                (p + ".mlp.gate_proj", cfg.ffn, h), (p + ".mlp.up_proj", cfg.ffn, h), (p + ".mlp.down_proj", h, cfg.ffn)]
    return out


def check_drafter(st, cfg: ModelConfig, prefix: str, n_layers: int, group_size: int = 64) -> List[str]:
    """Everything wrong with a drafter snapshot's tensors, by name: missing tensors, element types and shapes that do
    not fit the configuration -- read from the file headers only, before any weight is touched (the reference checks
    its drafter checkpoint the same way: src/loader/dflash_loader.h:24-53).  An empty list: the snapshot loads."""
    bad: List[str] = []

    def want(name, dtypes, shape):
        if not st.has(name):
            bad.append(f"{name}: missing")
            return
        dt, sh = st.dtype(name), tuple(st.shape(name))
        if dt not in dtypes:
            bad.append(f"{name}: element type {dt}, expected one of {sorted(dtypes)}")
        if shape is not None and sh != tuple(shape):
            bad.append(f"{name}: shape {list(sh)}, expected {list(shape)}")

    fl = {"BF16", "F16", "F32"}
    h = cfg.hidden
    for nm in ("pre_fc_norm_embedding.weight", "pre_fc_norm_hidden.weight", "norm.weight"):
        want(prefix + nm, fl, (h,))
    for i in range(n_layers):
        want(f"{prefix}layers.{i}.input_layernorm.weight", fl, (h,))
        want(f"{prefix}layers.{i}.post_attention_layernorm.weight", fl, (h,))
    for name, n, k in _drafter_linears(cfg, prefix, n_layers):
        if st.has(name + ".qweight"):
            want(name + ".qweight", {"I32"}, (k // 8, n))
            want(name + ".scales", {"F16", "BF16"}, (k // group_size, n))
        elif st.has(name + ".weight_scale"):
            want(name + ".weight", {"I8"}, (n, k))
            want(name + ".weight_scale", {"F32", "F16", "BF16"}, None)
        else:
            want(name + ".weight", fl, (n, k))
    return bad


def load_drafter(snapshot: str, device="cuda", report=sys.stderr, tp: Tuple[int, int] = (0, 1)) -> MtpWeights:
    """A draft head from its own snapshot (``--draft-model``): the front (``fc`` over [norm(embed) ‖ norm(hidden)],
    the two pre-norms), its decoder layers and its output norm.  Linears come as int4 (the GPTQ layout of the main
    checkpoint), dense bf16 / fp16, or int8 with a scale per output row; the last two are quantised to int4 g64 on the
    host.  Tensor names may carry the prefix ``mtp.`` (a head cut out of a main checkpoint), ``drafter.`` or none.
    ``mask_token_id`` of ``config.json`` names the token whose embedding row stands for "not drafted yet" in a block.
    The snapshot's tensors are checked against the configuration before anything is read; one error lists every
    problem.  ``tp`` = (rank, world): the layers are sliced like the trunk's (the reference splits its drafter for two
    cards: src/loader/dflash_tp_split.h), the front and the norms are held whole.  The reference: src/loader/dflash_loader.h:24-75, src/loader/loader.cc:521 load_mtp."""
    snap = resolve_snapshot(snapshot)
    with open(os.path.join(snap, "config.json")) as f:
        hf = json.load(f)
    if "text_config" in hf:
        hf = {**hf["text_config"], "quantization_config": hf.get("quantization_config", hf["text_config"].get("quantization_config")),
              "mask_token_id": hf.get("mask_token_id", hf["text_config"].get("mask_token_id"))}
    cfg = ModelConfig.from_hf_config(hf)
    # an unquantised drafter has no quantization_config: its linears take the host quantiser's group size
    qc = QuantConfig.parse(hf) if hf.get("quantization_config") else QuantConfig("none", 4, 64, True, False)
    st = SafetensorsSet(snap)
    view = NameView(st, copy=torch.device(device).type == "cpu")
    prefix = next((p for p in ("mtp.", "drafter.", "")
                   if any(view.has(p + "fc" + sfx) for sfx in (".qweight", ".weight"))), None)
    if prefix is None:
        raise KeyError(f"{snap}: no draft head found (fc.qweight or fc.weight under mtp., drafter. or no prefix)")
    n_layers = 0
    while view.has(f"{prefix}layers.{n_layers}.input_layernorm.weight"):
        n_layers += 1
    bad = check_drafter(view, cfg, prefix, n_layers, qc.group_size)
    if bad:
        raise ValueError(f"{snap}: the draft head does not fit its configuration:\n  " + "\n  ".join(bad))
    fc = _LinearSrc(view, prefix + "fc", qc)
    head = MtpWeights(view.get(prefix + "pre_fc_norm_embedding.weight").float().to(device),
                      view.get(prefix + "pre_fc_norm_hidden.weight").float().to(device),
                      _ql(fc.q, fc.scales, device),
                      [_load_layer(view, cfg, f"{prefix}layers.{i}", qc, device, tp) for i in range(n_layers)],
                      view.get(prefix + "norm.weight").float().to(device))
    mt = hf.get("mask_token_id")
    head.mask_token = int(mt) if mt is not None and 0 <= int(mt) < cfg.vocab else None
    if report is not None:
        fmt = "int4" if view.has(prefix + "fc.qweight") else ("int8" if view.has(prefix + "fc.weight_scale") else "dense")
        report.write(f"load: draft head with {n_layers} layer(s) ({fmt} linears) from {snap}\n")
    return head

"""Synthetic checkpoints in the exact Hugging Face layout the loader reads.

``write_checkpoint`` turns a random-init ``ModelWeights`` into a snapshot directory: sharded
safetensors with per-projection ``qweight`` (int32 ``[K/8][N]``) / ``scales`` (fp16 ``[K/64][N]``)
/ ``qzeros`` (all 0x77777777) / ``g_idx`` (identity), bf16 norms / embeddings / head,
``model.safetensors.index.json`` and ``config.json`` with its ``quantization_config`` -- what the
reference's tools/quantize/*/make_synth.py produce for its tests.  Loading the snapshot gives back
the same kernel-layout bytes.
"""
from __future__ import annotations

import json
import os
from typing import Dict

import torch

from ..models.config import ModelConfig
from ..models.weights import LayerWeights, ModelWeights, QLinear
from . import quant as Q
from .safetensors_io import save_file


def _emit_linear(out: Dict[str, torch.Tensor], name: str, q: torch.Tensor, scales: torch.Tensor, g_idx: bool):
    k, n = q.shape
    out[name + ".qweight"] = Q.pack_gptq(q)
    out[name + ".scales"] = scales.contiguous()
    out[name + ".qzeros"] = Q.make_qzeros(k, n)
    if g_idx:
        out[name + ".g_idx"] = (torch.arange(k) // 64).to(torch.int32)


def _split_gate_up(ql: QLinear):
    q, s = Q.from_w4b(ql.w4b.cpu(), ql.n)
    k = q.shape[0]
    qv = q.reshape(k, ql.n // 32, 2, 16)
    sv = s.reshape(s.shape[0], ql.n // 32, 2, 16)
    return ((qv[:, :, 0].reshape(k, -1), sv[:, :, 0].reshape(s.shape[0], -1)),
            (qv[:, :, 1].reshape(k, -1), sv[:, :, 1].reshape(s.shape[0], -1)))


def _emit_layer(out, cfg: ModelConfig, prefix: str, lw: LayerWeights, g_idx: bool, fused_experts: bool = False):
    out[prefix + ".input_layernorm.weight"] = lw.input_norm.cpu().to(torch.bfloat16)
    out[prefix + ".post_attention_layernorm.weight"] = lw.post_norm.cpu().to(torch.bfloat16)
    if lw.gdn is not None:
        g, p = lw.gdn, prefix + ".linear_attn"
        q, s = Q.from_w4b(g.in_proj.w4b.cpu(), g.in_proj.n)
        a = g.in_proj.n - 2 * cfg.gdn_v_heads
        _emit_linear(out, p + ".in_proj_qkvz", q[:, :a], s[:, :a], g_idx)
        _emit_linear(out, p + ".in_proj_ba", q[:, a:], s[:, a:], g_idx)
        _emit_linear(out, p + ".out_proj", *Q.from_w4b(g.out_proj.w4b.cpu(), g.out_proj.n), g_idx)
        out[p + ".conv1d.weight"] = g.conv_w.cpu().reshape(-1, 1, 4).contiguous()
        out[p + ".A_log"], out[p + ".dt_bias"], out[p + ".norm.weight"] = g.a_log.cpu(), g.dt_bias.cpu(), g.norm_w.cpu()
    else:
        q, s = Q.from_w4b(lw.qkv.w4b.cpu(), lw.qkv.n)
        a, b = cfg.q_dim, cfg.q_dim + cfg.kv_dim
        _emit_linear(out, prefix + ".self_attn.q_proj", q[:, :a], s[:, :a], g_idx)
        _emit_linear(out, prefix + ".self_attn.k_proj", q[:, a:b], s[:, a:b], g_idx)
        _emit_linear(out, prefix + ".self_attn.v_proj", q[:, b:], s[:, b:], g_idx)
        _emit_linear(out, prefix + ".self_attn.o_proj", *Q.from_w4b(lw.o.w4b.cpu(), lw.o.n), g_idx)

    def mlp(p, gate_up: QLinear, down: QLinear):
        (gq, gs), (uq, us) = _split_gate_up(gate_up)
        _emit_linear(out, p + ".gate_proj", gq, gs, g_idx)
        _emit_linear(out, p + ".up_proj", uq, us, g_idx)
        _emit_linear(out, p + ".down_proj", *Q.from_w4b(down.w4b.cpu(), down.n), g_idx)

    if lw.experts is not None:
        out[prefix + ".mlp.gate.weight"] = lw.router.cpu()
        for e, ex in enumerate(lw.experts):
            if fused_experts:     # one gate_up_proj per expert: gate columns first, then up
                (gq, gs), (uq, us) = _split_gate_up(ex.gate_up)
                p = f"{prefix}.mlp.experts.{e}"
                _emit_linear(out, p + ".gate_up_proj", torch.cat([gq, uq], dim=1), torch.cat([gs, us], dim=1), g_idx)
                _emit_linear(out, p + ".down_proj", *Q.from_w4b(ex.down.w4b.cpu(), ex.down.n), g_idx)
            else:
                mlp(f"{prefix}.mlp.experts.{e}", ex.gate_up, ex.down)
        if lw.shared is not None:
            mlp(prefix + ".mlp.shared_expert", lw.shared.gate_up, lw.shared.down)
            out[prefix + ".mlp.shared_expert_gate.weight"] = lw.shared_gate.cpu()
    else:
        mlp(prefix + ".mlp", lw.gate_up, lw.down)


def write_checkpoint(w: ModelWeights, path: str, shards: int = 2, g_idx: bool = False, wrapper_prefix: bool = False,
                     quant_method: str = "gptq", fused_experts: bool = False) -> str:
    """Writes ``w`` as a snapshot directory and returns it.  Norm weights are stored in bf16 (as real
    checkpoints do), so ``w``'s norms should be bf16-representable for a bit-exact round trip."""
    os.makedirs(path, exist_ok=True)
    cfg = w.cfg
    tensors: Dict[str, torch.Tensor] = {"model.embed_tokens.weight": w.embed.cpu(), "lm_head.weight": w.lm_head.cpu(),
                                        "model.norm.weight": w.final_norm.cpu().to(torch.bfloat16)}
    for i, lw in enumerate(w.layers):
        _emit_layer(tensors, cfg, f"model.layers.{i}", lw, g_idx, fused_experts)
    if w.mtp is not None:
        m = w.mtp
        tensors["mtp.pre_fc_norm_embedding.weight"] = m.pre_norm_embed.cpu().to(torch.bfloat16)
        tensors["mtp.pre_fc_norm_hidden.weight"] = m.pre_norm_hidden.cpu().to(torch.bfloat16)
        tensors["mtp.norm.weight"] = m.norm.cpu().to(torch.bfloat16)
        _emit_linear(tensors, "mtp.fc", *Q.from_w4b(m.fc.w4b.cpu(), m.fc.n), g_idx)
        for i, lw in enumerate(m.layers):
            _emit_layer(tensors, cfg, f"mtp.layers.{i}", lw, g_idx)
    if wrapper_prefix:   # multimodal wrappers nest the language model and carry a vision tower the loader skips
        tensors = {("model.language_model." + k[len("model."):] if k.startswith("model.") else k): v
                   for k, v in tensors.items()}
        tensors["model.visual.patch_embed.weight"] = torch.zeros(4, 4, dtype=torch.bfloat16)
    names = list(tensors)
    per = (len(names) + shards - 1) // shards
    weight_map = {}
    for si in range(shards):
        part = names[si * per: (si + 1) * per]
        if not part:
            continue
        fname = f"model-{si + 1:05d}-of-{shards:05d}.safetensors"
        save_file({n: tensors[n] for n in part}, os.path.join(path, fname), {"format": "pt"})
        for n in part:
            weight_map[n] = fname
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    hf = cfg.to_hf_config()
    hf["quantization_config"]["quant_method"] = quant_method
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f, indent=1)
    return path


def write_drafter(head, cfg: ModelConfig, path: str, fmt: str = "int4", prefix: str = "drafter.",
                  mask_token_id: int = -1) -> str:
    """Writes a draft head (front, decoder layers, norm) as a snapshot of its own in one of the formats a drafter
    ships in: ``int4`` (GPTQ g64, as the main checkpoint), ``bf16`` (dense ``.weight`` [out][in]) or ``int8``
    (``.weight`` int8 [out][in] + ``.weight_scale`` fp32 [out])."""
    os.makedirs(path, exist_ok=True)
    t: Dict[str, torch.Tensor] = {}
    t[prefix + "pre_fc_norm_embedding.weight"] = head.pre_norm_embed.cpu().to(torch.bfloat16)
    t[prefix + "pre_fc_norm_hidden.weight"] = head.pre_norm_hidden.cpu().to(torch.bfloat16)
    t[prefix + "norm.weight"] = head.norm.cpu().to(torch.bfloat16)
    _emit_linear(t, prefix + "fc", *Q.from_w4b(head.fc.w4b.cpu(), head.fc.n), False)
    for i, lw in enumerate(head.layers):
        _emit_layer(t, cfg, f"{prefix}layers.{i}", lw, False)
    if fmt != "int4":
        for name in [n[: -len(".qweight")] for n in list(t) if n.endswith(".qweight")]:
            q = Q.unpack_gptq(t.pop(name + ".qweight"))
            sc = t.pop(name + ".scales")
            t.pop(name + ".qzeros")
            dense = ((q.float() - 8.0) * sc.float().repeat_interleave(64, dim=0)).t().contiguous()     # [out][in]
            if fmt == "bf16":
                t[name + ".weight"] = dense.to(torch.bfloat16)
            else:
                s8 = dense.abs().amax(dim=1).clamp_min(1e-12) / 127.0
                t[name + ".weight"] = torch.round(dense / s8[:, None]).clamp_(-127, 127).to(torch.int8)
                t[name + ".weight_scale"] = s8.float()
    save_file(t, os.path.join(path, "model.safetensors"), {"format": "pt"})
    hf = cfg.to_hf_config()
    if fmt != "int4":
        hf.pop("quantization_config", None)
    if mask_token_id >= 0:
        hf["mask_token_id"] = mask_token_id
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(hf, f, indent=1)
    return path

"""Quantisation config parsing, tensor classification and invariant checks.

Accepted, as by the reference (src/loader/quant.h:33-200, quant.cc:331 parse, :434 classify, :523
assert_quant_invariants): GPTQ and AutoRound (both vocabularies), and compressed-tensors
pack-quantized; int4, symmetric, group size 64 or 128 (128 is expanded to 64), no act-order.
Invariants checked on every quantised linear: ``qzeros`` words all 0x77777777, ``g_idx`` (when
present) the identity ``k // group``, scales finite.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class QuantError(ValueError):
    pass


@dataclass
class QuantConfig:
    method: str            # gptq | auto-round | compressed-tensors
    bits: int
    group_size: int
    sym: bool
    desc_act: bool

    @staticmethod
    def parse(cfg: dict) -> "QuantConfig":
        q = cfg.get("quantization_config")
        if q is None:
            raise QuantError("config.json has no quantization_config: only W4A16 checkpoints are served")
        method = str(q.get("quant_method", "")).lower().replace("_", "-")
        if method in ("gptq", "auto-round", "autoround", "intel/auto-round"):
            method = "gptq" if method == "gptq" else "auto-round"
            bits = int(q.get("bits", q.get("w_bit", 0)))
            group = int(q.get("group_size", q.get("q_group_size", 0)))
            sym = bool(q.get("sym", q.get("symmetric", not q.get("zero_point", False))))
            desc = bool(q.get("desc_act", False))
            pf = q.get("packing_format", "auto_round:auto_gptq")
            if method == "auto-round" and "gptq" not in str(pf):
                raise QuantError(f"auto-round packing_format {pf!r} is not the GPTQ layout")
        elif method == "compressed-tensors":
            if q.get("format") != "pack-quantized":
                raise QuantError("compressed-tensors: only format pack-quantized is supported")
            groups = q.get("config_groups", {})
            if len(groups) != 1:
                raise QuantError("compressed-tensors: exactly one config group is supported")
            w = next(iter(groups.values())).get("weights", {})
            bits, group = int(w.get("num_bits", 0)), int(w.get("group_size", 0))
            sym, desc = bool(w.get("symmetric", False)), w.get("actorder") not in (None, False, "none")
        else:
            raise QuantError(f"unsupported quant_method {q.get('quant_method')!r}")
        if bits != 4:
            raise QuantError(f"bits = {bits}: only int4 weights are supported")
        if group not in (64, 128):
            raise QuantError(f"group_size = {group}: only 64 and 128 are supported")
        if not sym:
            raise QuantError("asymmetric quantisation is not supported (zero point must be 8)")
        if desc:
            raise QuantError("desc_act / act-order checkpoints are not supported")
        return QuantConfig(method, bits, group, sym, desc)


def classify(name: str) -> Optional[str]:
    """Which part of a linear a tensor name is: qweight | scales | qzeros | g_idx | weight | bias | None."""
    for suf, kind in ((".qweight", "qweight"), (".scales", "scales"), (".qzeros", "qzeros"), (".g_idx", "g_idx"),
                      (".weight_packed", "qweight"), (".weight_scale", "scales"), (".weight_shape", "shape"),
                      (".weight", "weight"), (".bias", "bias")):
        if name.endswith(suf):
            return kind
    return None


def assert_quant_invariants(name: str, qweight: torch.Tensor, scales: torch.Tensor, qzeros: Optional[torch.Tensor],
                            g_idx: Optional[torch.Tensor], group: int):
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    if qweight.dtype != torch.int32:
        raise QuantError(f"{name}.qweight: expected int32, found {qweight.dtype}")
    if tuple(scales.shape) != (k // group, n):
        raise QuantError(f"{name}.scales: shape {tuple(scales.shape)} does not match [{k // group}][{n}]")
    if not torch.isfinite(scales.float()).all():
        raise QuantError(f"{name}.scales: non-finite values")
    if qzeros is not None:
        if (qzeros != 0x77777777).any():
            raise QuantError(f"{name}.qzeros: not all 0x77777777 (the checkpoint is not symmetric int4)")
    if g_idx is not None:
        want = torch.arange(k, dtype=g_idx.dtype) // group
        if not torch.equal(g_idx.cpu(), want):
            raise QuantError(f"{name}.g_idx: not the identity (act-order is not supported)")

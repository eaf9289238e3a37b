"""Checkpoint round trip on CPU: synthetic HF snapshot -> loader -> the same kernel-layout bytes;
quantisation config and invariant checks; safetensors reader bounds checks; snapshot resolution."""
import json
import os
import struct
from dataclasses import replace

import pytest
import torch

from b200serve.loader.loader import load
from b200serve.loader.quant_config import QuantConfig, QuantError, assert_quant_invariants, classify
from b200serve.loader.snapshot import resolve_snapshot
from b200serve.models.config import small_dense, tiny_dense, tiny_moe
from b200serve.models.oracle import OracleModel
from b200serve.models.weights import random_weights
from b200serve.native import host as H
from b200serve.utils import quant as Q
from b200serve.utils.safetensors_io import SafetensorsSet, save_file
from b200serve.utils.synth import write_checkpoint


def _bf16_norms(w):
    for lw in w.layers + (w.mtp.layers if w.mtp else []):
        lw.input_norm = lw.input_norm.to(torch.bfloat16).float()
        lw.post_norm = lw.post_norm.to(torch.bfloat16).float()
    return w


@pytest.mark.parametrize("make,kw", [(tiny_dense, {}), (tiny_moe, {}), (tiny_moe, {"fused_experts": True}),
                                     (tiny_dense, {"g_idx": True, "wrapper_prefix": True, "quant_method": "auto-round"})])
def test_checkpoint_round_trip(tmp_path, make, kw):
    cfg = make()
    if not cfg.is_moe:
        cfg = replace(cfg, mtp_layers=1)
    w = _bf16_norms(random_weights(cfg, seed=5))
    snap = write_checkpoint(w, str(tmp_path / "snap"), **kw)
    got = load(snap, device="cpu", report=None)
    assert got.cfg == replace(cfg, name=got.cfg.name)
    assert torch.equal(got.embed, w.embed) and torch.equal(got.lm_head, w.lm_head)
    for a, b in zip(got.layers, w.layers):
        assert torch.equal(a.qkv.w4b, b.qkv.w4b) and torch.equal(a.o.w4b, b.o.w4b)
        assert torch.equal(a.input_norm, b.input_norm) and torch.equal(a.post_norm, b.post_norm)
        if b.gate_up is not None:
            assert torch.equal(a.gate_up.w4b, b.gate_up.w4b) and torch.equal(a.down.w4b, b.down.w4b)
        else:
            assert torch.equal(a.experts_gate_up_w4b, b.experts_gate_up_w4b)
            assert torch.equal(a.experts_down_w4b, b.experts_down_w4b)
            assert torch.equal(a.router, b.router) and torch.equal(a.shared.down.w4b, b.shared.down.w4b)
    if cfg.mtp_layers:
        assert torch.equal(got.mtp.fc.w4b, w.mtp.fc.w4b)
    # the loaded model computes what the original does
    ids = torch.arange(12) % cfg.vocab
    assert torch.equal(OracleModel(got).forward(ids), OracleModel(w).forward(ids))


def test_tensor_parallel_slices_reassemble(tmp_path):
    cfg = small_dense()
    w = _bf16_norms(random_weights(cfg, seed=2))
    snap = write_checkpoint(w, str(tmp_path / "s"))
    parts = [load(snap, device="cpu", tp=(r, 2), report=None) for r in range(2)]
    full_qkv = Q.dequant_w4b(w.layers[0].qkv.w4b, cfg.qkv_dim)
    hd, qh, kh = cfg.head_dim, cfg.n_q_heads // 2, cfg.n_kv_heads // 2
    for r, p in enumerate(parts):
        got = Q.dequant_w4b(p.layers[0].qkv.w4b, p.layers[0].qkv.n)
        want = torch.cat([full_qkv[r * qh * hd:(r + 1) * qh * hd],
                          full_qkv[cfg.q_dim + r * kh * hd: cfg.q_dim + (r + 1) * kh * hd],
                          full_qkv[cfg.q_dim + cfg.kv_dim + r * kh * hd: cfg.q_dim + cfg.kv_dim + (r + 1) * kh * hd]])
        assert torch.equal(got, want)
    # row-parallel o: the two partial products add up to the full one
    x = torch.randn(3, cfg.q_dim)
    full = x @ Q.dequant_w4b(w.layers[0].o.w4b, cfg.hidden).t()
    half = cfg.q_dim // 2
    acc = sum(x[:, r * half:(r + 1) * half] @ Q.dequant_w4b(p.layers[0].o.w4b, cfg.hidden).t() for r, p in enumerate(parts))
    assert torch.allclose(acc, full, atol=1e-5)
    # vocabulary-parallel head
    assert torch.equal(torch.cat([p.lm_head for p in parts]), w.lm_head)


def test_quant_config_accepts_and_refuses():
    ok = {"quantization_config": {"quant_method": "gptq", "bits": 4, "group_size": 64, "sym": True, "desc_act": False}}
    assert QuantConfig.parse(ok).group_size == 64
    ar = {"quantization_config": {"quant_method": "auto-round", "bits": 4, "group_size": 128, "sym": True,
                                  "packing_format": "auto_round:auto_gptq"}}
    assert QuantConfig.parse(ar).method == "auto-round"
    ct = {"quantization_config": {"quant_method": "compressed-tensors", "format": "pack-quantized", "config_groups": {
        "g0": {"weights": {"num_bits": 4, "group_size": 64, "symmetric": True}}}}}
    assert QuantConfig.parse(ct).method == "compressed-tensors"
    for bad in ({}, {"quantization_config": {"quant_method": "awq"}},
                {"quantization_config": {"quant_method": "gptq", "bits": 8, "group_size": 64, "sym": True}},
                {"quantization_config": {"quant_method": "gptq", "bits": 4, "group_size": 32, "sym": True}},
                {"quantization_config": {"quant_method": "gptq", "bits": 4, "group_size": 64, "sym": False}},
                {"quantization_config": {"quant_method": "gptq", "bits": 4, "group_size": 64, "sym": True, "desc_act": True}}):
        with pytest.raises(QuantError):
            QuantConfig.parse(bad)
    assert classify("a.b.qweight") == "qweight" and classify("x.weight") == "weight" and classify("x.foo") is None


def test_quant_invariants():
    q = torch.randint(0, 16, (128, 16), dtype=torch.uint8)
    qw, sc = Q.pack_gptq(q), torch.ones(2, 16, dtype=torch.float16)
    assert_quant_invariants("l", qw, sc, Q.make_qzeros(128, 16), torch.arange(128) // 64, 64)
    z = Q.make_qzeros(128, 16); z[0, 0] = 0x77777778
    with pytest.raises(QuantError):
        assert_quant_invariants("l", qw, sc, z, None, 64)
    with pytest.raises(QuantError):
        assert_quant_invariants("l", qw, sc, None, torch.arange(128).flip(0) // 64, 64)
    bad = sc.clone(); bad[1, 3] = float("inf")
    with pytest.raises(QuantError):
        assert_quant_invariants("l", qw, bad, None, None, 64)
    with pytest.raises(QuantError):
        assert_quant_invariants("l", qw, torch.ones(3, 16, dtype=torch.float16), None, None, 64)


def test_safetensors_reader_bounds(tmp_path):
    p = str(tmp_path / "a.safetensors")
    save_file({"x": torch.arange(6, dtype=torch.int32).reshape(2, 3), "y": torch.ones(4, dtype=torch.bfloat16)}, p)
    f = H.SafetensorsFile(p)
    assert sorted(f.names()) == ["x", "y"] and f.shape("x") == [2, 3] and f.dtype("y") == "BF16"
    st = SafetensorsSet(str(tmp_path))
    assert st.get("x").tolist() == [[0, 1, 2], [3, 4, 5]]
    raw = open(p, "rb").read()
    hlen = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + hlen])
    # a header length beyond the file, and a tensor range beyond the data section, are refused
    open(str(tmp_path / "b.safetensors"), "wb").write(struct.pack("<Q", 1 << 40) + raw[8:])
    with pytest.raises(RuntimeError):
        H.SafetensorsFile(str(tmp_path / "b.safetensors"))
    hdr["x"]["data_offsets"] = [0, 10 ** 6]
    hj = json.dumps(hdr).encode()
    open(str(tmp_path / "c.safetensors"), "wb").write(struct.pack("<Q", len(hj)) + hj + raw[8 + hlen:])
    with pytest.raises(RuntimeError):
        H.SafetensorsFile(str(tmp_path / "c.safetensors"))


def test_snapshot_resolution(tmp_path, monkeypatch):
    base = tmp_path / "hub" / "models--org--name"
    (base / "refs").mkdir(parents=True)
    (base / "snapshots" / "abc").mkdir(parents=True)
    (base / "refs" / "main").write_text("abc")
    monkeypatch.setenv("HF_HOME", str(tmp_path))
    assert resolve_snapshot("org/name") == str(base / "snapshots" / "abc")
    assert resolve_snapshot(str(tmp_path)) == str(tmp_path)
    with pytest.raises(FileNotFoundError):
        resolve_snapshot("org/missing")


def test_hybrid_checkpoint_round_trip(tmp_path):
    """Gated delta-net layers (linear_attn.*) beside attention layers: write, load, same logits."""
    from b200serve.models.config import preset
    cfg = preset("small-hybrid")
    w = _bf16_norms(random_weights(cfg, seed=7))
    snap = write_checkpoint(w, str(tmp_path / "snap"))
    got = load(snap, device="cpu", report=None)
    assert got.cfg == replace(cfg, name=got.cfg.name)
    assert [lw.gdn is not None for lw in got.layers] == [True, False, True, False]
    for a, b in zip(got.layers, w.layers):
        if b.gdn is None:
            assert torch.equal(a.qkv.w4b, b.qkv.w4b)
            continue
        assert a.qkv is None and a.o is None
        assert torch.equal(a.gdn.in_proj.w4b, b.gdn.in_proj.w4b) and torch.equal(a.gdn.out_proj.w4b, b.gdn.out_proj.w4b)
        for f in ("conv_w", "a_log", "dt_bias", "norm_w"):
            assert torch.equal(getattr(a.gdn, f), getattr(b.gdn, f)), f
    ids = torch.arange(12) % cfg.vocab
    assert torch.equal(OracleModel(got).forward(ids), OracleModel(w).forward(ids))


@pytest.mark.parametrize("fmt", ["int4", "bf16", "int8"])
def test_drafter_snapshot_formats(tmp_path, fmt):
    """A block drafter's snapshot loads from int4 (GPTQ), dense bf16 and int8-with-row-scales linears; the unquantised
    forms are quantised on the host and stay close to the original; the mask token comes from config.json."""
    from b200serve.loader.loader import load_drafter
    from b200serve.runtime.spec import random_drafter
    from b200serve.utils.synth import write_drafter
    cfg = tiny_dense()
    head = random_drafter(cfg, "cpu", seed=3, layers=2)
    snap = write_drafter(head, cfg, str(tmp_path / fmt), fmt=fmt, mask_token_id=cfg.vocab - 2)
    got = load_drafter(snap, device="cpu", report=None)
    assert len(got.layers) == 2 and got.mask_token == cfg.vocab - 2
    pairs = [(head.fc, got.fc)] + [(a.qkv, b.qkv) for a, b in zip(head.layers, got.layers)] + \
            [(a.down, b.down) for a, b in zip(head.layers, got.layers)]
    for a, b in pairs:
        qa, sa = Q.from_w4b(a.w4b, a.n)
        qb, sb = Q.from_w4b(b.w4b, b.n)
        da = (qa.float() - 8) * sa.float().repeat_interleave(64, dim=0)
        db = (qb.float() - 8) * sb.float().repeat_interleave(64, dim=0)
        if fmt == "int4":
            assert torch.equal(qa, qb) and torch.equal(sa, sb)
        else:   # one more rounding (bf16 or int8) and a second round-to-nearest int4
            assert (da - db).abs().max() <= 0.6 * sa.float().max()


def test_drafter_snapshot_check_lists_every_problem(tmp_path):
    from b200serve.loader.loader import load_drafter
    from b200serve.runtime.spec import random_drafter
    from b200serve.utils.synth import write_drafter
    cfg = tiny_dense()
    head = random_drafter(cfg, "cpu", seed=3, layers=1)
    snap = write_drafter(head, cfg, str(tmp_path / "d"), fmt="bf16")
    st = SafetensorsSet(snap)
    t = {n: st.get(n) for n in st.names()}
    del t["drafter.norm.weight"]
    t["drafter.layers.0.mlp.down_proj.weight"] = t["drafter.layers.0.mlp.down_proj.weight"][:, :-64].contiguous()
    t["drafter.fc.weight"] = t["drafter.fc.weight"].to(torch.int32)
    save_file(t, os.path.join(snap, "model.safetensors"), {"format": "pt"})
    with pytest.raises(ValueError) as e:
        load_drafter(snap, device="cpu", report=None)
    msg = str(e.value)
    assert "drafter.norm.weight: missing" in msg
    assert "drafter.layers.0.mlp.down_proj.weight: shape" in msg
    assert "drafter.fc.weight: element type I32" in msg


def test_mixed_expert_forms_in_a_layer_are_refused(tmp_path):
    """Experts of one layer come either all as gate_proj / up_proj or all as one gate_up_proj; a mix names the expert."""
    cfg = tiny_moe()
    w = _bf16_norms(random_weights(cfg, seed=6))
    snap = write_checkpoint(w, str(tmp_path / "snap"), shards=1, fused_experts=True)
    st = SafetensorsSet(snap)
    t = {n: st.get(n) for n in st.names()}
    p = "model.layers.0.mlp.experts.1"
    both = Q.unpack_gptq(t[p + ".gate_up_proj.qweight"])
    half = both.shape[1] // 2
    for name, cols in (("gate_proj", slice(0, half)), ("up_proj", slice(half, 2 * half))):
        t[f"{p}.{name}.qweight"] = Q.pack_gptq(both[:, cols].contiguous())
        t[f"{p}.{name}.scales"] = t[p + ".gate_up_proj.scales"][:, cols].contiguous()
        t[f"{p}.{name}.qzeros"] = t[p + ".gate_up_proj.qzeros"][:, : half // 8].contiguous()
    for sfx in (".qweight", ".scales", ".qzeros"):
        del t[p + ".gate_up_proj" + sfx]
    fname = [f for f in os.listdir(snap) if f.endswith(".safetensors")][0]
    save_file(t, os.path.join(snap, fname), {"format": "pt"})
    with open(os.path.join(snap, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": {n: fname for n in t}}, f)
    with pytest.raises(ValueError, match="experts.1: mixed expert forms"):
        load(snap, device="cpu", report=None)


def test_gdn_gate_projection_forms(tmp_path):
    """The gate projection of gated delta-net layers as two tensors (in_proj_b, in_proj_a) loads to the same fused
    projection as in_proj_ba; a checkpoint that mixes the forms is refused by name."""
    from b200serve.models.config import preset
    cfg = preset("small-hybrid")
    w = _bf16_norms(random_weights(cfg, seed=8))
    snap = write_checkpoint(w, str(tmp_path / "snap"), shards=1)
    fname = [f for f in os.listdir(snap) if f.endswith(".safetensors")][0]
    st = SafetensorsSet(snap)
    base = {n: st.get(n) for n in st.names()}
    nv = cfg.gdn_v_heads

    def split(t, layer):
        p = f"model.layers.{layer}.linear_attn"
        q = Q.unpack_gptq(t[p + ".in_proj_ba.qweight"])
        sc = t[p + ".in_proj_ba.scales"]
        for name, cols in (("in_proj_b", slice(0, nv)), ("in_proj_a", slice(nv, 2 * nv))):
            t[f"{p}.{name}.qweight"] = Q.pack_gptq(q[:, cols].contiguous())
            t[f"{p}.{name}.scales"] = sc[:, cols].contiguous()
            t[f"{p}.{name}.qzeros"] = Q.make_qzeros(q.shape[0], nv)
        for sfx in (".qweight", ".scales", ".qzeros"):
            del t[p + ".in_proj_ba" + sfx]

    def write(t):
        save_file(t, os.path.join(snap, fname), {"format": "pt"})
        with open(os.path.join(snap, "model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {}, "weight_map": {n: fname for n in t}}, f)

    t = dict(base)
    for layer in (0, 2):
        split(t, layer)
    write(t)
    got = load(snap, device="cpu", report=None)
    for a, b in zip(got.layers, w.layers):
        if b.gdn is not None:
            assert torch.equal(a.gdn.in_proj.w4b, b.gdn.in_proj.w4b)
    t = dict(base)
    split(t, 2)            # layer 0 keeps in_proj_ba
    write(t)
    with pytest.raises(ValueError, match="layers.2.linear_attn: gate projection is split"):
        load(snap, device="cpu", report=None)

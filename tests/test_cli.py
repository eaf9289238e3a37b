"""Flag system, parallel-placement parsing and the draft-head loader (CPU)."""
import dataclasses

import pytest
import torch

from b200serve.cli import flags as F
from b200serve.models.config import preset
from b200serve.models.weights import random_weights


def test_serve_flags_parse_and_help():
    f = F.parse(F.ServeFlags, ["dense-27b", "--spec", "mtp", "--kv-cache", "int8", "--prefill-backend", "int8",
                               "--parallel", "tp4", "--prefix-split-last", "--max-num-seqs", "8", "--max-len", "auto"],
                "serve", "x")
    assert (f.model, f.spec, f.kv_cache, f.prefill_backend, f.parallel) == ("dense-27b", "mtp", "int8", "int8", "tp4")
    assert f.prefix_split_last is True and f.max_num_seqs == 8 and f.max_len == "auto"
    help_text = F.build_parser(F.ServeFlags, "serve", "x").format_help()
    for name in ("--spec", "--draft-model", "--kv-cache", "--prefill-backend", "--parallel", "--prefix-split-last"):
        assert name in help_text
    with pytest.raises(SystemExit):
        F.parse(F.ServeFlags, ["m", "--kv-cache", "fp8"], "serve", "x")


def test_decode_flags_defaults():
    f = F.parse(F.DecodeFlags, ["tiny-dense", "--bench", "--depth", "1024"], "decode", "x")
    assert f.bench and f.depth == 1024 and f.tg == 128 and not f.profile


def test_draft_head_roundtrip_through_a_snapshot(tmp_path):
    from b200serve.loader.loader import load, load_drafter
    from b200serve.utils.synth import write_checkpoint
    cfg = dataclasses.replace(preset("tiny-dense"), mtp_layers=1)
    w = random_weights(cfg, device="cpu", seed=3)
    write_checkpoint(w, str(tmp_path))
    head = load_drafter(str(tmp_path), device="cpu", report=None)
    full = load(str(tmp_path), device="cpu", report=None)
    assert len(head.layers) == 1
    assert torch.equal(head.fc.w4b, full.mtp.fc.w4b)
    assert torch.equal(head.norm, full.mtp.norm)
    assert torch.equal(head.layers[0].qkv.w4b, full.mtp.layers[0].qkv.w4b)


def test_draft_vocabulary_rule():
    from b200serve.loader.draft_vocab import build_draft_vocab
    ids = build_draft_vocab(1000, 16, forced=[999, 2], ranked=[500, 2, 501, 7])
    assert len(ids) == 16 and ids == sorted(ids)
    assert {999, 2, 500, 501, 7} <= set(ids)
    assert set(ids) - {999, 2, 500, 501, 7} == set(i for i in range(13) if i not in (2, 7))   # lowest ids fill the rest
    assert build_draft_vocab(100, 0) == list(range(100)) and build_draft_vocab(100, 200) == list(range(100))
    with pytest.raises(ValueError):
        build_draft_vocab(100, 2, forced=[1, 2, 3])


def test_parallel_auto_picks_the_fewest_gpus_that_hold_the_model(tmp_path):
    import dataclasses
    from b200serve.cli import common
    from b200serve.models.config import preset
    from b200serve.models.weights import random_weights
    from b200serve.utils.synth import write_checkpoint
    gib = 1 << 30
    dense, moe = preset("dense-27b"), preset("moe-35b-a3b")
    assert common.parallel_auto(dense, 8, 180 * gib) == "1"
    assert common.parallel_auto(moe, 8, 180 * gib) == "1"
    # a 24 GiB card does not hold the 27B shape (12.8 GB of weights + head + scratch): two of them do
    assert common.parallel_auto(dense, 8, 16 * gib) == "tp2"
    big = dataclasses.replace(dense, n_layers=1280, name="dense-540b")       # 256 GB of W4 weights
    assert common.parallel_auto(big, 8, 180 * gib) == "tp2"
    assert common.parallel_auto(big, 8, 60 * gib) == "tp8"
    big_moe = dataclasses.replace(moe, n_layers=400, name="moe-350b")
    assert common.parallel_auto(big_moe, 8, 80 * gib) == "ep4"
    assert common.parallel_auto(big_moe, 8, 180 * gib) == "1"
    with pytest.raises(SystemExit):
        common.parallel_auto(big, 1, 16 * gib)
    # the shape comes from config.json without loading a weight
    cfg = preset("tiny-dense")
    snap = write_checkpoint(random_weights(cfg, seed=1), str(tmp_path / "snap"))
    got = common.peek_config(snap)
    assert (got.n_layers, got.hidden, got.vocab) == (cfg.n_layers, cfg.hidden, cfg.vocab)
    assert common.peek_config("small-hybrid").n_gdn_layers == 2

"""Tensor parallelism on real GPUs: one process per GPU, fused wires against the one-GPU answer.

Runs the package's own self-check (``parallel/tp_check.py``) under the torch launcher on 2 GPUs (and 4
when the box has them); it passes when logits agree with the one-GPU run within rounding, the
teacher-forced tokens agree, and every rank holds identical tokens and residual bits.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world: int, extra):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29640 + world), "-m", "b200serve.parallel.tp_check"] + extra
    p = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    lines = [l for l in p.stdout.splitlines() if l.startswith("{")]
    assert p.returncode == 0 and lines, p.stdout[-2000:] + p.stderr[-2000:]
    return json.loads(lines[-1])


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_tp_decode_matches_one_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    rep = _run(world, ["--model", "small-dense", "--check"])
    for mode in ("fused", "nccl"):
        assert rep[mode]["ok"], rep
        assert rep[mode]["ranks_same_tokens"] and rep[mode]["ranks_same_residual"]


@pytest.mark.gpu
@pytest.mark.parametrize("prompt", [40, 600])
def test_draft_heads_under_tensor_parallelism(prompt):
    """MTP chain and block drafter with the head sliced over two ranks: greedy drafts + verify + accept give the tokens
    of the same sharded engine decoding plainly; every rank proposes the same drafts (the block drafter merges the
    candidates of the ranks' vocabulary slices).  The longer prompt goes through the fused prompt pass, whose hidden
    rows are gathered for the head's ingestion."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    rep = _run(2, ["--model", "small-dense", "--spec", "--prompt", str(prompt)])
    for kind in ("spec_mtp", "spec_dflash"):
        assert rep[kind]["ok"], rep
        assert rep[kind]["tokens_equal_plain"] and rep[kind]["ranks_same_tokens"] and rep[kind]["ranks_same_drafts"]

"""bench.py's contract pieces that need no GPU: the reference arm's `unavailable` line and the flag defaults."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_prints_unavailable_and_exits_zero():
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2",
                        "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert p.returncode == 0
    line = json.loads(p.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 20


def test_defaults_are_one_gpu_and_at_least_three_warmups():
    src = open(os.path.join(ROOT, "bench.py")).read()
    assert '"--gpus", type=int, default=1' in src
    assert '"--warmup", type=int, default=4' in src
    for key in ('"metric"', '"value"', '"n_gpus"', '"ms_per_step"', '"higher_is_better"', '"scaling"', '"vs_baseline"',
                '"dtype"', '"data"', '"config"', '"clocks"', '"e2e"', '"gpu_launches"'):
        assert key in src, key

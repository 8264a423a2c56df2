"""The measurement tools run end to end on small inputs (they are what the profiles' commands call)."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args):
    out = subprocess.run([sys.executable, "-m"] + args, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


def test_shapes_tool_decode_prefill_and_moe(cuda, tbl):
    d = _run(["reimagined_b200.shapes", "--m", "2", "--n", "512", "--k", "768", "--iters", "3"])
    assert d["device_status"] == 0 and d["us_per_call"] > 0
    d = _run(["reimagined_b200.shapes", "--m", "130", "--n", "256", "--k", "512", "--iters", "2", "--no-graph"])
    assert d["device_status"] == 0 and d["tops"] > 0
    d = _run(["reimagined_b200.shapes", "--moe", "--m", "40", "--k", "256", "--n", "512", "--experts", "4", "--iters", "2"])
    assert d["device_status"] == 0 and d["kernel_launches"] == 6


def test_decode_step_tool(cuda, tbl):
    d = _run(["reimagined_b200.decode_step", "--batch", "2", "--iters", "2"])
    assert d["device_status"] == 0 and d["linears"] == 107 and d["ternary_weights"] == 96043008
    assert d["kernel_launches_per_step"] <= 43

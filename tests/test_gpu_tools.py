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


def test_decode_and_chain_tools(cuda, tbl):
    """The decode timing tool (a small context so that it stays quick) and the stack timing tool."""
    d = _run(["reimagined_b200.decode", "--batch", "2", "--iters", "2", "--context", "4"])
    assert d["device_status"] == 0 and d["ternary_weights"] == 96043008 and d["kernel_launches_per_step"] > 0
    d = _run(["reimagined_b200.shapes", "--chain", "3", "--m", "1", "--n", "1024", "--k", "1024", "--iters", "2"])
    assert d["device_status"] == 0 and d["kernel_launches"] == 1
    d = _run(["reimagined_b200.shapes", "--norm", "--m", "600", "--k", "1536", "--gated", "--codes", "only", "--iters", "2"])
    assert d["device_status"] == 0 and d["row_norm"]


def test_layers_loaded_from_an_edge_pack_run_bit_exact(cuda, port, tbl, tmp_path):
    """Pack file -> BitLinear mirror -> device -> forward, against the oracle on the packed state."""
    import numpy as np
    import torch
    from reimagined_b200 import edge_pack
    rng = np.random.default_rng(11)
    layers = []
    for (n, k, bias) in [(96, 768, True), (40, 256, False)]:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        words, scale, *_ = port.pack_weights(w)
        layers.append({"sensitive": False, "in_features": k, "out_features": n, "use_bias": bias,
                       "weight_scale": np.float32(scale), "packed_weights": np.asarray(words, np.uint32),
                       "magnitude": (1 + 0.1 * rng.standard_normal(n)).astype(np.float32),
                       "bias": rng.standard_normal(n).astype(np.float32) if bias else np.zeros(0, np.float32),
                       "flat_alpha": np.ones(k, np.float32), "flat_beta": np.zeros(k, np.float32), "weight": None})
    path = tmp_path / "model.edge"
    edge_pack.save(str(path), layers)
    for layer in edge_pack.load(str(path)):
        lin = edge_pack.to_bitlinear(layer).to("cuda")
        lin.rms_mode = 2          # reference-order RMSNorm: bit-identical to the CPU path
        for m in (1, 5, 70):
            x = rng.standard_normal((m, layer["in_features"])).astype(np.float32)
            want = port.linear_forward(x, layer["packed_weights"], layer["weight_scale"], layer["out_features"],
                                       rms_input=1, magnitude=layer["magnitude"],
                                       bias=layer["bias"] if layer["use_bias"] else None)[0]
            got = lin.forward(torch.from_numpy(x).cuda()).cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (layer["out_features"], m)

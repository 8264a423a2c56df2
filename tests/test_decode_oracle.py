"""Pins of the model-level pieces to the reference's own model code (CPU only).

  * oracle/decode.py (one streaming decode step composed from the C port: norms, five Mamba-2 projections, conv
    step, SSD step, gated norm, attention over the KV cache, FFN, gates, LM head) against
    JambaModel::forward_ids_last, bit for bit, residual stream after every block included: from the committed
    fixture, and live against oracle/_ref/libnsos_model_ref.so where that library exists;
  * the edge-linear pack reader / writer against a pack written by JambaModel::save_edge_linear_pack;
  * the router post-processing against MoERouter::forward.
"""
import os

import numpy as np
import pytest

from conftest import GOLDEN_DIR


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def load_decode_fixture():
    g = dict(np.load(os.path.join(GOLDEN_DIR, "decode_tiny.npz")))
    params = {k[len("param:"):]: v for k, v in g.items() if k.startswith("param:")}
    return g, params


def test_port_decoder_matches_the_reference_model_fixture(port):
    from oracle.decode import PortDecoder
    g, params = load_decode_fixture()
    dec = PortDecoder(params, rows=1, capacity=64)
    for i, tok in enumerate(g["tokens"]):
        hidden, logits = dec.step([int(tok)])
        assert bits_equal(hidden[:, 0], g["hidden"][i]), f"token {i}: residual stream differs"
        assert bits_equal(logits[0], g["logits"][i]), f"token {i}: logits differ"


def test_port_decoder_rows_are_independent_sequences(port):
    """A batch of three sequences equals three single-sequence decoders (state is per row)."""
    from oracle.decode import PortDecoder
    g, params = load_decode_fixture()
    seqs = [[5, 90, 17, 3], [1, 1, 2, 95], [63, 0, 8, 8]]
    batch = PortDecoder(params, rows=3, capacity=16)
    singles = [PortDecoder(params, rows=1, capacity=16) for _ in seqs]
    for t in range(4):
        _, lb = batch.step([s[t] for s in seqs])
        for r, dec in enumerate(singles):
            _, l1 = dec.step([seqs[r][t]])
            assert bits_equal(lb[r], l1[0])


@pytest.mark.parametrize("cfg", [
    dict(num_layers=8, d_model=256, vocab_size=512, n_heads=4, n_kv_heads=4, mamba_d_state=16, mamba_expand=2,
         mamba_conv_kernel=4, mamba_head_dim=64, mamba_n_groups=1, attention_period=8, attention_slot=7),
    dict(num_layers=4, d_model=128, vocab_size=200, n_heads=2, n_kv_heads=1, mamba_d_state=16, mamba_expand=2,
         mamba_conv_kernel=4, mamba_head_dim=64, mamba_n_groups=1, attention_period=2, attention_slot=1),
], ids=["d256_l8", "d128_l4_gqa"])
def test_port_decoder_matches_the_live_reference_model(port, cfg):
    import oracle
    from oracle.decode import PortDecoder
    if not oracle.model_ref_available():
        pytest.skip("oracle/_ref/libnsos_model_ref.so not built (needs the reference checkout)")
    MR = oracle.model_ref()
    api, blocks = MR.model(cfg, seed=7), MR.model(cfg, seed=7)
    dec = PortDecoder(api.export(), rows=1, capacity=32)
    rng = np.random.default_rng(0)
    for tok in rng.integers(0, cfg["vocab_size"], 6):
        want = api.step(int(tok))                        # JambaModel::forward_ids_last
        hidden, want2 = blocks.step_trace(int(tok))      # the same step block by block
        assert bits_equal(want, want2)
        got_hidden, got = dec.step([int(tok)])
        assert bits_equal(got_hidden[:, 0], hidden)
        assert bits_equal(got[0], want)
    api.close()
    blocks.close()


def test_edge_pack_written_by_the_reference_model(tbl):
    """tests/golden/edge_pack_tiny.bin was written by JambaModel::save_edge_linear_pack: the reader must hand
    back the model's own packed states (in collect_bitlinear_layers order) and the writer must reproduce the
    file byte for byte."""
    from reimagined_b200 import edge_pack
    with open(os.path.join(GOLDEN_DIR, "edge_pack_tiny.bin"), "rb") as f:
        image = f.read()
    layers = edge_pack.loads(image)
    _, params = load_decode_fixture()
    order = ["head"] + [f"L0.mamba.{n}" for n in ("x", "z", "B", "C", "dt", "out")] + \
            [f"L1.attn.{n}" for n in ("q", "kv", "out")] + [f"L1.mamba.{n}" for n in ("x", "z", "B", "C", "dt", "out")] + \
            ["L1.ffn.up", "L1.ffn.down"]
    assert len(layers) == len(order)
    for layer, name in zip(layers, order):
        meta = params[name + ".meta"]
        assert (layer["in_features"], layer["out_features"], int(layer["use_bias"])) == tuple(int(v) for v in meta[:3])
        assert not layer["sensitive"] and layer["version"] == 3
        assert np.array_equal(layer["packed_weights"], params[name + ".words"])
        assert bits_equal(layer["weight_scale"], params[name + ".scale"][0])
        assert bits_equal(layer["magnitude"], params[name + ".magnitude"])
        if layer["use_bias"]:
            assert bits_equal(layer["bias"], params[name + ".bias"])
    assert edge_pack.dumps(layers) == image


@pytest.mark.parametrize("name", ["router_40x64_e8_top2", "router_9x32_e4_top1"])
def test_router_matches_moe_router_forward(port, name):
    """MoERouter::forward = gate (a default-mode BitLinear kept on the fp32 path) -> softmax -> top-k mask ->
    renormalise; the restated post-processing must reproduce its routing weights from its logits."""
    g = dict(np.load(os.path.join(GOLDEN_DIR, name + ".npz")))
    got = port.router_topk(g["logits"], int(g["top_k"]))
    assert np.array_equal(got != 0, g["weights"] != 0), "different experts kept (ties go to the lower index)"
    assert bits_equal(got, g["weights"])
    assert (g["weights"] != 0).sum(axis=1).tolist() == [int(g["top_k"])] * g["weights"].shape[0]


def test_pack_to_layers_and_back_is_byte_identical(tbl):
    """edge pack -> BitLinear mirror objects -> exported states -> edge pack: nothing is lost on the way."""
    from reimagined_b200 import edge_pack
    with open(os.path.join(GOLDEN_DIR, "edge_pack_tiny.bin"), "rb") as f:
        image = f.read()
    layers = [edge_pack.to_bitlinear(rec) for rec in edge_pack.loads(image)]
    assert edge_pack.dumps([edge_pack.from_bitlinear(lin) for lin in layers]) == image

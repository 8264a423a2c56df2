"""The C oracle against (a) the committed golden vectors produced by the reference's own C++ and
(b) the reference build itself where it is available.  CPU only."""
import numpy as np
import pytest

from conftest import golden_cases, load_golden

LINEAR = [p for p in golden_cases() if "moe_" not in p]


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


@pytest.mark.parametrize("path", LINEAR, ids=lambda p: p.split("/")[-1][:-4])
def test_port_matches_golden(port, path):
    g = load_golden(path)
    N, K = int(g["N"]), int(g["K"])
    words, scale, t, row_sums = port.pack_weights(g["w"])
    assert np.array_equal(words, g["words"]), "2-bit packing differs from the reference"
    assert bits_equal(scale, g["weight_scale"])
    assert np.array_equal(port.unpack_i8(words, N, K), t)
    assert np.array_equal(row_sums, t.astype(np.int32).sum(axis=1))
    exact = bool(g["exact_linear"])
    mag = g.get("magnitude") if not exact else None
    bias = g.get("bias")
    y, q, sc, acc = port.linear_forward(g["x"], words, scale, N, rms_input=0 if exact else 1,
                                        bits=int(g["bits"]), magnitude=mag, bias=bias)
    assert bits_equal(y, g["y"]), f"max abs diff {np.abs(y - g['y']).max()}"
    # the debug outputs are self-consistent with y
    assert np.array_equal(acc, q.astype(np.int32) @ t.astype(np.int32).T)
    assert np.abs(q).max() <= 127


def test_port_moe_matches_golden(port):
    g = load_golden([p for p in golden_cases() if "moe_" in p][0])
    E, H, D = g["up"].shape
    ups, dns, us, ds = [], [], [], []
    for e in range(E):
        w, s, _, _ = port.pack_weights(g["up"][e]); ups.append(w); us.append(s)
        w, s, _, _ = port.pack_weights(g["down"][e]); dns.append(w); ds.append(s)
    out = port.moe_forward(g["x"], g["routing"], ups, us, dns, ds, H, rms_input=1)
    assert bits_equal(out, g["out"]), f"max abs diff {np.abs(out - g['out']).max()}"


@pytest.mark.parametrize("N,K,M", [(768, 768, 1), (40, 16, 2), (7, 1000, 3), (130, 520, 9), (5, 4100, 1)])
@pytest.mark.parametrize("exact", [True, False])
def test_port_matches_reference_build(port, ref, N, K, M, exact):
    rng = np.random.default_rng(1000 + N + K + M)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.1, 30)).astype(np.float32)
    mag = None if exact else (1 + 0.2 * rng.standard_normal(N)).astype(np.float32)
    bias = None if exact else rng.standard_normal(N).astype(np.float32)
    words, scale, _, _ = port.pack_weights(w)
    rwords, rscale = ref.pack(w)
    assert np.array_equal(words, rwords) and bits_equal(scale, rscale)
    y, *_ = port.linear_forward(x, words, scale, N, rms_input=0 if exact else 1, magnitude=mag, bias=bias)
    yr = ref.linear_forward(w, x, exact_linear=exact, magnitude=mag, bias=bias)
    assert bits_equal(y, yr)


def test_tie_rule(port):
    # max |x| = 127 makes scale exactly 1.0f (127 + 1e-8f == 127.0f): ties are decided by the rule
    x = np.zeros((1, 16), np.float32)
    x[0, :8] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5]
    q_even, sc = port.quantize_rows(x, tie_mode=0)
    q_away, _ = port.quantize_rows(x, tie_mode=1)
    assert list(q_even[0, :8]) == [127, 0, 2, 2, 0, -2, -2, 4]
    assert list(q_away[0, :8]) == [127, 1, 2, 3, -1, -2, -3, 4]
    assert sc[0] == np.float32(1.0)
    # default build: K % 8 tail uses round-half-away
    xt = np.zeros((1, 12), np.float32)
    xt[0, 0] = 127.0; xt[0, 1] = 0.5; xt[0, 9] = 0.5; xt[0, 10] = 2.5
    qt, _ = port.quantize_rows(xt, tie_mode=0)
    assert qt[0, 1] == 0 and qt[0, 9] == 1 and qt[0, 10] == 3


def test_zero_row_and_router(port):
    x = np.zeros((2, 32), np.float32)
    q, sc = port.quantize_rows(x)
    assert not q.any() and np.all(sc == np.float32(np.float32(1e-8) / np.float32(127.0)))
    logits = np.array([[0.1, 0.1, 0.3, 0.3], [1, 2, 3, 4]], np.float32)
    w = port.router_topk(logits, 2)
    assert (w != 0).sum(axis=1).tolist() == [2, 2]
    assert w[0, 2] != 0 and w[0, 3] != 0 and w[1, 2] != 0 and w[1, 3] != 0
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)


@pytest.mark.parametrize("N,K,M,rms", [(33, 48, 3, 0), (130, 520, 9, 1), (64, 4096, 5, 1), (17, 16384, 2, 0)])
def test_fast_form_matches_port(port, N, K, M, rms):
    """oracle/fast.py (BLAS products of the codes, exact below 2^24) against the scalar C restatement."""
    from oracle import fast
    rng = np.random.default_rng(N * 7 + K + M)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.1, 30)).astype(np.float32)
    mag = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    words, scale, t, _ = port.pack_weights(w)
    y, q, sc, acc = port.linear_forward(x, words, scale, N, rms_input=rms, magnitude=mag, bias=bias)
    fy, fq, fsc, facc = fast.linear_forward(x, t, scale, rms_input=rms, magnitude=mag, bias=bias)
    assert np.array_equal(fq, q) and bits_equal(fsc, sc) and np.array_equal(facc, acc)
    assert bits_equal(fy, y)
    # worst case for exactness: every product at its extreme
    qx = np.full((2, K), 127, np.int8)
    tx = np.ones((3, K), np.int8)
    assert np.array_equal(fast.acc_exact(qx, tx), np.full((2, 3), 127 * K, np.int32))


def test_fast_moe_matches_port(port):
    from oracle import fast
    g = load_golden([p for p in golden_cases() if "moe_" in p][0])
    E, H, D = g["up"].shape
    up_t, dn_t, us, ds = [], [], [], []
    for e in range(E):
        _, s, t, _ = port.pack_weights(g["up"][e]); up_t.append(t); us.append(s)
        _, s, t, _ = port.pack_weights(g["down"][e]); dn_t.append(t); ds.append(s)
    out = fast.moe_forward(g["x"], g["routing"], up_t, us, dn_t, ds, rms_input=1)
    assert bits_equal(out, g["out"]), f"max abs diff {np.abs(out - g['out']).max()}"

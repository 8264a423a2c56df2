"""GPU parity at the sizes the benchmark configurations name, every output compared bit for bit.

The scalar C oracle needs minutes at these sizes, so the expected values come from oracle/fast.py: the same
floating-point steps (reference-order RMSNorm, per-row quantiser, epilogue order) with the integer dot products
taken by float32 BLAS on the codes, which is exact while 127*K < 2^24 (tests/test_oracle.py pins that form to
the C restatement).  Covered here:

  * the standalone sweep, K = N in {4096, 8192, 16384}: M in {1, 16, 128} on the 2-bit strip path and
    M in {1024, 8192} on the tcgen05 GEMM, full output compared;
  * the 8-expert top-2 FFN, D = 2048, H = 5632, 256 tokens N(0,1) rounded to bf16, seed 3, default-mode
    experts (input RMSNorm in the reference's summation order), on the grouped tcgen05 path and on the 2-bit
    strip path.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def _pack_with_library(tbl, w):
    """The product packer (host C++): canonical words + weight_scale."""
    N, K = w.shape
    w = np.ascontiguousarray(w, np.float32)
    words = np.zeros(tbl.tbl_packed_words(N, K), dtype=np.uint32)
    scale = np.zeros(1, np.float32)
    rc = tbl.tbl_pack_weights(w.ctypes.data, N, K, words.ctypes.data, scale.ctypes.data)
    assert rc == 0, rc
    return words, scale[0]


_matrices = {}


def _matrix(tbl, port, size):
    """One N(0,0.02) matrix per size, packed by the library, unpacked by the oracle; kept for the module."""
    import gpu_helpers as H
    if size not in _matrices:
        _matrices.clear()                      # one size resident at a time (16384^2 is 1 GB of fp32 on the host)
        rng = np.random.default_rng(5000 + size)
        w = rng.standard_normal((size, size), dtype=np.float32)
        w *= np.float32(0.02)
        words, scale = _pack_with_library(tbl, w)
        del w
        t = port.unpack_i8(words, size, size)
        assert 0.25 < float((t == 0).mean()) < 0.37          # about 31 % zeros for N(0, s) under the absmean rule
        dwords = H.words_dev(words)
        strips = H.relayout_strips(dwords, size, size)
        _matrices[size] = {"words": dwords, "scale": scale, "t": t, "strips": strips, "i8": None}
    return _matrices[size]


@pytest.mark.parametrize("M", [1, 16, 128, 1024, 8192])
@pytest.mark.parametrize("size", [4096, 8192, 16384])
def test_sweep_grid_at_full_size(cuda, port, tbl, size, M):
    import gpu_helpers as H
    from oracle import fast
    mat = _matrix(tbl, port, size)
    rng = np.random.default_rng(size + M)
    x = rng.standard_normal((M, size), dtype=np.float32)
    gemm = M > 64
    if gemm and mat["i8"] is None:
        mat["i8"] = H.expand_i8(mat["words"], size, size)
    y = H.linear_forward(H.dev(x), mat["words"], mat["scale"], size, w_i8=mat["i8"] if gemm else None,
                         strips=None if gemm else mat["strips"]).cpu().numpy()
    want, *_ = fast.linear_forward(x, mat["t"], mat["scale"])
    assert bits_equal(y, want), f"K=N={size} M={M}: {int((y != want).sum())} of {y.size} outputs differ"
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K", [(5000, 7680, 512), (4999, 7712, 640), (9000, 4200, 256)])
def test_tall_tiles_with_ragged_edges(cuda, port, tbl, M, N, K):
    """Large prefill problems run on 256 x 256 tiles (two accumulator halves per tile); rows and columns that
    do not fill the last tile, and a last group of row tiles shorter than the others."""
    import gpu_helpers as H
    from oracle import fast
    rng = np.random.default_rng(M + N + K)
    w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
    words, scale = _pack_with_library(tbl, w)
    t = port.unpack_i8(words, N, K)
    dwords = H.words_dev(words)
    i8 = H.expand_i8(dwords, N, K)
    x = rng.standard_normal((M, K), dtype=np.float32)
    y = H.linear_forward(H.dev(x), dwords, scale, N, w_i8=i8).cpu().numpy()
    want, *_ = fast.linear_forward(x, t, scale)
    assert bits_equal(y, want), f"M={M} N={N} K={K}: {int((y != want).sum())} of {y.size} outputs differ"
    assert H.device_status() == 0


@pytest.mark.parametrize("size,M", [(8192, 128), (16384, 64), (16384, 128)])
def test_sweep_grid_two_bit_weights_only(cuda, port, tbl, size, M):
    """The same layer without its int8 expansion: every M must still be served from the 2-bit strips."""
    import gpu_helpers as H
    from oracle import fast
    mat = _matrix(tbl, port, size)
    rng = np.random.default_rng(size * 3 + M)
    x = rng.standard_normal((M, size), dtype=np.float32)
    y = H.linear_forward(H.dev(x), mat["words"], mat["scale"], size, strips=mat["strips"]).cpu().numpy()
    want, *_ = fast.linear_forward(x, mat["t"], mat["scale"])
    assert bits_equal(y, want)
    assert H.device_status() == 0


@pytest.mark.parametrize("path", ["grouped_tcgen05", "strips"])
def test_expert_ffn_at_full_size(cuda, port, tbl, path):
    """256 decode tokens through 8 experts (top-2) of 2048 -> 5632 -> 2048 with squared ReLU.  The routing
    weights come from the oracle's router on an fp32 gate (the reference keeps that layer in fp32)."""
    import gpu_helpers as H
    import torch
    from oracle import fast
    _matrices.clear()
    rows, D, Hd, E, top_k = 256, 2048, 5632, 8, 2
    rng = np.random.default_rng(3)
    x = torch.from_numpy(rng.standard_normal((rows, D), dtype=np.float32)).bfloat16().float().numpy()
    gate = (rng.standard_normal((E, D), dtype=np.float32) * np.float32(0.02))
    logits = port.rmsnorm_rows(x, 1e-6) @ gate.T
    routing = port.router_topk(logits.astype(np.float32), top_k)
    counts = (routing != 0).sum(axis=0)
    assert counts.sum() == rows * top_k and counts.min() > 16          # near-uniform load, all experts active
    views_up, views_down, keep, up_t, dn_t, us, ds = [], [], [], [], [], [], []
    for e in range(E):
        for (n, k, views, ts, ss) in ((Hd, D, views_up, up_t, us), (D, Hd, views_down, dn_t, ds)):
            w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
            words, scale = _pack_with_library(tbl, w)
            ts.append(port.unpack_i8(words, n, k)); ss.append(scale)
            dw = H.words_dev(words)
            st = H.relayout_strips(dw, n, k) if path == "strips" else None
            i8 = H.expand_i8(dw, n, k) if path == "grouped_tcgen05" else None
            keep += [dw, st, i8]
            views.append(H.make_view(dw, k, n, scale, rms_input=1, strips=st, w_i8=i8))
    want = fast.moe_forward(x, routing, up_t, us, dn_t, ds, rms_input=1)
    out = H.moe_forward(views_up + views_down, H.dev(routing), H.dev(x), Hd, top_k, rms_mode=2).cpu().numpy()
    assert bits_equal(out, want), f"{int((out != want).sum())} of {out.size} differ, max {np.abs(out - want).max()}"
    assert H.device_status() == 0

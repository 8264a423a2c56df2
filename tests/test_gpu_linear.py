"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and the golden
vectors produced by the reference.  Integer results (int8 codes, int32 accumulators) must be
bit-exact; fp32 outputs are compared bit-for-bit where the operation order is the reference's and
with rel 1e-5 otherwise."""
import numpy as np
import pytest

from conftest import golden_cases, load_golden

pytestmark = pytest.mark.gpu

REL = 1e-5  # tolerance north_star states for dequantised fp32 outputs


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def assert_close(y, ref, rel=REL):
    scale = np.abs(ref).max() + 1e-30
    assert np.abs(y - ref).max() <= rel * scale, f"max abs diff {np.abs(y - ref).max()} vs scale {scale}"


def make_case(seed, N, K, M, affine=False, xscale=1.0):
    rng = np.random.default_rng(seed)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((M, K)) * xscale).astype(np.float32)
    mag = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32) if affine else None
    bias = rng.standard_normal(N).astype(np.float32) if affine else None
    return w, x, mag, bias


@pytest.mark.parametrize("M,K", [(1, 16), (3, 48), (5, 52), (2, 768), (7, 4096), (64, 1024), (1, 16384)])
@pytest.mark.parametrize("bits", [8, 4, 2])
def test_quantize_rows_bit_exact(cuda, port, tbl, M, K, bits):
    import gpu_helpers as H
    rng = np.random.default_rng(M * 31 + K + bits)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.01, 50)).astype(np.float32)
    x[0, : min(K, 4)] = 0.0
    q, sc, sums = H.quantize_rows(H.dev(x), bits=bits)
    oq, osc = port.quantize_rows(x, bits=bits)
    assert np.array_equal(q.cpu().numpy(), oq)
    assert bits_equal(sc.cpu().numpy(), osc)
    assert np.array_equal(sums.cpu().numpy(), oq.astype(np.int32).sum(axis=1))
    assert H.device_status() == 0


@pytest.mark.parametrize("M,K", [(256, 2048), (300, 4096), (449, 8192), (256, 16384), (257, 8208), (1000, 12288)])
@pytest.mark.parametrize("bits,tie", [(8, 0), (4, 1)])
def test_quantize_rows_prefill_sized_bit_exact(cuda, port, tbl, M, K, bits, tie):
    """Many rows: the persistent streaming quantiser (K >= 8192: rows dealt round-robin to 148 CTAs, ragged
    last round, gathered rows, zero rows) and the one-CTA-per-row kernel below that, against the oracle."""
    import gpu_helpers as H
    rng = np.random.default_rng(M + K + bits)
    x = (rng.standard_normal((M, K)) * rng.uniform(0.01, 50, size=(M, 1))).astype(np.float32)
    x[5] = 0.0
    x[7, ::2] = 0.5 * np.abs(x[7]).max() / 127.0 * 3.0     # values on rounding boundaries
    idx = rng.permutation(M).astype(np.int32)
    q, sc, sums = H.quantize_rows(H.dev(x), bits=bits, tie_mode=tie, row_index=H.dev(idx))
    oq, osc = port.quantize_rows(x[idx], bits=bits, tie_mode=tie)
    assert np.array_equal(q.cpu().numpy(), oq)
    assert bits_equal(sc.cpu().numpy(), osc)
    assert np.array_equal(sums.cpu().numpy(), oq.astype(np.int32).sum(axis=1))
    assert H.device_status() == 0


def test_prefill_linear_reference_order_rms_wide_rows(cuda, port, tbl):
    """M > 64 at K = 8192 with the reference-order RMSNorm: rms kernel -> streaming quantiser -> tcgen05 GEMM."""
    import gpu_helpers as H
    N, K, M = 48, 8192, 200
    w, x, mag, bias = make_case(99, N, K, M, affine=True)
    words, scale, t, _ = port.pack_weights(w)
    oy, *_ = port.linear_forward(x, words, scale, N, rms_input=1, magnitude=mag, bias=bias)
    dwords = H.words_dev(words)
    y = H.linear_forward(H.dev(x), dwords, scale, N, w_i8=H.expand_i8(dwords, N, K), rms_mode=2,
                         magnitude=H.dev(mag), bias=H.dev(bias))
    assert bits_equal(y.cpu().numpy(), oy), f"max diff {np.abs(y.cpu().numpy() - oy).max()}"
    assert H.device_status() == 0


def test_quantize_ties_zero_rows_and_gather(cuda, port, tbl):
    import gpu_helpers as H
    x = np.zeros((3, 32), np.float32)
    x[0, :8] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5]
    x[2, :] = np.linspace(-3, 3, 32)
    for tie in (0, 1):
        q, sc, _ = H.quantize_rows(H.dev(x), tie_mode=tie)
        oq, osc = port.quantize_rows(x, tie_mode=tie)
        assert np.array_equal(q.cpu().numpy(), oq) and bits_equal(sc.cpu().numpy(), osc)
    idx = np.array([2, 0, 2, 1], np.int32)
    q, sc, _ = H.quantize_rows(H.dev(x), row_index=H.dev(idx))
    oq, osc = port.quantize_rows(x[idx])
    assert np.array_equal(q[:4].cpu().numpy(), oq)
    # RMS-normalised input, fast mode: codes may differ by one step only at rounding boundaries
    xr = np.random.default_rng(5).standard_normal((4, 2048)).astype(np.float32)
    q, sc, _ = H.quantize_rows(H.dev(xr), rms_mode=1)
    oq, osc = port.quantize_rows(port.rmsnorm_rows(xr))
    d = np.abs(q.cpu().numpy().astype(np.int32) - oq.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 1e-3
    np.testing.assert_allclose(sc.cpu().numpy(), osc, rtol=1e-6)


SMALL_SHAPES = [(768, 768), (33, 64), (17, 1024), (300, 2048), (129, 4096), (40, 5632), (24, 768),
                (16, 1536), (50, 3072), (9, 16384), (3, 32768), (1000, 256)]


@pytest.mark.parametrize("N,K", SMALL_SHAPES)
@pytest.mark.parametrize("M", [1, 2, 3, 4])
def test_fused_decode_gemv_small_m(cuda, port, tbl, N, K, M):
    """M <= 4: one kernel (quantiser fused into the streamed dp4a GEMV)."""
    import gpu_helpers as H
    w, x, mag, bias = make_case(N + K + M, N, K, M, affine=(N % 2 == 0))
    words, scale, t, _ = port.pack_weights(w)
    oy, oq, osc, oacc = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    before = tbl.tbl_launch_count()
    y = H.linear_forward(H.dev(x), H.words_dev(words), scale, N, magnitude=None if mag is None else H.dev(mag),
                         bias=None if bias is None else H.dev(bias))
    assert tbl.tbl_launch_count() - before == 1
    assert bits_equal(y.cpu().numpy(), oy), f"max diff {np.abs(y.cpu().numpy() - oy).max()}"
    assert H.device_status() == 0


@pytest.mark.parametrize("N,K", [(768, 768), (33, 64), (129, 4096), (40, 5632), (9, 16384), (17, 48), (5, 16)])
@pytest.mark.parametrize("M", [1, 3, 4])
def test_gemv_on_codes_int32_exact(cuda, port, tbl, N, K, M):
    """tbl_gemv on given int8 codes: int32 accumulators bit-exact, y bit-exact."""
    import gpu_helpers as H
    w, x, mag, bias = make_case(7 * N + K + M, N, K, M, affine=True, xscale=3.0)
    words, scale, t, _ = port.pack_weights(w)
    oq, osc = port.quantize_rows(x)
    oacc = oq.astype(np.int32) @ t.astype(np.int32).T
    oy, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    y, acc = H.gemv(H.dev(oq), H.dev(osc), H.words_dev(words), scale, N, H.dev(mag), H.dev(bias))
    assert np.array_equal(acc.cpu().numpy(), oacc)
    assert bits_equal(y.cpu().numpy(), oy)
    assert H.device_status() == 0


@pytest.mark.parametrize("N,K", [(768, 768), (1536, 768), (32000, 768), (100, 1024), (130, 2048), (16, 768),
                                 (2048, 5632), (64, 16384), (47, 256), (3000, 512)])
@pytest.mark.parametrize("M", [1, 2, 4, 5, 8, 16, 17, 33, 64])
def test_gemv_strip_tensor_path(cuda, port, tbl, N, K, M):
    """1 <= M <= 64 on the strip-major weights (mma.sync path): accumulators and outputs bit-exact."""
    import gpu_helpers as H
    if N * K * M > 3e9:
        pytest.skip("oracle too slow at this size")
    w, x, mag, bias = make_case(3 * N + K + M, N, K, M, affine=(M % 2 == 1))
    words, scale, t, _ = port.pack_weights(w)
    oq, osc = port.quantize_rows(x)
    oacc = oq.astype(np.int32) @ t.astype(np.int32).T
    oy, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    dm = None if mag is None else H.dev(mag)
    db = None if bias is None else H.dev(bias)
    dwords = H.words_dev(words)
    strips = H.relayout_strips(dwords, N, K)
    y, acc = H.gemv(H.dev(oq), H.dev(osc), None, scale, N, dm, db, strips=strips)
    assert np.array_equal(acc.cpu().numpy(), oacc)
    assert bits_equal(y.cpu().numpy(), oy)
    y2 = H.linear_forward(H.dev(x), None, scale, N, magnitude=dm, bias=db, strips=strips)
    assert bits_equal(y2.cpu().numpy(), oy)
    assert H.device_status() == 0


@pytest.mark.parametrize("N,K,M", [(100, 1024, 9), (33, 48, 12), (768, 768, 64), (17, 80, 5)])
def test_gemv_canonical_words_any_m(cuda, port, tbl, N, K, M):
    """Canonical words only (no strip copy): the generic kernel serves M > 4 and odd K."""
    import gpu_helpers as H
    w, x, mag, bias = make_case(N + K + M, N, K, M, affine=True)
    words, scale, t, _ = port.pack_weights(w)
    oq, osc = port.quantize_rows(x)
    oy, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    y, acc = H.gemv(H.dev(oq), H.dev(osc), H.words_dev(words), scale, N, H.dev(mag), H.dev(bias))
    assert np.array_equal(acc.cpu().numpy(), oq.astype(np.int32) @ t.astype(np.int32).T)
    assert bits_equal(y.cpu().numpy(), oy)


def test_strip_relayout_is_a_permutation(cuda, port, tbl):
    """Every canonical 16-byte chunk appears exactly once in the strip copy; padding rows are zero weights."""
    import gpu_helpers as H
    N, K = 40, 512
    words = np.arange(N * K // 16, dtype=np.uint32)  # distinct words (not valid codes: layout test only)
    strips = H.relayout_strips(H.words_dev(words), N, K).cpu().numpy().view(np.uint32).reshape(-1, 4)
    canon = words.reshape(-1, 4)
    pad = (strips == 0x55555555).all(axis=1)
    assert pad.sum() == (48 - N) * (K // 64)
    got = strips[~pad]
    order = np.lexsort(got.T[::-1])
    assert np.array_equal(got[order], canon[np.lexsort(canon.T[::-1])])
    # 1 KB block (strip s, k-block b) sits at slab-major position 4*(b//4)*S + s*4 + b%4 (K = 512: one
    # half slab of 2 blocks per strip): lane 4g+t holds chunk 4b+t of row 16s+g, rows +8 at +512 bytes
    cpr, S = K // 64, 3
    for s_ in range(S):
        for b in range(2):
            base = (s_ * 2 + b) * 64
            for g in range(8):
                for t_ in range(4):
                    for h in range(2):
                        row = 16 * s_ + 8 * h + g
                        got_chunk = strips[base + 32 * h + 4 * g + t_]
                        if row < N:
                            assert np.array_equal(got_chunk, canon[row * cpr + 4 * b + t_])
                        else:
                            assert (got_chunk == 0x55555555).all()


@pytest.mark.parametrize("M,N,K,rms", [(33, 136, 1536, 0), (48, 1000, 2560, 1), (64, 776, 1536, 2), (100, 300, 1024, 0),
                                       (128, 1024, 4096, 1), (40, 129, 512, 0), (64, 3352, 768, 0), (50, 200, 1280, 2),
                                       (128, 140, 256, 1), (200, 260, 768, 0)])
def test_mid_batch_widening_tensor_core_path(cuda, port, tbl, M, N, K, rms):
    """33 <= M <= 256 on the strip-major 2-bit weights with K % 256 == 0: widened in shared memory and multiplied by
    tcgen05 MMAs, up to 128 rows per pass; ragged row tiles, a short last slab (K % 1024 != 0), half a last k-block
    (K % 512 == 256: the plane-major codes are zero-padded), every RMS mode."""
    import gpu_helpers as H
    w, x, mag, bias = make_case(7 * M + N + K, N, K, M, affine=True, xscale=3.0)
    words, scale, *_ = port.pack_weights(w)
    oy, *_ = port.linear_forward(x, words, scale, N, rms_input=1 if rms else 0, magnitude=mag, bias=bias)
    dwords = H.words_dev(words)
    y = H.linear_forward(H.dev(x), dwords, scale, N, rms_mode=rms, magnitude=H.dev(mag), bias=H.dev(bias),
                         strips=H.relayout_strips(dwords, N, K)).cpu().numpy()
    if rms == 1:
        # parallel sum of squares: a code may move by one step at a rounding boundary -> bounded, tiny drift
        assert np.abs(y - oy).max() <= 2e-2 * np.abs(oy).max()
        assert np.median(np.abs(y - oy)) <= 1e-5 * np.abs(oy).max()
    else:
        assert bits_equal(y, oy)
    assert H.device_status() == 0


@pytest.mark.parametrize("M", [65, 100, 200])
def test_packed_path_for_large_m_without_int8_copy(cuda, port, tbl, M):
    """w_i8 == NULL: every M runs on the packed words (activation tiles of 64 per pass)."""
    import gpu_helpers as H
    N, K = 200, 512
    w, x, mag, bias = make_case(M, N, K, M, affine=True)
    words, scale, *_ = port.pack_weights(w)
    oy, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    dwords = H.words_dev(words)
    y = H.linear_forward(H.dev(x), dwords, scale, N, magnitude=H.dev(mag), bias=H.dev(bias))
    assert bits_equal(y.cpu().numpy(), oy)
    y = H.linear_forward(H.dev(x), None, scale, N, magnitude=H.dev(mag), bias=H.dev(bias),
                         strips=H.relayout_strips(dwords, N, K))
    assert bits_equal(y.cpu().numpy(), oy)


@pytest.mark.parametrize("path", [p for p in golden_cases() if "moe_" not in p and "tail_" not in p
                                 ], ids=lambda p: p.split("/")[-1][:-4])
def test_linear_forward_matches_reference_golden(cuda, tbl, path):
    """End to end against vectors computed by the reference's own C++ BitLinear::forward."""
    import gpu_helpers as H
    g = load_golden(path)
    N, K, M = int(g["N"]), int(g["K"]), int(g["M"])
    exact = bool(g["exact_linear"])
    mag = None if exact or "magnitude" not in g else H.dev(g["magnitude"])
    bias = None if "bias" not in g else H.dev(g["bias"])
    words = H.words_dev(g["words"])
    w_i8 = H.expand_i8(words, N, K) if M > 64 else None
    y = H.linear_forward(H.dev(g["x"]), words, float(g["weight_scale"]), N, w_i8=w_i8, bits=int(g["bits"]),
                         rms_mode=0 if exact else 2, magnitude=mag, bias=bias).cpu().numpy()
    assert bits_equal(y, g["y"]), f"max diff {np.abs(y - g['y']).max()}"
    if K % 256 == 0:
        ys = H.linear_forward(H.dev(g["x"]), None, float(g["weight_scale"]), N, bits=int(g["bits"]),
                              rms_mode=0 if exact else 2, magnitude=mag, bias=bias,
                              strips=H.relayout_strips(words, N, K)).cpu().numpy()
        assert bits_equal(ys, g["y"]), f"strip path max diff {np.abs(ys - g['y']).max()}"
    if not exact:
        yf = H.linear_forward(H.dev(g["x"]), words, float(g["weight_scale"]), N, w_i8=w_i8, bits=int(g["bits"]),
                              rms_mode=1, magnitude=mag, bias=bias).cpu().numpy()
        # parallel RMS sum: a code may move by one step at a rounding boundary -> bounded, tiny drift
        assert np.abs(yf - g["y"]).max() <= 2e-2 * np.abs(g["y"]).max()


def test_reference_gemv_contract_fixture(cuda, tbl):
    """The reference's own RNG-free GPU fixture (tests/gpu/test_gpu_decode_runtime.cpp:49-83):
    codes (n+k)%3, x = 0.4*sin(0.071*(i+1)), magnitude/bias patterns, bits 2/4/8, atol=rtol=2e-5."""
    import gpu_helpers as H

    def pattern(n, f):
        return (np.sin((np.arange(n, dtype=np.float32) + np.float32(1)) * np.float32(f)) * np.float32(0.4)).astype(np.float32)

    for K in (16, 48, 512, 1024):
        for N in (3, 17, 33):
            x = pattern(K, 0.071)
            n_idx, k_idx = np.meshgrid(np.arange(N), np.arange(K), indexing="ij")
            codes = ((n_idx + k_idx) % 3).astype(np.uint32)
            words = np.zeros((N, K // 16), np.uint32)
            for b in range(16):
                words |= codes[:, b::16] << np.uint32(2 * b)
            mag, bias = pattern(N, 0.12), pattern(N, 0.1)
            for bits in (2, 4, 8):
                qmax = np.float32((1 << (bits - 1)) - 1)
                denom = np.float32(np.abs(x).max() + np.float32(1e-8))
                q = np.round(x * (qmax / denom))  # fixture uses std::round
                acc = (q[None, :].astype(np.int64) * (codes.astype(np.int64) - 1)).sum(axis=1)
                ref = ((acc.astype(np.float32) * np.float32(0.3)) * (denom / qmax)) * mag + bias
                y = H.linear_forward(H.dev(x[None, :]), H.words_dev(words.reshape(-1)), 0.3, N, bits=bits,
                                     magnitude=H.dev(mag), bias=H.dev(bias)).cpu().numpy()[0]
                assert np.all(np.abs(y - ref) <= 2e-5 + 2e-5 * np.abs(ref)), (K, N, bits)


def test_roundtrip_properties_at_scale(cuda, port, tbl):
    """Size-independent checks at a benchmark-size shape (K=N=4096): linearity in the weight scale,
    zero input -> bias only, and a checksum of int32 accumulators against a row-sampled oracle."""
    import gpu_helpers as H
    N = K = 4096
    M = 16
    w, x, _, _ = make_case(99, N, K, M)
    words, scale, t, _ = port.pack_weights(w)
    dw = H.words_dev(words)
    oq, osc = port.quantize_rows(x)
    strips = H.relayout_strips(dw, N, K)
    y1, acc = H.gemv(H.dev(oq), H.dev(osc), None, scale, N, strips=strips)
    y2, _ = H.gemv(H.dev(oq), H.dev(osc), None, 2 * float(scale), N, strips=strips)
    assert bits_equal(y2.cpu().numpy(), 2 * y1.cpu().numpy())  # scaling by 2 is exact in fp32
    rows = np.random.default_rng(0).choice(N, 64, replace=False)
    oacc = oq.astype(np.int32) @ t[rows].astype(np.int32).T
    assert np.array_equal(acc.cpu().numpy()[:, rows], oacc)
    # checksum identity: sum_n acc[m,n] == q[m,:] . (sum_n t[n,:])
    col = t.astype(np.int64).sum(axis=0)
    assert np.array_equal(acc.cpu().numpy().astype(np.int64).sum(axis=1), oq.astype(np.int64) @ col)
    bias = np.random.default_rng(1).standard_normal(N).astype(np.float32)
    y0 = H.linear_forward(H.dev(np.zeros((2, K), np.float32)), dw, scale, N, bias=H.dev(bias)).cpu().numpy()
    assert bits_equal(y0, np.broadcast_to(bias, (2, N)))


@pytest.mark.parametrize("M", [1, 8, 200])
def test_checksums_at_full_size_16384(cuda, port, tbl, M):
    """K = N = 16384 (the bench's size; 64 MiB of packed weights, codes drawn on the device): the layer's
    outputs through the fused decode kernel (M = 1), the strip GEMV behind a separate quantiser (M = 8)
    and the tcgen05 GEMM (M = 200) agree with (i) the oracle on 48 sampled weight rows, bit for bit, and
    (ii) the checksum identity sum_n acc[m,n] = q[m,:] . sum_n t[n,:] over all 16384 columns."""
    import gpu_helpers as H
    import torch
    N = K = 16384
    gen = torch.Generator(device="cuda").manual_seed(16384 + M)
    codes = torch.randint(0, 3, (N, K), dtype=torch.int32, device="cuda", generator=gen)     # 0, 1, 2
    shifts = (2 * torch.arange(16, device="cuda", dtype=torch.int32)).view(1, 1, 16)
    words = (codes.view(N, K // 16, 16) << shifts).sum(dim=2, dtype=torch.int32).contiguous().view(-1)
    scale = 0.0159
    x = (np.random.default_rng(M).standard_normal((M, K)) * 1.7).astype(np.float32)
    oq, osc = port.quantize_rows(x)
    strips = H.relayout_strips(words, N, K)
    w_i8 = H.expand_i8(words, N, K) if M > 64 else None
    y = H.linear_forward(H.dev(x), words, scale, N, strips=strips, w_i8=w_i8).cpu().numpy()
    # (i) sampled rows against the integer oracle and the reference's epilogue
    rows = np.random.default_rng(7).choice(N, 48, replace=False)
    t_rows = (codes[torch.from_numpy(rows).cuda()].cpu().numpy().astype(np.int32) - 1)
    acc = oq.astype(np.int32) @ t_rows.T
    want = acc.astype(np.float32) * (osc[:, None] * np.float32(scale)).astype(np.float32)
    assert bits_equal(y[:, rows], want)
    # (ii) checksum over every column, from the raw accumulators of the GEMV / GEMM entry points
    col = (codes.to(torch.int64) - 1).sum(dim=0).cpu().numpy()
    if M <= 64:
        _, acc_all = H.gemv(H.dev(oq), H.dev(osc), None, scale, N, strips=strips)
    else:
        _, acc_all = H.gemm(H.dev(oq), H.dev(osc), w_i8, scale)
    assert np.array_equal(acc_all.cpu().numpy().astype(np.int64).sum(axis=1), oq.astype(np.int64) @ col)
    assert H.device_status() == 0


@pytest.mark.parametrize("K", [2048, 4096, 6144])
@pytest.mark.parametrize("M", [2, 5, 8, 9, 13, 16])
def test_few_row_pipelined_path_bit_exact(cuda, port, tbl, M, K):
    """2..16 rows with K a multiple of the 2048-deep stage: the unrolled, software-pipelined variant of the strip
    kernel (fused quantiser while rows*K <= 16384, staged activations above), ragged N, magnitude and bias."""
    import gpu_helpers as H
    N = {2048: 1000, 4096: 130, 6144: 17}[K]
    w, x, mag, bias = make_case(1000 * M + K, N, K, M, affine=True)
    words, scale, t, _ = port.pack_weights(w)
    oy, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    dwords = H.words_dev(words)
    y = H.linear_forward(H.dev(x), None, scale, N, magnitude=H.dev(mag), bias=H.dev(bias),
                         strips=H.relayout_strips(dwords, N, K)).cpu().numpy()
    assert bits_equal(y, oy), f"max diff {np.abs(y - oy).max()}"
    assert H.device_status() == 0

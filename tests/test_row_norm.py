"""Row norms either side of a linear (block RMSNorm x weight; SiLU gate -> RMSNorm x weight): the C restatement
against fixtures made by the reference's own Tensor ops, the reference build where present, and the CUDA kernel
(fp32 to 1e-5 relative; its fused int8 codes bit for bit what the stand-alone quantiser gives)."""
import numpy as np
import pytest

from conftest import golden_cases

REL_TOL = 1e-5      # fp32 tolerance of the path: the device sums squares as a tree and uses the device's expf
CASES = golden_cases("rownorm_")


def load(path):
    g = dict(np.load(path))
    return g["value"], g.get("gate"), g.get("weight"), float(g["eps"]), g["out"]


def close(a, b, tol=REL_TOL):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return bool(np.all(np.abs(a - b) <= tol * np.maximum(np.abs(b), 1e-3)))


def test_fixtures_present():
    assert len(CASES) == 4


@pytest.mark.parametrize("path", CASES, ids=lambda p: p.split("/")[-1][:-4])
def test_restatement_matches_the_reference_fixture_bit_for_bit(port, path):
    value, gate, weight, eps, want = load(path)
    got = port.row_norm(value, gate, weight, eps)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_restatement_matches_the_reference_build(port, ref):
    rng = np.random.default_rng(5)
    for rows, dim in [(1, 1), (2, 7), (3, 768), (1, 4100)]:
        value = rng.standard_normal((rows, dim)).astype(np.float32)
        gate = (4 * rng.standard_normal((rows, dim))).astype(np.float32)
        gate[0, 0] = -90.0          # exp(-gate) overflows the one-sided sigmoid; the two-sided one gives 0
        weight = rng.standard_normal(dim).astype(np.float32)
        for g in (None, gate):
            for w in (None, weight):
                a, b = port.row_norm(value, g, w, 1e-5), ref.row_norm(value, g, w, 1e-5)
                assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_entry_point_validates_before_touching_a_device(tbl):
    f = tbl.tbl_row_norm
    assert f(None, None, None, 4, 64, 1e-5, 0x1000, 8, None, None, None, None) == -1          # no input
    assert f(0x1000, None, None, 4, 64, 1e-5, None, 8, None, None, None, None) == -1         # no output at all
    assert f(0x1000, None, None, 4, 64, 0.0, 0x2000, 8, None, None, None, None) == -1        # eps must be > 0
    assert f(0x1000, None, None, 4, 64, float("nan"), 0x2000, 8, None, None, None, None) == -1
    assert f(0x1000, None, None, 0, 64, 1e-5, 0x2000, 8, None, None, None, None) == -1
    assert f(0x1000, None, None, 4, 49153, 1e-5, 0x2000, 8, None, None, None, None) == -2    # row too long to cache
    assert f(0x1000, None, None, 4, 72, 1e-5, None, 8, 0x3000, 0x4000, None, None) == -2     # codes need dim % 16 == 0
    assert f(0x1000, None, None, 4, 64, 1e-5, None, 8, 0x3000, None, None, None) == -1       # codes without scales
    assert f(0x1000, None, None, 4, 64, 1e-5, None, 9, 0x3000, 0x4000, None, None) == -5     # TBL_ERR_BITS


def run(H, value, gate, weight, eps, want_out=True, want_q=False, bits=8):
    import torch
    from reimagined_b200 import capi
    L = capi.lib()
    rows, dim = value.shape
    dv = H.dev(value)
    dg = None if gate is None else H.dev(gate)
    dw = None if weight is None else H.dev(weight)
    out = torch.empty((rows, dim), dtype=torch.float32, device="cuda") if want_out else None
    q = torch.empty((rows, dim), dtype=torch.int8, device="cuda") if want_q else None
    sc = torch.empty(rows, dtype=torch.float32, device="cuda") if want_q else None
    sums = torch.empty(rows, dtype=torch.int32, device="cuda") if want_q else None
    capi.check(L.tbl_row_norm(H.ptr(dv), H.ptr(dg), H.ptr(dw), rows, dim, eps, H.ptr(out), bits, H.ptr(q), H.ptr(sc),
                              H.ptr(sums), H.stream_ptr()), "tbl_row_norm")
    return out, q, sc, sums


@pytest.mark.gpu
@pytest.mark.parametrize("path", CASES, ids=lambda p: p.split("/")[-1][:-4])
def test_kernel_matches_the_reference_fixture(cuda, tbl, path):
    import gpu_helpers as H
    value, gate, weight, eps, want = load(path)
    out, *_ = run(H, value, gate, weight, eps)
    assert close(out.cpu().numpy(), want)
    assert H.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("rows,dim", [(1, 768), (8, 1536), (64, 3072), (5, 33), (3, 1), (2, 16384), (1, 49152),
                                      (700, 2048), (1500, 1536), (2000, 768), (515, 36), (600, 1028)])
@pytest.mark.parametrize("gated", [False, True])
def test_kernel_matches_the_oracle(cuda, port, tbl, rows, dim, gated):
    import gpu_helpers as H
    rng = np.random.default_rng(rows * 131 + dim)
    value = rng.standard_normal((rows, dim)).astype(np.float32)
    gate = (3 * rng.standard_normal((rows, dim))).astype(np.float32) if gated else None
    if gated:
        gate[0, 0] = -95.0
    weight = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    for w in (weight, None):
        want = port.row_norm(value, gate, w, 1e-5)
        out, *_ = run(H, value, gate, w, 1e-5)
        # the CPU reference sums the squares one by one in fp32, and that sum itself drifts by about sqrt(dim)
        # half-ulps: beyond 16384 elements it is the oracle, not the kernel's tree, that leaves 1e-5
        tol = REL_TOL if dim <= 16384 else 5e-5
        assert close(out.cpu().numpy(), want, tol), np.abs(out.cpu().numpy() - want).max()
    assert H.device_status() == 0


@pytest.mark.gpu
@pytest.mark.parametrize("rows,dim,bits", [(1, 768, 8), (8, 1536, 8), (64, 3072, 8), (3, 16, 8), (5, 1536, 4),
                                           (300, 4096, 8), (600, 1536, 8), (1030, 768, 8), (513, 48, 3),
                                           (520, 2048, 8)])
@pytest.mark.parametrize("gated", [False, True])
def test_fused_codes_are_the_quantiser_on_the_stored_values(cuda, tbl, rows, dim, bits, gated):
    """One launch gives the fp32 row and its int8 codes; the codes, scales and sums equal tbl_quantize_rows
    of that fp32 row bit for bit, with or without the fp32 store."""
    import gpu_helpers as H
    rng = np.random.default_rng(rows + dim + bits)
    value = rng.standard_normal((rows, dim)).astype(np.float32)
    gate = (3 * rng.standard_normal((rows, dim))).astype(np.float32) if gated else None
    weight = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    out, q, sc, sums = run(H, value, gate, weight, 1e-5, want_q=True, bits=bits)
    q2, sc2, sums2 = H.quantize_rows(out, bits=bits)
    assert cuda.equal(q, q2) and cuda.equal(sc.view(cuda.int32), sc2.view(cuda.int32)) and cuda.equal(sums, sums2)
    _, q3, sc3, sums3 = run(H, value, gate, weight, 1e-5, want_out=False, want_q=True, bits=bits)
    assert cuda.equal(q, q3) and cuda.equal(sc.view(cuda.int32), sc3.view(cuda.int32)) and cuda.equal(sums, sums3)
    assert H.device_status() == 0


@pytest.mark.gpu
def test_gated_norm_feeds_the_out_projection_without_an_fp32_round_trip(cuda, port, tbl):
    """Mamba-2 epilogue of the decode step: gate -> norm -> codes in one launch, then the 1536 -> 768
    out-projection on the codes, equals norm -> fp32 -> tbl_linear_forward bit for bit."""
    import gpu_helpers as H
    rng = np.random.default_rng(77)
    rows, dim, n = 8, 1536, 768
    value = rng.standard_normal((rows, dim)).astype(np.float32)
    gate = (2 * rng.standard_normal((rows, dim))).astype(np.float32)
    weight = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    w = (rng.standard_normal((n, dim)) * 0.02).astype(np.float32)
    words, scale, *_ = port.pack_weights(w)
    dwords = H.words_dev(words)
    strips = H.relayout_strips(dwords, n, dim)
    before = tbl.tbl_launch_count()
    out, q, sc, _ = run(H, value, gate, weight, 1e-5, want_q=True)
    assert tbl.tbl_launch_count() - before == 1
    y_codes, _ = H.gemv(q, sc, None, scale, n, want_acc=False, strips=strips)
    y_fp32 = H.linear_forward(out, None, scale, n, strips=strips)
    assert cuda.equal(y_codes.view(cuda.int32), y_fp32.view(cuda.int32))
    # and the whole chain against the CPU restatement of the same composition
    want = port.linear_forward(port.row_norm(value, gate, weight, 1e-5), words, scale, n)[0]
    got = y_fp32.cpu().numpy()
    assert np.abs(got - want).max() <= 0.02 * np.abs(want).max()      # a code may flip where the norms differ by an ulp
    assert H.device_status() == 0


@pytest.mark.gpu
def test_norm_codes_feed_the_prefill_gemm(cuda, port, tbl):
    """Prefill: norm -> codes in one launch, then the tensor-core GEMM on the codes, equals
    norm -> fp32 -> tbl_linear_forward (quantiser launch + GEMM) bit for bit."""
    import gpu_helpers as H
    rng = np.random.default_rng(78)
    rows, dim, n = 640, 1536, 768
    value = rng.standard_normal((rows, dim)).astype(np.float32)
    gate = (2 * rng.standard_normal((rows, dim))).astype(np.float32)
    weight = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    w = (rng.standard_normal((n, dim)) * 0.02).astype(np.float32)
    words, scale, *_ = port.pack_weights(w)
    dwords = H.words_dev(words)
    w_i8 = H.expand_i8(dwords, n, dim)
    out, q, sc, _ = run(H, value, gate, weight, 1e-5, want_q=True)
    before = tbl.tbl_launch_count()
    y_codes, _ = H.gemm(q, sc, w_i8, scale, want_acc=False)
    assert tbl.tbl_launch_count() - before == 1
    y_fp32 = H.linear_forward(out, dwords, scale, n, w_i8=w_i8)
    assert cuda.equal(y_codes.view(cuda.int32), y_fp32.view(cuda.int32))
    assert H.device_status() == 0

"""GPU parity of the grouped variant: projections sharing one input row, and the MoE expert FFN
(routing lists built on the device, grouped up -> squared ReLU -> down, merge in expert order)."""
import numpy as np
import pytest

from conftest import golden_cases, load_golden

pytestmark = pytest.mark.gpu


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


@pytest.mark.parametrize("K,outs,strips", [(768, [1536, 1536, 16, 16, 24], True), (768, [768, 1536], False),
                                           (48, [3, 17, 33], False), (1024, [40], True),
                                           (4096, [100, 16, 2064], True), (32768, [20, 33], True)])
def test_grouped_projections_share_one_quantised_row(cuda, port, tbl, K, outs, strips):
    """Mamba x/z/B/C/dt or attention Q/KV: several ternary linears on the same input row, one call."""
    import gpu_helpers as H
    rng = np.random.default_rng(K + len(outs))
    x = rng.standard_normal((1, K)).astype(np.float32)
    views, keep, want = [], [], []
    for n in outs:
        w = (rng.standard_normal((n, K)) * 0.02).astype(np.float32)
        words, scale, *_ = port.pack_weights(w)
        mag = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        dw, dm, db = H.words_dev(words), H.dev(mag), H.dev(bias)
        ds = H.relayout_strips(dw, n, K) if strips else None
        keep += [dw, dm, db, ds]
        views.append(H.make_view(dw, K, n, scale, magnitude=dm, bias=db, strips=ds))
        want.append(port.linear_forward(x, words, scale, n, magnitude=mag, bias=bias)[0][0])
    before = tbl.tbl_launch_count()
    out = H.grouped_forward(views, H.dev(x), max(outs)).cpu().numpy()
    if strips:
        # one grouped GEMV launch with the quantiser in its prologue; a row too long for that (K > 16384)
        # is quantised by a kernel of its own first
        assert tbl.tbl_launch_count() - before == (1 if K <= 16384 else 2)
    for g, n in enumerate(outs):
        assert bits_equal(out[g, :n], want[g]), f"group {g}"
    assert H.device_status() == 0


@pytest.mark.parametrize("rows,K,outs,strips", [(8, 768, [1536, 1536, 16, 16, 24], True), (3, 4096, [100, 2064], True),
                                                (16, 768, [768, 1536], True), (64, 1024, [40, 17], True),
                                                (5, 48, [3, 33], False), (2, 32768, [20], True),
                                                (48, 768, [1536, 1568, 24], True), (64, 768, [768, 1536], True),
                                                (33, 1280, [100, 129, 16, 300], True)])
def test_grouped_projections_on_a_batch_of_rows(cuda, port, tbl, rows, K, outs, strips):
    """Batched decode: the same projections on several rows, one grouped call (fused quantiser when
    rows*K <= 16384, separate quantiser kernel above that -- from 33 rows on followed by one launch of the widening
    tensor-core kernel over all the views --, canonical-words fallback without strips)."""
    import gpu_helpers as H
    rng = np.random.default_rng(rows + K + len(outs))
    x = rng.standard_normal((rows, K)).astype(np.float32)
    views, keep, want = [], [], []
    for n in outs:
        w = (rng.standard_normal((n, K)) * 0.02).astype(np.float32)
        words, scale, *_ = port.pack_weights(w)
        mag = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        dw, dm, db = H.words_dev(words), H.dev(mag), H.dev(bias)
        ds = H.relayout_strips(dw, n, K) if strips else None
        keep += [dw, dm, db, ds]
        views.append(H.make_view(dw, K, n, scale, magnitude=dm, bias=db, strips=ds))
        want.append(port.linear_forward(x, words, scale, n, magnitude=mag, bias=bias)[0])
    before = tbl.tbl_launch_count()
    got = H.grouped_forward_rows(views, H.dev(x))
    if strips:
        assert tbl.tbl_launch_count() - before == (1 if rows * K <= 16384 and rows <= 8 else 2)
    for g in range(len(outs)):
        assert bits_equal(got[g].cpu().numpy(), want[g]), f"group {g}"
    assert H.device_status() == 0


def _moe_setup(port, H, x, up, down, strips, i8=False):
    E, Hd, D = up.shape
    views_up, views_down, keep, packed = [], [], [], []
    for e in range(E):
        wu, su, *_ = port.pack_weights(up[e])
        wd, sd, *_ = port.pack_weights(down[e])
        du, dd = H.words_dev(wu), H.words_dev(wd)
        su_t = H.relayout_strips(du, Hd, D) if strips else None
        sd_t = H.relayout_strips(dd, D, Hd) if strips else None
        iu = H.expand_i8(du, Hd, D) if i8 else None
        idn = H.expand_i8(dd, D, Hd) if i8 else None
        keep += [du, dd, su_t, sd_t, iu, idn]
        views_up.append(H.make_view(du, D, Hd, su, rms_input=1, strips=su_t, w_i8=iu))
        views_down.append(H.make_view(dd, Hd, D, sd, rms_input=1, strips=sd_t, w_i8=idn))
        packed.append((wu, su, wd, sd))
    return views_up + views_down, keep, packed


def test_moe_matches_reference_golden(cuda, port, tbl):
    """Against the vector computed by the reference's own CPU composition (jamba.cpp:3865-3972)."""
    import gpu_helpers as H
    g = load_golden([p for p in golden_cases() if "moe_" in p][0])
    E, Hd, D = g["up"].shape
    for strips in (False,):   # D = 64, H = 128 are not multiples of 256: generic grouped path
        views, keep, _ = _moe_setup(port, H, g["x"], g["up"], g["down"], strips)
        out = H.moe_forward(views, H.dev(g["routing"]), H.dev(g["x"]), Hd, int(g["top_k"]), rms_mode=2).cpu().numpy()
        assert bits_equal(out, g["out"]), f"max diff {np.abs(out - g['out']).max()}"
    assert H.device_status() == 0


@pytest.mark.parametrize("rows,D,Hd,E,top_k", [(6, 256, 512, 4, 2), (40, 512, 768, 8, 2), (130, 256, 256, 3, 1),
                                               (9, 64, 128, 4, 2)])
def test_moe_matches_oracle(cuda, port, tbl, rows, D, Hd, E, top_k):
    """Strip tensor path (D, H multiples of 256) and generic path; more rows than one 64-row tile;
    bit-exact with the reference-order RMS, close with the fast one."""
    import gpu_helpers as H
    rng = np.random.default_rng(rows * 11 + D)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    up = (rng.standard_normal((E, Hd, D)) * 0.02).astype(np.float32)
    down = (rng.standard_normal((E, D, Hd)) * 0.02).astype(np.float32)
    routing = port.router_topk(rng.standard_normal((rows, E)).astype(np.float32), top_k)
    strips = D % 256 == 0 and Hd % 256 == 0
    views, keep, packed = _moe_setup(port, H, x, up, down, strips)
    want = port.moe_forward(x, routing, [p[0] for p in packed], [p[1] for p in packed], [p[2] for p in packed],
                            [p[3] for p in packed], Hd, rms_input=1)
    out = H.moe_forward(views, H.dev(routing), H.dev(x), Hd, top_k, rms_mode=2).cpu().numpy()
    assert bits_equal(out, want), f"max diff {np.abs(out - want).max()}"
    fast = H.moe_forward(views, H.dev(routing), H.dev(x), Hd, top_k, rms_mode=1).cpu().numpy()
    assert np.abs(fast - want).max() <= 3e-2 * np.abs(want).max()
    assert H.device_status() == 0


@pytest.mark.parametrize("rows,D,Hd,E,top_k", [(130, 256, 256, 3, 1), (300, 512, 768, 4, 2), (257, 272, 144, 5, 3),
                                               (64, 64, 128, 4, 2)])
def test_moe_grouped_tensor_core_gemm_matches_oracle(cuda, port, tbl, rows, D, Hd, E, top_k):
    """Views that carry the int8 expansion and >= 16 routed rows per expert: both expert stages run as one
    grouped tcgen05 GEMM each (device-side row counts, ragged last tiles, experts with few or no rows)."""
    import gpu_helpers as H
    rng = np.random.default_rng(rows * 13 + D)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    up = (rng.standard_normal((E, Hd, D)) * 0.02).astype(np.float32)
    down = (rng.standard_normal((E, D, Hd)) * 0.02).astype(np.float32)
    logits = rng.standard_normal((rows, E)).astype(np.float32)
    logits[:, E - 1] -= 4.0                      # the last expert gets (almost) no rows
    routing = port.router_topk(logits, top_k)
    views, keep, packed = _moe_setup(port, H, x, up, down, False, i8=True)
    want = port.moe_forward(x, routing, [p[0] for p in packed], [p[1] for p in packed], [p[2] for p in packed],
                            [p[3] for p in packed], Hd, rms_input=1)
    before = tbl.tbl_launch_count()
    out = H.moe_forward(views, H.dev(routing), H.dev(x), Hd, top_k, rms_mode=2).cpu().numpy()
    assert tbl.tbl_launch_count() - before == 8      # route, 2 x (rms, quantise, grouped GEMM), merge
    assert bits_equal(out, want), f"max diff {np.abs(out - want).max()}"
    assert H.device_status() == 0


@pytest.mark.parametrize("rows,D,Hd,E,top_k", [(130, 256, 256, 3, 1), (300, 512, 768, 4, 2), (257, 768, 1280, 5, 3),
                                               (64, 1024, 256, 8, 2)])
def test_moe_widening_tensor_core_path_matches_oracle(cuda, port, tbl, rows, D, Hd, E, top_k):
    """Views with strip-major 2-bit weights only and >= 16 routed rows per expert: both expert stages run as one
    grouped launch of the widening tcgen05 kernel each (device-side row counts, passes of 128 rows, experts with few
    or no rows, K % 512 == 256)."""
    import gpu_helpers as H
    rng = np.random.default_rng(rows * 17 + D)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    up = (rng.standard_normal((E, Hd, D)) * 0.02).astype(np.float32)
    down = (rng.standard_normal((E, D, Hd)) * 0.02).astype(np.float32)
    logits = rng.standard_normal((rows, E)).astype(np.float32)
    logits[:, E - 1] -= 4.0                      # the last expert gets (almost) no rows
    routing = port.router_topk(logits, top_k)
    views, keep, packed = _moe_setup(port, H, x, up, down, True)
    want = port.moe_forward(x, routing, [p[0] for p in packed], [p[1] for p in packed], [p[2] for p in packed],
                            [p[3] for p in packed], Hd, rms_input=1)
    before = tbl.tbl_launch_count()
    out = H.moe_forward(views, H.dev(routing), H.dev(x), Hd, top_k, rms_mode=2).cpu().numpy()
    assert tbl.tbl_launch_count() - before == 8      # route, 2 x (rms, quantise, grouped widening GEMM), merge
    assert bits_equal(out, want), f"max diff {np.abs(out - want).max()}"
    assert H.device_status() == 0


def test_moe_inactive_experts_are_never_read(cuda, port, tbl):
    """The reference's inactive_experts_contract (tests/gpu/test_gpu_decode_runtime.cpp:98-144): experts
    with routing weight 0 must not contribute -- here their scale and bias are NaN-poisoned."""
    import gpu_helpers as H
    rows, D, Hd, E = 4, 256, 256, 3
    rng = np.random.default_rng(3)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    up = (rng.standard_normal((E, Hd, D)) * 0.02).astype(np.float32)
    down = (rng.standard_normal((E, D, Hd)) * 0.02).astype(np.float32)
    routing = np.zeros((rows, E), np.float32)
    routing[:, 0] = 0.25
    routing[:, 2] = 0.75
    views, keep, packed = _moe_setup(port, H, x, up, down, True)
    poison = H.dev(np.full(max(D, Hd), np.nan, np.float32))
    for v in (views[1], views[E + 1]):   # expert 1 is never selected
        v.bias = poison.data_ptr()
        v.magnitude = poison.data_ptr()
    out = H.moe_forward(views, H.dev(routing), H.dev(x), Hd, 2, rms_mode=2).cpu().numpy()
    want = port.moe_forward(x, routing, [p[0] for p in packed], [p[1] for p in packed], [p[2] for p in packed],
                            [p[3] for p in packed], Hd, rms_input=1)
    assert np.isfinite(out).all()
    assert bits_equal(out, want)


def test_moe_route_overflow_is_reported(cuda, port, tbl):
    import gpu_helpers as H
    rows, D, Hd, E = 4, 256, 256, 4
    rng = np.random.default_rng(4)
    x = rng.standard_normal((rows, D)).astype(np.float32)
    up = (rng.standard_normal((E, Hd, D)) * 0.02).astype(np.float32)
    down = (rng.standard_normal((E, D, Hd)) * 0.02).astype(np.float32)
    routing = np.full((rows, E), 0.25, np.float32)      # 4 routes per row, capacity sized for 2
    views, keep, _ = _moe_setup(port, H, x, up, down, True)
    H.moe_forward(views, H.dev(routing), H.dev(x), Hd, 2, rms_mode=1)
    assert H.device_status() == 2   # TBL_DEV_ROUTE_OVERFLOW, and the status word is cleared by the read
    assert H.device_status() == 0


@pytest.mark.parametrize("rows,E,top_k", [(256, 8, 2), (5, 4, 1), (33, 32, 4), (7, 3, 3), (9, 6, 0)])
def test_router_topk_on_device(cuda, port, tbl, rows, E, top_k):
    """softmax -> top-k mask -> renormalise: same experts kept as the CPU path (ties -> lower index), weights
    within 1e-6 relative (the device's expf is not the host's), rows sum to one; then the routed MoE on those
    weights runs without a host round trip."""
    import gpu_helpers as H
    import torch
    rng = np.random.default_rng(rows + E)
    logits = rng.standard_normal((rows, E)).astype(np.float32) * 2
    logits[0, :] = 0.25                      # a full tie: the lowest indices win
    if E > 2:
        logits[1, 1] = logits[1, 2] = logits[1].max() + 1.0
    want = port.router_topk(logits, top_k)
    d_logits = H.dev(logits)
    out = torch.empty_like(d_logits)
    from reimagined_b200 import capi
    capi.check(tbl.tbl_router_topk(H.ptr(d_logits), rows, E, top_k, H.ptr(out), H.stream_ptr()), "tbl_router_topk")
    got = out.cpu().numpy()
    assert np.array_equal(got != 0, want != 0)
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-9)
    np.testing.assert_allclose(got.sum(axis=1), 1.0, rtol=1e-6)
    # in place
    capi.check(tbl.tbl_router_topk(H.ptr(d_logits), rows, E, top_k, H.ptr(d_logits), H.stream_ptr()), "tbl_router_topk")
    assert np.array_equal(d_logits.cpu().numpy(), got)
    assert H.device_status() == 0

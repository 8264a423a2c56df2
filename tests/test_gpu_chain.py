"""GPU parity of tbl_chain_forward: a stack of ternary linears (optionally with squared ReLU between them) in one
persistent cooperative launch, against the CPU oracle applied layer by layer, bit for bit."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


def _stack(port, H, rng, widths, affine=True, strips=True, rms_input=0):
    views, keep, host = [], [], []
    for k, n in zip(widths[:-1], widths[1:]):
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        words, scale, t, _ = port.pack_weights(w)
        mag = (1 + 0.1 * rng.standard_normal(n)).astype(np.float32) if affine else None
        bias = (0.05 * rng.standard_normal(n)).astype(np.float32) if affine else None
        dw = H.words_dev(words)
        ds = H.relayout_strips(dw, n, k) if strips and k % 256 == 0 else None
        dm = H.dev(mag) if affine else None
        db = H.dev(bias) if affine else None
        keep += [dw, ds, dm, db]
        views.append(H.make_view(dw, k, n, scale, rms_input=rms_input, magnitude=dm, bias=db, strips=ds))
        host.append((words, scale, t, mag, bias))
    return views, keep, host


def _oracle(port, host, x, relu, rms_input=0):
    from oracle import fast
    h = x
    for i, (words, scale, t, mag, bias) in enumerate(host):
        h, *_ = fast.linear_forward(h, t, scale, rms_input=rms_input, magnitude=mag, bias=bias)
        if relu and relu[i]:
            h = port.squared_relu(h)
    return h


@pytest.mark.parametrize("rows,widths,relu", [
    (1, [2048, 2048, 2048, 2048], None),                 # single-row path, full 2048-deep stages
    (1, [1024, 512, 2048, 300], [1, 0, 0]),              # mixed depths, odd last width
    (1, [768, 3072, 768], [1, 0]),                       # the block FFN of the 768-wide hybrid
    (4, [768, 3072, 768], [1, 0]),
    (8, [2048, 512, 2048], None),
    (2, [768, 768, 32000], None),                        # a wide last layer: several passes per CTA
    (3, [256, 256, 512], [0, 1]),                        # fewer strips than CTAs
    (1, [4096, 4096], None),                             # a single layer
    (5, [1536, 768, 1536, 768, 1536, 768, 1536], None),  # six layers
])
def test_chain_matches_oracle_layer_by_layer(cuda, port, tbl, rows, widths, relu):
    import gpu_helpers as H
    rng = np.random.default_rng(rows * 1000 + len(widths) + widths[0])
    views, keep, host = _stack(port, H, rng, widths)
    x = rng.standard_normal((rows, widths[0])).astype(np.float32)
    before = tbl.tbl_launch_count()
    y = H.chain_forward(views, H.dev(x), relu).cpu().numpy()
    assert tbl.tbl_launch_count() - before == 1, "the stack must run as one persistent launch"
    want = _oracle(port, host, x, relu)
    assert bits_equal(y, want), f"{int((y != want).sum())} of {y.size} differ, max {np.abs(y - want).max()}"
    assert H.device_status() == 0
    # a second call on the same workspace-sized buffers gives the same bits (counters are re-armed per call)
    y2 = H.chain_forward(views, H.dev(x), relu).cpu().numpy()
    assert bits_equal(y2, want)


def test_chain_at_the_benchmark_width(cuda, port, tbl):
    """Two 16384 x 16384 layers, one row: the configuration the headline benchmark chains."""
    import gpu_helpers as H
    rng = np.random.default_rng(77)
    size = 16384
    views, keep, host = [], [], []
    for i in range(2):
        w = rng.standard_normal((size, size), dtype=np.float32)
        w *= np.float32(0.02)
        words, scale, t, _ = port.pack_weights(w)
        del w
        dw = H.words_dev(words)
        ds = H.relayout_strips(dw, size, size)
        keep += [dw, ds]
        views.append(H.make_view(dw, size, size, scale, strips=ds))
        host.append((words, scale, t, None, None))
    x = rng.standard_normal((1, size), dtype=np.float32)
    y = H.chain_forward(views, H.dev(x)).cpu().numpy()
    want = _oracle(port, host, x, None)
    assert bits_equal(y, want)
    assert H.device_status() == 0


def test_chain_with_input_norm_matches_the_single_layer_calls(cuda, port, tbl):
    """Default-mode layers (input RMSNorm): the persistent kernel uses the parallel sum of TBL_RMS_FAST, so it
    must equal tbl_linear_forward(rms_mode = 1) bit for bit and the CPU oracle to the norm's tolerance."""
    import gpu_helpers as H
    import torch
    rng = np.random.default_rng(5)
    rows, widths, relu = 2, [1024, 2048, 1024], [1, 0]
    views, keep, host = _stack(port, H, rng, widths, rms_input=1)
    x = rng.standard_normal((rows, widths[0])).astype(np.float32)
    y = H.chain_forward(views, H.dev(x), relu, rms_mode=1)
    h = H.dev(x)
    for i, v in enumerate(views):
        h = H.linear_forward(h, keep[4 * i], v.weight_scale, v.outputs, rms_mode=1, magnitude=keep[4 * i + 2],
                             bias=keep[4 * i + 3], strips=keep[4 * i + 1])
        if relu[i]:
            h = torch.clamp(h, min=0.0) ** 2
    assert torch.equal(y, h)
    want = _oracle(port, host, x, relu, rms_input=1)
    assert np.abs(y.cpu().numpy() - want).max() <= 3e-2 * np.abs(want).max()
    assert H.device_status() == 0


@pytest.mark.parametrize("rows,widths,strips,rms_mode", [
    (20, [768, 1536, 768], True, 0),        # more rows than the persistent kernel takes
    (3, [48, 32, 64], True, 0),             # widths that are not multiples of 256
    (2, [1024, 512, 1024], False, 0),       # canonical words only
    (2, [1024, 512, 1024], True, 2),        # reference-order input norm
    (48, [768, 3072, 768], True, 0),        # mid-size batch: the widening tensor-core kernel, squared ReLU in its epilogue
    (40, [1024, 768, 512], True, 2),
])
def test_chain_layer_by_layer_route(cuda, port, tbl, rows, widths, strips, rms_mode):
    import gpu_helpers as H
    rng = np.random.default_rng(rows + widths[0])
    rms_input = 1 if rms_mode else 0
    views, keep, host = _stack(port, H, rng, widths, strips=strips, rms_input=rms_input)
    relu = [1] + [0] * (len(widths) - 2)
    x = rng.standard_normal((rows, widths[0])).astype(np.float32)
    before = tbl.tbl_launch_count()
    y = H.chain_forward(views, H.dev(x), relu, rms_mode=rms_mode).cpu().numpy()
    assert tbl.tbl_launch_count() - before > 1
    want = _oracle(port, host, x, relu, rms_input=rms_input)
    assert bits_equal(y, want)
    assert H.device_status() == 0


def test_chain_rejects_bad_stacks(cuda, port, tbl):
    import gpu_helpers as H
    rng = np.random.default_rng(1)
    views, keep, _ = _stack(port, H, rng, [256, 512, 256])
    views[1].inputs = 256                    # does not match the first layer's outputs
    arr = (type(views[0]) * 2)(*views)
    x = H.dev(np.zeros((1, 256), np.float32))
    y = H.dev(np.zeros((1, 256), np.float32))
    ws = H.dev(np.zeros(1 << 20, np.uint8))
    assert tbl.tbl_chain_forward(arr, 2, None, H.ptr(x), 1, 0, H.ptr(y), H.ptr(ws), 1 << 20, H.stream_ptr()) == -2
    assert tbl.tbl_chain_forward(arr, 0, None, H.ptr(x), 1, 0, H.ptr(y), H.ptr(ws), 1 << 20, H.stream_ptr()) == -1
    assert tbl.tbl_chain_forward(arr, 17, None, H.ptr(x), 1, 0, H.ptr(y), H.ptr(ws), 1 << 20, H.stream_ptr()) == -1
    views[1].inputs = 512
    arr = (type(views[0]) * 2)(*views)
    assert tbl.tbl_chain_forward(arr, 2, None, H.ptr(x), 1, 0, H.ptr(y), H.ptr(ws), 16, H.stream_ptr()) == -7


@pytest.mark.parametrize("bad", [np.inf, -np.inf, np.nan, 3.0e38])
def test_non_finite_values_between_layers_do_not_stall_the_stack(cuda, port, tbl, bad):
    """A layer's output travels to the next layer through buffers whose filler word marks "not written yet".  Values
    that are not finite (an infinite or NaN input spreads through every layer) must neither be mistaken for the
    filler nor keep a reader waiting: the call returns at once with a clean status word; rows that are finite are
    still exact."""
    import time
    import gpu_helpers as H
    rng = np.random.default_rng(17)
    rows, widths = 2, [1024, 2048, 512, 1024]
    views, keep, host = _stack(port, H, rng, widths)
    x = rng.standard_normal((rows, widths[0])).astype(np.float32)
    x[1, 5] = bad
    import torch
    t0 = time.perf_counter()
    y = H.chain_forward(views, H.dev(x))
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 5.0
    assert H.device_status() == 0
    want = _oracle(port, host, x[:1], None)
    assert bits_equal(y[:1].cpu().numpy(), want)

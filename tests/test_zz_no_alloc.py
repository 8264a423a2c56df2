"""The allocation-free layer forward (tbl_linear_forward_noalloc) against the ordinary entry point.

Some callers cannot provide device scratch: a plugin that a host runtime hands only input and output
buffers, code running where cudaMalloc is off limits (inside a latency-critical decode loop), or a
foreign-language binding that cannot own device memory.  For them the library keeps the quantiser's
scratch in a fixed array of its own.  The results must be bit-identical to tbl_linear_forward, on
consecutive calls that reuse the array, and oversize shapes must be refused with a clear status.

This file sorts last on purpose: a run that stops at the first failure has then already run every
other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

NOALLOC_SCRATCH_BYTES = 2 * 1024 * 1024 + 64 * 1024


def _noalloc(tbl, H, torch, x, words, strips, w_i8, scale, N, rms_mode=0, magnitude=None, bias=None):
    M, K = x.shape
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    rc = tbl.tbl_linear_forward_noalloc(H.ptr(x), H.ptr(words), H.ptr(strips), H.ptr(w_i8), float(scale), M, K, N, 8,
                                        rms_mode, H.ptr(magnitude), H.ptr(bias), H.ptr(y), H.stream_ptr())
    assert rc == 0, rc
    return y


def test_noalloc_matches_workspace_entry_point_on_consecutive_calls(cuda, port, tbl):
    import gpu_helpers as H
    torch = cuda
    rng = np.random.default_rng(123)
    # Two back-to-back calls per shape, with different inputs, share the same fixed scratch.  The shapes visit
    # every kernel family and every part of the scratch: the fused strip GEMV (no scratch), strips with more
    # rows than the fused prologue takes (interleaved codes + row sums), strips serving more than one 64-row
    # tile, the canonical-words GEMV, the generic kernel and the tcgen05 GEMM (row-major codes); a large shape
    # is followed by a small one so that stale contents of the array would show.
    shapes = [(1, 1024, 300, True, False), (8, 768, 96, True, False), (24, 1024, 300, True, False),
              (70, 768, 96, True, False), (3, 256, 64, False, False), (5, 48, 17, False, False),
              (130, 256, 160, False, True), (64, 16384, 48, True, False), (2, 256, 64, True, False)]
    for rms_mode in (1, 2):
        for (M, K, N, use_strips, use_i8) in shapes:
            w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
            words, scale, *_ = port.pack_weights(w)
            dwords = H.words_dev(words)
            strips = H.relayout_strips(dwords, N, K) if use_strips else None
            w_i8 = H.expand_i8(dwords, N, K) if use_i8 else None
            mag_h = (1 + 0.1 * rng.standard_normal(N)).astype(np.float32)
            bias_h = rng.standard_normal(N).astype(np.float32)
            mag, bias = H.dev(mag_h), H.dev(bias_h)
            for call in range(2):
                x_h = (rng.standard_normal((M, K)) * (1 + call)).astype(np.float32)
                x = H.dev(x_h)
                want = H.linear_forward(x, dwords, scale, N, w_i8=w_i8, rms_mode=rms_mode, magnitude=mag, bias=bias,
                                        strips=strips)
                got = _noalloc(tbl, H, torch, x, dwords, strips, w_i8, scale, N, rms_mode=rms_mode, magnitude=mag,
                               bias=bias)
                # same kernels, same inputs: the tolerance of this suite for integer-exact paths is zero
                assert torch.equal(got, want), f"M={M} K={K} N={N} call {call}: max diff {(got - want).abs().max().item()}"
                if rms_mode == 2 and M * K * N <= 1 << 27:
                    # with the reference's summation order in the input norm the CPU oracle must agree too
                    oy, *_ = port.linear_forward(x_h, words, scale, N, rms_input=1, magnitude=mag_h, bias=bias_h)
                    assert np.array_equal(got.cpu().numpy().view(np.uint32), oy.view(np.uint32))
    assert H.device_status() == 0


def test_noalloc_rejects_shapes_beyond_the_fixed_scratch(cuda, tbl):
    import gpu_helpers as H
    torch = cuda
    before = tbl.tbl_launch_count()
    M, K, N = 4096, 1024, 16   # needs ~8 MiB of codes: more than the fixed array
    assert tbl.tbl_linear_workspace_bytes(M, K, N) > NOALLOC_SCRATCH_BYTES
    x = torch.zeros((M, K), device="cuda")
    words = torch.zeros(N * K // 16, dtype=torch.int32, device="cuda")
    y = torch.zeros((M, N), device="cuda")
    rc = tbl.tbl_linear_forward_noalloc(H.ptr(x), H.ptr(words), None, None, 0.5, M, K, N, 8, 0, None, None,
                                        H.ptr(y), H.stream_ptr())
    assert rc == -7, rc  # TBL_ERR_WORKSPACE
    assert b"workspace" in tbl.tbl_status_string(rc)
    assert tbl.tbl_launch_count() == before  # nothing was launched
    # the largest shape that still fits is accepted (the call itself is made in the test above)
    assert tbl.tbl_linear_workspace_bytes(64, 16384, 48) <= NOALLOC_SCRATCH_BYTES

"""GPU parity of the tcgen05 prefill GEMM (int8 tensor cores, TMEM accumulators) and of the
2-bit -> int8 weight expansion that feeds it."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def bits_equal(a, b):
    return np.array_equal(np.asarray(a, np.float32).view(np.uint32), np.asarray(b, np.float32).view(np.uint32))


@pytest.mark.parametrize("N,K", [(3, 16), (17, 48), (64, 64), (100, 1024), (257, 80)])
def test_expand_weights_i8_matches_oracle(cuda, port, tbl, N, K):
    import gpu_helpers as H
    rng = np.random.default_rng(N + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    words, scale, t, _ = port.pack_weights(w)
    got = H.expand_i8(H.words_dev(words), N, K).cpu().numpy()
    assert np.array_equal(got, t)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (128, 256, 256), (130, 160, 256), (1, 16, 16), (300, 24, 48),
                                   (257, 515, 400), (4096, 1536, 768), (512, 768, 1536), (64, 33, 64),
                                   (1000, 1000, 1008)])
def test_gemm_int32_and_fp32_exact(cuda, port, tbl, M, N, K):
    """Accumulators bit-exact against an int32 reference; fp32 outputs bit-exact against the oracle's
    epilogue (same operation order)."""
    import torch
    import gpu_helpers as H
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = (rng.standard_normal((M, K)) * 2).astype(np.float32)
    mag = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    words, scale, t, _ = port.pack_weights(w)
    oq, osc = port.quantize_rows(x)
    w_i8 = H.expand_i8(H.words_dev(words), N, K)
    y, acc = H.gemm(H.dev(oq), H.dev(osc), w_i8, scale, H.dev(mag), H.dev(bias))
    assert H.device_status() == 0
    # int32 reference on the GPU in float64-free integer arithmetic (exact: |acc| <= 127*K < 2^24)
    ref_acc = (torch.from_numpy(oq).cuda().float() @ torch.from_numpy(t).cuda().float().T).round().int().cpu().numpy() \
        if K * 127 < (1 << 24) else oq.astype(np.int32) @ t.astype(np.int32).T
    assert np.array_equal(acc.cpu().numpy(), ref_acc)
    comb = (osc * np.float32(scale)).astype(np.float32)
    ref_y = ((ref_acc.astype(np.float32) * comb[:, None]) * mag[None, :] + bias[None, :]).astype(np.float32)
    assert bits_equal(y.cpu().numpy(), ref_y)
    if M * N * K <= 2e8:
        oy, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
        assert bits_equal(y.cpu().numpy(), oy)


def test_linear_forward_routes_large_m_to_gemm(cuda, port, tbl):
    import gpu_helpers as H
    M, N, K = 200, 96, 512
    rng = np.random.default_rng(5)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    words, scale, *_ = port.pack_weights(w)
    oy, *_ = port.linear_forward(x, words, scale, N, rms_input=1)
    dw = H.words_dev(words)
    y = H.linear_forward(H.dev(x), dw, scale, N, w_i8=H.expand_i8(dw, N, K), rms_mode=2)
    assert bits_equal(y.cpu().numpy(), oy)
    assert H.device_status() == 0


@pytest.mark.parametrize("M,N,K,parts", [(130, 256, 512, 2), (200, 96, 256, 3), (520, 1024, 4096, 2)])
def test_scatter_epilogue_writes_column_blocks_of_one_output(cuda, port, tbl, M, N, K, parts):
    """tbl_linear_forward_scatter on one GPU: the layer is split by output columns into `parts` calls, each storing its
    block into TWO copies of the full [M, N] output at its column offset (the peers' mappings in the multi-GPU use);
    both copies must equal the unsharded oracle bit for bit, and nothing outside a call's columns may be touched."""
    import ctypes
    import torch
    import gpu_helpers as H
    from reimagined_b200 import capi
    L = capi.lib()
    rng = np.random.default_rng(M + N + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((M, K)).astype(np.float32)
    mag = (1 + 0.2 * rng.standard_normal(N)).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    words, scale, *_ = port.pack_weights(w)
    want, *_ = port.linear_forward(x, words, scale, N, magnitude=mag, bias=bias)
    n_local = N // parts
    outs = [torch.full((M, N), 7.5, dtype=torch.float32, device="cuda") for _ in range(2)]
    dx, dmag, dbias = H.dev(x), H.dev(mag), H.dev(bias)
    wpr = K // 16
    for p in range(parts):
        shard = np.ascontiguousarray(words.reshape(N, wpr)[p * n_local:(p + 1) * n_local]).reshape(-1)
        dshard = H.words_dev(shard)
        i8 = H.expand_i8(dshard, n_local, K)
        nbytes = L.tbl_linear_workspace_bytes(M, K, n_local)
        ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
        dests = (ctypes.c_void_p * 2)(outs[0].data_ptr(), outs[1].data_ptr())
        rc = L.tbl_linear_forward_scatter(dx.data_ptr(), i8.data_ptr(), float(scale), M, K, n_local, 8, 0,
                                          dmag[p * n_local:].data_ptr(), dbias[p * n_local:].data_ptr(), dests, 2, N,
                                          p * n_local, ws.data_ptr(), nbytes, H.stream_ptr())
        assert rc == 0, rc
        torch.cuda.synchronize()
        got = outs[0].cpu().numpy()
        assert np.all(got[:, (p + 1) * n_local:] == 7.5)          # later blocks untouched so far
    for o in outs:
        y = o.cpu().numpy()
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
    # refused: rows the tensor-core path does not serve, misaligned column offset
    assert L.tbl_linear_forward_scatter(dx.data_ptr(), i8.data_ptr(), float(scale), 64, K, n_local, 8, 0, None, None, dests, 2, N, 0,
                                        ws.data_ptr(), nbytes, H.stream_ptr()) == -10
    assert L.tbl_linear_forward_scatter(dx.data_ptr(), i8.data_ptr(), float(scale), M, K, n_local, 8, 0, None, None, dests, 2, N + 2, 2,
                                        ws.data_ptr(), nbytes, H.stream_ptr()) == -6
    assert H.device_status() == 0

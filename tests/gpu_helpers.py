"""Thin wrappers that call the C ABI with torch-owned device memory (test infrastructure)."""
import ctypes as C

import numpy as np
import torch

from reimagined_b200 import capi


def dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def words_dev(words):
    return torch.from_numpy(np.ascontiguousarray(words).view(np.int32)).cuda()


def ptr(t):
    return 0 if t is None else t.data_ptr()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def device_status():
    return capi.lib().tbl_device_status(stream_ptr())


def quantize_rows(x, bits=8, rms_mode=0, tie_mode=0, row_index=None):
    L = capi.lib()
    M, K = x.shape
    if row_index is not None:
        M = row_index.numel()
    q = torch.empty((M, K), dtype=torch.int8, device="cuda")
    sc = torch.empty(M, dtype=torch.float32, device="cuda")
    sums = torch.empty(M, dtype=torch.int32, device="cuda")
    capi.check(L.tbl_quantize_rows(ptr(x), ptr(row_index), M, K, bits, rms_mode, tie_mode, ptr(q), ptr(sc),
                                   ptr(sums), stream_ptr()), "tbl_quantize_rows")
    return q, sc, sums


def relayout_strips(words, N, K):
    L = capi.lib()
    nbytes = L.tbl_strip_bytes(N, K)
    assert nbytes > 0
    out = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_relayout_strips(ptr(words), N, K, ptr(out), stream_ptr()), "tbl_relayout_strips")
    return out


def gemv(q, sc, words, weight_scale, N, magnitude=None, bias=None, want_acc=True, strips=None):
    L = capi.lib()
    M, K = q.shape
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    acc = torch.empty((M, N), dtype=torch.int32, device="cuda") if want_acc else None
    nbytes = L.tbl_gemv_workspace_bytes(M, K)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_gemv(ptr(q), ptr(sc), ptr(words), ptr(strips), float(weight_scale), ptr(magnitude), ptr(bias), M, K, N,
                          ptr(y), ptr(acc), ptr(ws), nbytes, stream_ptr()), "tbl_gemv")
    return y, acc


def expand_i8(words, N, K):
    L = capi.lib()
    out = torch.empty((N, K), dtype=torch.int8, device="cuda")
    capi.check(L.tbl_expand_weights_i8(ptr(words), N, K, ptr(out), stream_ptr()), "tbl_expand_weights_i8")
    return out


def gemm(q, sc, w_i8, weight_scale, magnitude=None, bias=None, want_acc=True):
    L = capi.lib()
    M, K = q.shape
    N = w_i8.shape[0]
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    acc = torch.empty((M, N), dtype=torch.int32, device="cuda") if want_acc else None
    capi.check(L.tbl_gemm(ptr(q), ptr(sc), ptr(w_i8), float(weight_scale), ptr(magnitude), ptr(bias), M, K, N,
                          ptr(y), ptr(acc), stream_ptr()), "tbl_gemm")
    return y, acc


def linear_forward(x, words, weight_scale, N, w_i8=None, bits=8, rms_mode=0, magnitude=None, bias=None,
                   strips=None):
    L = capi.lib()
    M, K = x.shape
    y = torch.empty((M, N), dtype=torch.float32, device="cuda")
    nbytes = L.tbl_linear_workspace_bytes(M, K, N)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_linear_forward(ptr(x), ptr(words), ptr(strips), ptr(w_i8), float(weight_scale), M, K, N, bits, rms_mode,
                                    ptr(magnitude), ptr(bias), ptr(y), ptr(ws), nbytes, stream_ptr()),
               "tbl_linear_forward")
    return y


def make_view(words_t, inputs, outputs, weight_scale, bits=8, rms_input=0, magnitude=None, bias=None,
              strips=None, w_i8=None):
    return capi.LinearView(None, ptr(words_t), ptr(magnitude) or None, ptr(bias) or None, inputs, outputs, bits,
                           rms_input, float(weight_scale), ptr(strips) or None, ptr(w_i8) or None)


def grouped_forward(views, x_row, output_stride, rms_mode=0):
    L = capi.lib()
    G = len(views)
    arr = (capi.LinearView * G)(*views)
    out = torch.zeros((G, output_stride), dtype=torch.float32, device="cuda")
    nbytes = L.tbl_grouped_workspace_bytes(G, views[0].inputs)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_grouped_forward(arr, G, ptr(x_row), ptr(out), output_stride, rms_mode, ptr(ws), nbytes,
                                     stream_ptr()), "tbl_grouped_forward")
    return out


def grouped_forward_rows(views, x, rms_mode=0):
    """x [rows, K] -> list of [rows, outputs_g] tensors."""
    L = capi.lib()
    G = len(views)
    rows = x.shape[0]
    arr = (capi.LinearView * G)(*views)
    stride = rows * max(v.outputs for v in views)
    out = torch.zeros((G, stride), dtype=torch.float32, device="cuda")
    nbytes = L.tbl_grouped_rows_workspace_bytes(G, rows, views[0].inputs)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_grouped_forward_rows(arr, G, ptr(x), rows, ptr(out), stride, rms_mode, ptr(ws), nbytes,
                                          stream_ptr()), "tbl_grouped_forward_rows")
    return [out[g, : rows * views[g].outputs].view(rows, views[g].outputs) for g in range(G)]


def moe_forward(views, routing, x, hidden_dim, max_routes, rms_mode=2, tie_mode=0):
    L = capi.lib()
    rows, dim = x.shape
    E = routing.shape[1]
    arr = (capi.LinearView * (2 * E))(*views)
    out = torch.empty((rows, dim), dtype=torch.float32, device="cuda")
    nbytes = L.tbl_moe_workspace_bytes(rows, dim, hidden_dim, E, max_routes)
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_moe_forward(arr, ptr(routing), ptr(x), rows, dim, hidden_dim, E, max_routes, rms_mode,
                                 tie_mode, ptr(out), ptr(ws), nbytes, stream_ptr()), "tbl_moe_forward")
    return out


def chain_forward(views, x, squared_relu=None, rms_mode=0):
    """x [rows, views[0].inputs] through the stack of linears; returns [rows, views[-1].outputs]."""
    L = capi.lib()
    n = len(views)
    rows = x.shape[0]
    arr = (capi.LinearView * n)(*views)
    flags = None if squared_relu is None else (C.c_int * n)(*[int(bool(f)) for f in squared_relu])
    y = torch.empty((rows, views[-1].outputs), dtype=torch.float32, device="cuda")
    nbytes = L.tbl_chain_workspace_bytes(arr, n, rows)
    assert nbytes > 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    capi.check(L.tbl_chain_forward(arr, n, flags, ptr(x), rows, rms_mode, ptr(y), ptr(ws), nbytes, stream_ptr()),
               "tbl_chain_forward")
    return y

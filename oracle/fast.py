"""Large-shape form of the CPU oracle (TEST INFRASTRUCTURE ONLY; same rules as oracle/__init__.py).

The plain-C restatement walks acc = sum_k q*t with scalar loops, which takes minutes at the sizes the
benchmark configurations name (K = N = 16384 with thousands of rows; the 8-expert 2048 x 5632 FFN).  This
module keeps every floating-point step of that restatement -- the reference-order RMSNorm and the per-row
quantiser are the C port's own functions -- and only replaces the integer dot products by a float32 BLAS
product of the int8 codes and the ternary weights.  That product is exact: every partial sum is an integer
of magnitude <= 127*K, and 127*K < 2^24 for K <= 131072, so no fp32 addition (or fused multiply-add) in any
order ever rounds.  The epilogue is then evaluated in numpy float32 in the reference's operation order
(OXN/nsos/src/bitnet_adapter_avx2.cpp:70,150-155): c = act_scale*weight_scale; y = float(acc)*c;
y *= magnitude; y += bias -- one IEEE operation each.

Pinned: tests/test_oracle.py compares these functions bit for bit with ternary_oracle.c (itself pinned to the
reference build) on shapes the C loops finish quickly.
"""
from __future__ import annotations

import numpy as np

from . import port as _port

_EXACT_K = (1 << 24) // 127


def acc_exact(q_i8: np.ndarray, t_i8: np.ndarray, block: int = 4096) -> np.ndarray:
    """int32 [M,N] accumulators of q int8 [M,K] against ternary int8 [N,K] via exact float32 BLAS products."""
    M, K = q_i8.shape
    N = t_i8.shape[0]
    assert t_i8.shape[1] == K and K <= _EXACT_K, "fp32 products are exact only while 127*K < 2^24"
    qf = q_i8.astype(np.float32)
    acc = np.empty((M, N), dtype=np.int32)
    for n0 in range(0, N, block):
        tf = t_i8[n0:n0 + block].astype(np.float32)
        acc[:, n0:n0 + block] = (qf @ tf.T).astype(np.int32)
    return acc


def epilogue(acc: np.ndarray, act_scales: np.ndarray, weight_scale, magnitude=None, bias=None) -> np.ndarray:
    c = act_scales.astype(np.float32) * np.float32(weight_scale)
    y = acc.astype(np.float32) * c[:, None]
    if magnitude is not None:
        y = y * np.asarray(magnitude, np.float32)[None, :]
    if bias is not None:
        y = y + np.asarray(bias, np.float32)[None, :]
    return y


def linear_forward(x, t_i8, weight_scale, rms_input=0, bits=8, tie_mode=0, magnitude=None, bias=None):
    """One packed BitLinear forward (tor_linear_forward) on unpacked ternary weights int8 [N,K].
    Returns (y fp32 [M,N], q int8 [M,K], act_scales fp32 [M], acc int32 [M,N])."""
    P = _port()
    x = np.ascontiguousarray(x, np.float32)
    if rms_input:
        x = P.rmsnorm_rows(x, 1e-6)
    q, sc = P.quantize_rows(x, bits, tie_mode)
    acc = acc_exact(q, t_i8)
    return epilogue(acc, sc, weight_scale, magnitude, bias), q, sc, acc


def moe_forward(x, routing, up_t, up_scale, down_t, down_scale, rms_input=1, bits=8, tie_mode=0):
    """The CPU composition of JambaBlock::forward_moe (OXN/nsos/src/jamba.cpp:3865-3972) as restated by
    tor_moe_forward: experts in index order; rows with a non-zero routing weight, in row order; up ->
    squared ReLU -> down, both default-mode layers without affine; out[r] += y * weight."""
    P = _port()
    x = np.ascontiguousarray(x, np.float32)
    routing = np.ascontiguousarray(routing, np.float32)
    rows, D = x.shape
    E = routing.shape[1]
    out = np.zeros((rows, D), dtype=np.float32)
    for e in range(E):
        sel = np.nonzero(routing[:, e] != 0.0)[0]
        if sel.size == 0:
            continue
        hid, *_ = linear_forward(x[sel], up_t[e], up_scale[e], rms_input, bits, tie_mode)
        hid = P.squared_relu(hid)
        yo, *_ = linear_forward(hid, down_t[e], down_scale[e], rms_input, bits, tie_mode)
        out[sel] = out[sel] + yo * routing[sel, e][:, None]
    return out

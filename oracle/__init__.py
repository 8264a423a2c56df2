"""ctypes/numpy front-end for the two CPU checkers (TEST INFRASTRUCTURE ONLY).

``port``  -> libternary_oracle.so, the plain-C restatement in ternary_oracle.c.
``ref``   -> _ref/libnsos_ref.so, the reference's own C++ compiled by oracle/Makefile
             (present only where that build ran or travelled to).

Nothing in the shipped package may import this module; the tests, the smoke check and the
bench's CPU-baseline legs are its only users.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(_HERE, "libternary_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libnsos_ref.so")

_f32p = C.POINTER(C.c_float)
_i8p = C.POINTER(C.c_int8)
_i32p = C.POINTER(C.c_int32)
_u32p = C.POINTER(C.c_uint32)


def reference_root():
    """The reference checkout: $REFERENCE_ROOT, else a directory named `reference` beside this repository."""
    root = os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    return root if os.path.isdir(os.path.join(root, "OXN", "nsos", "src")) else None


def build(verbose: bool = False) -> None:
    """Runs oracle/Makefile (builds the port always, the reference lib when its sources exist)."""
    out = None if verbose else subprocess.DEVNULL
    cmd = ["make", "-C", _HERE, "-j8"]
    root = reference_root()
    if root:
        cmd.append(f"REFERENCE_ROOT={root}")
    subprocess.run(cmd, check=True, stdout=out)


def _ptr(a, typ):
    if a is None:
        return None
    return a.ctypes.data_as(typ)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class _Port:
    def __init__(self):
        if not os.path.exists(PORT_SO):
            build()
        self.lib = L = C.CDLL(PORT_SO)
        L.tor_abs_mean.restype = C.c_float
        L.tor_abs_mean.argtypes = [_f32p, C.c_int64]
        L.tor_packed_words.restype = C.c_int64
        L.tor_packed_words.argtypes = [C.c_int, C.c_int]
        L.tor_pack_weights.restype = C.c_float
        L.tor_pack_weights.argtypes = [_f32p, C.c_int, C.c_int, _u32p, _i8p, _i32p]
        L.tor_unpack_i8.argtypes = [_u32p, C.c_int, C.c_int, _i8p]
        L.tor_rmsnorm_rows.argtypes = [_f32p, C.c_int, C.c_int, C.c_float, _f32p]
        L.tor_quantize_rows.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _i8p, _f32p]
        L.tor_gemm_i8.argtypes = [_i8p, _i8p, _f32p, C.c_float, C.c_int, C.c_int, C.c_int,
                                  _f32p, _f32p, _f32p, _i32p]
        L.tor_linear_forward.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _u32p, C.c_float,
                                         C.c_int, C.c_int, C.c_int, _f32p, _f32p, _f32p,
                                         _i8p, _f32p, _i32p]
        L.tor_linear_forward_i8_mt.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _i8p, C.c_float,
                                               C.c_int, C.c_int, C.c_int, _f32p, _f32p, _f32p, C.c_int]
        L.tor_squared_relu.argtypes = [_f32p, C.c_int64, _f32p]
        L.tor_row_norm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_float, _f32p]
        L.tor_row_norm.restype = None
        L.tor_router_topk.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p]
        pp_u32 = C.POINTER(_u32p)
        pp_f32 = C.POINTER(_f32p)
        L.tor_mamba_conv_step.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
        L.tor_mamba_ssd_step.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _f32p]
        L.tor_attention_decode.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_int, _i32p, _f32p, _f32p, C.c_int, C.c_int,
                                           C.c_int, C.c_int, C.c_int, _f32p]
        L.tor_moe_forward.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p,
                                      pp_u32, _f32p, pp_f32, pp_f32,
                                      pp_u32, _f32p, pp_f32, pp_f32,
                                      C.c_int, C.c_int, C.c_int, _f32p]

    # -- packer ---------------------------------------------------------------------
    def pack_weights(self, w):
        """w fp32 [N,K] -> (words uint32, weight_scale float32, ternary int8 [N,K], row_sums)."""
        w = _f32(w)
        N, K = w.shape
        nwords = self.lib.tor_packed_words(N, K)
        words = np.zeros(nwords, dtype=np.uint32)
        t = np.zeros((N, K), dtype=np.int8)
        rs = np.zeros(N, dtype=np.int32)
        s = self.lib.tor_pack_weights(_ptr(w, _f32p), N, K, _ptr(words, _u32p), _ptr(t, _i8p), _ptr(rs, _i32p))
        return words, np.float32(s), t, rs

    def unpack_i8(self, words, N, K):
        words = np.ascontiguousarray(words, dtype=np.uint32)
        t = np.zeros((N, K), dtype=np.int8)
        self.lib.tor_unpack_i8(_ptr(words, _u32p), N, K, _ptr(t, _i8p))
        return t

    # -- activations ----------------------------------------------------------------
    def rmsnorm_rows(self, x, eps=1e-6):
        x = _f32(x)
        M, K = x.shape
        out = np.empty_like(x)
        self.lib.tor_rmsnorm_rows(_ptr(x, _f32p), M, K, eps, _ptr(out, _f32p))
        return out

    def row_norm(self, value, gate=None, weight=None, eps=1e-6):
        """RMSNorm x weight of each row of value (x silu(gate) first when a gate is given)."""
        value = _f32(value)
        rows, dim = value.shape
        gate = None if gate is None else _f32(gate)
        weight = None if weight is None else _f32(weight)
        out = np.empty_like(value)
        self.lib.tor_row_norm(_ptr(value, _f32p), None if gate is None else _ptr(gate, _f32p),
                              None if weight is None else _ptr(weight, _f32p), rows, dim, eps, _ptr(out, _f32p))
        return out

    def quantize_rows(self, x, bits=8, tie_mode=0):
        """x fp32 [M,K] -> (q int8 [M,K], act_scales fp32 [M])."""
        x = _f32(x)
        M, K = x.shape
        q = np.zeros((M, K), dtype=np.int8)
        sc = np.zeros(M, dtype=np.float32)
        self.lib.tor_quantize_rows(_ptr(x, _f32p), M, K, bits, tie_mode, None, _ptr(q, _i8p), _ptr(sc, _f32p))
        return q, sc

    # -- linear ---------------------------------------------------------------------
    def linear_forward(self, x, words, weight_scale, N, rms_input=0, bits=8, tie_mode=0,
                       magnitude=None, bias=None):
        """Returns (y fp32 [M,N], q int8 [M,K], act_scales fp32 [M], acc int32 [M,N])."""
        x = _f32(x)
        M, K = x.shape
        words = np.ascontiguousarray(words, dtype=np.uint32)
        mag = None if magnitude is None else _f32(magnitude)
        b = None if bias is None else _f32(bias)
        y = np.zeros((M, N), dtype=np.float32)
        q = np.zeros((M, K), dtype=np.int8)
        sc = np.zeros(M, dtype=np.float32)
        acc = np.zeros((M, N), dtype=np.int32)
        self.lib.tor_linear_forward(_ptr(x, _f32p), M, K, N, _ptr(words, _u32p), float(weight_scale),
                                    int(rms_input), bits, tie_mode, _ptr(mag, _f32p), _ptr(b, _f32p),
                                    _ptr(y, _f32p), _ptr(q, _i8p), _ptr(sc, _f32p), _ptr(acc, _i32p))
        return y, q, sc, acc

    def linear_forward_i8_mt(self, x, t, weight_scale, threads, rms_input=0, bits=8, y=None):
        x = _f32(x)
        M, K = x.shape
        N = t.shape[0]
        if y is None:
            y = np.zeros((M, N), dtype=np.float32)
        self.lib.tor_linear_forward_i8_mt(_ptr(x, _f32p), M, K, N, _ptr(t, _i8p), float(weight_scale),
                                          int(rms_input), bits, 0, None, None, _ptr(y, _f32p), threads)
        return y

    # -- decode glue (all update their state arrays in place) -----------------------------
    def mamba_conv_step(self, xv, Bv, Cv, conv_w, conv_b, ring, K):
        """xv [R,d_inner], Bv/Cv [R,GS], ring [R,K-1,conv_dim] (updated) -> xBC [R,conv_dim]."""
        R, d_inner = xv.shape
        GS = Bv.shape[1]
        xBC = np.zeros((R, d_inner + 2 * GS), np.float32)
        self.lib.tor_mamba_conv_step(_ptr(_f32(xv), _f32p), _ptr(_f32(Bv), _f32p), _ptr(_f32(Cv), _f32p),
                                     _ptr(_f32(conv_w), _f32p), _ptr(_f32(conv_b), _f32p), _ptr(ring, _f32p),
                                     R, d_inner, GS, K, _ptr(xBC, _f32p))
        return xBC

    def mamba_ssd_step(self, xBC, dt, A_log, D, state, n_heads, d_head, N, n_groups):
        """state [R,d_inner,N] (updated) -> y [R,d_inner]."""
        R = xBC.shape[0]
        y = np.zeros((R, n_heads * d_head), np.float32)
        self.lib.tor_mamba_ssd_step(_ptr(_f32(xBC), _f32p), _ptr(_f32(dt), _f32p), _ptr(_f32(A_log), _f32p),
                                    _ptr(_f32(D), _f32p), _ptr(state, _f32p), R, n_heads, d_head, N, n_groups,
                                    _ptr(y, _f32p))
        return y

    def attention_decode(self, q, kv, k_cache, v_cache, tokens, cos_t, sin_t, n_heads, n_kv_heads, head_dim,
                         sliding_window):
        """caches [R,capacity,kv_dim] and tokens int32 [R] are updated -> out [R, n_heads*head_dim]."""
        R = q.shape[0]
        out = np.zeros((R, n_heads * head_dim), np.float32)
        self.lib.tor_attention_decode(_ptr(_f32(q), _f32p), _ptr(_f32(kv), _f32p), _ptr(k_cache, _f32p),
                                      _ptr(v_cache, _f32p), k_cache.shape[1], _ptr(tokens, _i32p),
                                      _ptr(_f32(cos_t), _f32p), _ptr(_f32(sin_t), _f32p), R, n_heads, n_kv_heads,
                                      head_dim, sliding_window, _ptr(out, _f32p))
        return out

    def squared_relu(self, x):
        x = _f32(x)
        out = np.empty_like(x)
        self.lib.tor_squared_relu(_ptr(x, _f32p), x.size, _ptr(out, _f32p))
        return out

    def router_topk(self, logits, top_k):
        logits = _f32(logits)
        rows, E = logits.shape
        w = np.zeros_like(logits)
        self.lib.tor_router_topk(_ptr(logits, _f32p), rows, E, top_k, _ptr(w, _f32p))
        return w

    def moe_forward(self, x, routing, up_words, up_scale, down_words, down_scale, H,
                    rms_input=1, bits=8, tie_mode=0):
        """up_words/down_words: lists of uint32 arrays (one per expert); no magnitude/bias."""
        x = _f32(x)
        routing = _f32(routing)
        rows, D = x.shape
        E = routing.shape[1]
        ups = [np.ascontiguousarray(u, dtype=np.uint32) for u in up_words]
        dns = [np.ascontiguousarray(d, dtype=np.uint32) for d in down_words]
        upp = (_u32p * E)(*[_ptr(u, _u32p) for u in ups])
        dnp = (_u32p * E)(*[_ptr(d, _u32p) for d in dns])
        us = _f32(up_scale)
        ds = _f32(down_scale)
        out = np.zeros((rows, D), dtype=np.float32)
        self.lib.tor_moe_forward(_ptr(x, _f32p), rows, D, H, E, _ptr(routing, _f32p),
                                 upp, _ptr(us, _f32p), None, None,
                                 dnp, _ptr(ds, _f32p), None, None,
                                 int(rms_input), bits, tie_mode, _ptr(out, _f32p))
        return out


class _Ref:
    """The reference's own BitLinear (CPU packed path) behind ref_shim.cpp."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO)
        self.lib = L = C.CDLL(REF_SO)
        L.ref_pack.restype = C.c_longlong
        L.ref_pack.argtypes = [_f32p, C.c_int, C.c_int, _u32p, _f32p]
        L.ref_linear_forward.argtypes = [_f32p, C.c_int, C.c_int, _f32p, C.c_int, C.c_int,
                                         _f32p, _f32p, C.c_int, _f32p]
        L.ref_layer_create.restype = C.c_void_p
        L.ref_layer_create.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p, _f32p, C.c_int]
        L.ref_layer_forward.argtypes = [C.c_void_p, _f32p, C.c_int, _f32p]
        L.ref_layer_forward_mt.argtypes = [C.POINTER(C.c_void_p), C.c_int, _f32p, C.c_int, _f32p]
        L.ref_layers_forward_parallel.argtypes = [C.POINTER(C.c_void_p), C.c_int, _f32p, C.c_int, C.POINTER(_f32p)]
        L.ref_layer_destroy.argtypes = [C.c_void_p]
        L.ref_row_norm.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_float, _f32p]
        L.ref_moe_forward.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p,
                                      _f32p, _f32p, C.c_int, _f32p]

    def pack(self, w):
        w = _f32(w)
        N, K = w.shape
        words = np.zeros((N * K + 15) // 16, dtype=np.uint32)
        scale = np.zeros(1, dtype=np.float32)
        n = self.lib.ref_pack(_ptr(w, _f32p), N, K, _ptr(words, _u32p), _ptr(scale, _f32p))
        if n != words.size:
            raise RuntimeError(f"ref_pack returned {n}, expected {words.size}")
        return words, scale[0]

    def linear_forward(self, w, x, exact_linear=True, magnitude=None, bias=None, bits=8):
        w = _f32(w)
        x = _f32(x)
        N, K = w.shape
        M = x.shape[0]
        mag = None if magnitude is None else _f32(magnitude)
        b = None if bias is None else _f32(bias)
        y = np.zeros((M, N), dtype=np.float32)
        rc = self.lib.ref_linear_forward(_ptr(w, _f32p), N, K, _ptr(x, _f32p), M, int(exact_linear),
                                         _ptr(mag, _f32p), _ptr(b, _f32p), bits, _ptr(y, _f32p))
        if rc != 0:
            raise RuntimeError("reference BitLinear::forward raised")
        return y

    def layer_create(self, w, exact_linear=True, bits=8):
        w = _f32(w)
        N, K = w.shape
        h = self.lib.ref_layer_create(_ptr(w, _f32p), N, K, int(exact_linear), None, None, bits)
        if not h:
            raise RuntimeError("reference layer construction raised")
        return h

    def layer_forward(self, h, x, y):
        rc = self.lib.ref_layer_forward(h, _ptr(x, _f32p), x.shape[0], _ptr(y, _f32p))
        if rc != 0:
            raise RuntimeError("reference BitLinear::forward raised")

    def layer_forward_mt(self, handles, x, y):
        arr = (C.c_void_p * len(handles))(*handles)
        rc = self.lib.ref_layer_forward_mt(arr, len(handles), _ptr(x, _f32p), x.shape[0], _ptr(y, _f32p))
        if rc != 0:
            raise RuntimeError("reference BitLinear::forward raised")

    def layers_forward_parallel(self, handles, x, ys):
        """Each handle (one per host thread) runs forward on the same x; ys[p] is its [M,N_p] output."""
        arr = (C.c_void_p * len(handles))(*handles)
        outs = (_f32p * len(handles))(*[_ptr(y, _f32p) for y in ys])
        rc = self.lib.ref_layers_forward_parallel(arr, len(handles), _ptr(x, _f32p), x.shape[0], outs)
        if rc != 0:
            raise RuntimeError("reference BitLinear::forward raised")

    def layer_destroy(self, h):
        self.lib.ref_layer_destroy(h)

    def row_norm(self, value, gate=None, weight=None, eps=1e-6):
        """The reference's own Tensor ops: value[.mul(gate.silu())].rmsnorm(eps)[.mul(weight)]."""
        value = _f32(value)
        rows, dim = value.shape
        gate = None if gate is None else _f32(gate)
        weight = None if weight is None else _f32(weight)
        out = np.empty_like(value)
        rc = self.lib.ref_row_norm(_ptr(value, _f32p), None if gate is None else _ptr(gate, _f32p),
                                   None if weight is None else _ptr(weight, _f32p), rows, dim, eps, _ptr(out, _f32p))
        if rc != 0:
            raise RuntimeError("reference norm composition raised")
        return out

    def moe_forward(self, x, routing, up_w, down_w, bits=8):
        """up_w fp32 [E,H,D], down_w fp32 [E,D,H]; experts are default-mode BitLinears."""
        x = _f32(x)
        routing = _f32(routing)
        up_w = _f32(up_w)
        down_w = _f32(down_w)
        rows, D = x.shape
        E, H, _ = up_w.shape
        out = np.zeros((rows, D), dtype=np.float32)
        rc = self.lib.ref_moe_forward(_ptr(x, _f32p), rows, D, H, E, _ptr(routing, _f32p),
                                      _ptr(up_w, _f32p), _ptr(down_w, _f32p), bits, _ptr(out, _f32p))
        if rc != 0:
            raise RuntimeError("reference MoE composition raised")
        return out


_port = None
_ref = None


def port() -> _Port:
    global _port
    if _port is None:
        _port = _Port()
    return _port


def ref_available() -> bool:
    return os.path.exists(REF_SO)


def ref() -> _Ref:
    global _ref
    if _ref is None:
        _ref = _Ref()
    return _ref


# ---- model-level checker: the reference's whole core library behind ref_model_shim.cpp ----------------
MODEL_REF_SO = os.path.join(_HERE, "_ref", "libnsos_model_ref.so")
_EMIT = C.CFUNCTYPE(None, C.c_char_p, C.c_int, C.c_void_p, C.c_longlong, C.c_void_p)
MODEL_CFG_FIELDS = ("num_layers", "d_model", "vocab_size", "n_heads", "n_kv_heads", "mamba_d_state", "mamba_expand",
                    "mamba_conv_kernel", "mamba_head_dim", "mamba_n_groups", "attention_period", "attention_slot")


class RefModel:
    """An nsos::JambaModel of the reference (CPU, packed ternary path, streaming decode), seeded weights."""

    def __init__(self, lib, cfg: dict, seed: int):
        self.lib, self.cfg = lib, dict(cfg)
        arr = (C.c_int * len(MODEL_CFG_FIELDS))(*[int(cfg[k]) for k in MODEL_CFG_FIELDS])
        self.handle = lib.refm_create(arr, seed)
        if not self.handle:
            raise RuntimeError("reference JambaModel construction raised")

    def close(self):
        if self.handle:
            self.lib.refm_destroy(self.handle)
            self.handle = None

    def reset(self):
        if self.lib.refm_reset(self.handle) != 0:
            raise RuntimeError("reset_session raised")

    def step(self, token: int) -> np.ndarray:
        """JambaModel::forward_ids_last({token}) in streaming mode: logits fp32 [vocab]."""
        logits = np.zeros(self.cfg["vocab_size"], np.float32)
        if self.lib.refm_step(self.handle, int(token), _ptr(logits, _f32p)) != logits.size:
            raise RuntimeError("forward_ids_last raised")
        return logits

    def step_trace(self, token: int):
        """The same step block by block: (hidden fp32 [layers + 1, d_model], logits)."""
        hidden = np.zeros((self.cfg["num_layers"] + 1, self.cfg["d_model"]), np.float32)
        logits = np.zeros(self.cfg["vocab_size"], np.float32)
        if self.lib.refm_step_trace(self.handle, int(token), _ptr(hidden, _f32p), _ptr(logits, _f32p)) != logits.size:
            raise RuntimeError("block-by-block step raised")
        return hidden, logits

    def export(self) -> dict:
        """Every parameter of the decode step as named numpy arrays (see ref_model_shim.cpp::refm_export)."""
        out = {}

        def cb(name, dtype, data, count, user):
            dt = (np.float32, np.uint32, np.int32)[dtype]
            if count:
                raw = C.string_at(data, count * 4)
                out[name.decode()] = np.frombuffer(raw, dtype=dt).copy()
            else:
                out[name.decode()] = np.zeros(0, dt)

        if self.lib.refm_export(self.handle, _EMIT(cb), None) != 0:
            raise RuntimeError("export raised")
        return out

    def save_edge_pack(self, path: str):
        if self.lib.refm_save_edge_pack(self.handle, path.encode()) != 0:
            raise RuntimeError("save_edge_linear_pack raised")


class _ModelRef:
    def __init__(self):
        if not os.path.exists(MODEL_REF_SO):
            raise FileNotFoundError(MODEL_REF_SO)
        self.lib = L = C.CDLL(MODEL_REF_SO)
        L.refm_create.restype = C.c_void_p
        L.refm_create.argtypes = [C.POINTER(C.c_int), C.c_uint]
        L.refm_destroy.argtypes = [C.c_void_p]
        L.refm_reset.argtypes = [C.c_void_p]
        L.refm_step.argtypes = [C.c_void_p, C.c_int, _f32p]
        L.refm_step_trace.argtypes = [C.c_void_p, C.c_int, _f32p, _f32p]
        L.refm_export.argtypes = [C.c_void_p, _EMIT, C.c_void_p]
        L.refm_save_edge_pack.argtypes = [C.c_void_p, C.c_char_p]
        L.refm_router.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, C.c_int, _f32p, _f32p, _f32p]

    def model(self, cfg: dict, seed: int = 1) -> RefModel:
        return RefModel(self.lib, cfg, seed)

    def router(self, x, gate_w, top_k):
        """MoERouter::forward: (logits, routing weights), both [rows, experts]."""
        x = _f32(x)
        gate_w = _f32(gate_w)
        rows, D = x.shape
        E = gate_w.shape[0]
        logits = np.zeros((rows, E), np.float32)
        weights = np.zeros((rows, E), np.float32)
        if self.lib.refm_router(_ptr(x, _f32p), rows, D, E, top_k, _ptr(gate_w, _f32p), _ptr(logits, _f32p),
                                _ptr(weights, _f32p)) != 0:
            raise RuntimeError("MoERouter::forward raised")
        return logits, weights


_model_ref = None


def model_ref_available() -> bool:
    return os.path.exists(MODEL_REF_SO)


def model_ref() -> _ModelRef:
    global _model_ref
    if _model_ref is None:
        _model_ref = _ModelRef()
    return _model_ref

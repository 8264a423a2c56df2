"""One streaming decode step of the D-wide Mamba-2 / attention hybrid, composed on the CPU from the C port's
functions (TEST INFRASTRUCTURE ONLY; same rules as oracle/__init__.py).

Follows JambaModel::forward_impl (OXN/nsos/src/jamba.cpp:851-992), JambaBlock::forward (:3158-3375),
Mamba2SSD::forward_faithful_step (OXN/nsos/src/mamba2.cpp:3947-4125) and the single-token branch of
Attention::forward (OXN/nsos/src/jamba.cpp:6291-6295, 6500-6640) on the parameter set handed out by
ref_model_shim.cpp::refm_export.  tests/test_decode_oracle.py pins it to the reference model itself.
"""
from __future__ import annotations

import numpy as np

from . import port as _port


class Linear:
    def __init__(self, params: dict, name: str):
        self.words = params[name + ".words"]
        self.scale = np.float32(params[name + ".scale"][0])
        meta = params[name + ".meta"]
        self.inputs, self.outputs = int(meta[0]), int(meta[1])
        self.use_bias, self.rms_input, self.use_magnitude, self.bits = bool(meta[2]), int(meta[3]), bool(meta[4]), int(meta[5])
        self.magnitude = params[name + ".magnitude"] if self.use_magnitude else None
        self.bias = params[name + ".bias"] if self.use_bias else None

    def __call__(self, x):
        y, *_ = _port().linear_forward(x, self.words, self.scale, self.outputs, rms_input=self.rms_input, bits=self.bits,
                                       magnitude=self.magnitude, bias=self.bias)
        return y


class PortDecoder:
    """Batch of `rows` independent sequences; state lives in numpy arrays and is advanced by step()."""

    def __init__(self, params: dict, rows: int = 1, capacity: int = 1024):
        P = self.params = params
        cfg = P["config"]
        self.layers, self.d_model, self.vocab = int(cfg[0]), int(cfg[1]), int(cfg[2])
        self.rows, self.capacity = rows, capacity
        self.embedding = P["embedding"].reshape(self.vocab, self.d_model)
        self.head = Linear(P, "head")
        self.blocks = []
        for i in range(self.layers):
            p = f"L{i}."
            d_inner, H, d_head, G, N, conv_dim, K = [int(v) for v in P[p + "mamba.dims"]]
            blk = {"hybrid": bool(P[p + "kind"][0]), "eps": float(P[p + "core_norm_eps"][0]),
                   "core_norm": P.get(p + "core_norm"),
                   "m": {n: Linear(P, p + "mamba." + n) for n in ("x", "z", "B", "C", "dt", "out")},
                   "dims": (d_inner, H, d_head, G, N, conv_dim, K), "norm_eps": float(P[p + "mamba.norm_eps"][0]),
                   "ring": np.zeros((rows, max(K - 1, 0), conv_dim), np.float32),
                   "state": np.zeros((rows, d_inner, N), np.float32)}
            if blk["hybrid"]:
                nh, nkv, hd, _, window, _ = [int(v) for v in P[p + "attn.dims"]]
                blk["attn"] = {n: Linear(P, p + "attn." + n) for n in ("q", "kv", "out")}
                blk["adims"] = (nh, nkv, hd, window)
                blk["cos"], blk["sin"] = P[p + "attn.cos"], P[p + "attn.sin"]
                blk["k_cache"] = np.zeros((rows, capacity, nkv * hd), np.float32)
                blk["v_cache"] = np.zeros((rows, capacity, nkv * hd), np.float32)
                blk["tokens"] = np.zeros(rows, np.int32)
                blk["ffn_up"], blk["ffn_down"] = Linear(P, p + "ffn.up"), Linear(P, p + "ffn.down")
            self.blocks.append(blk)

    def _mamba(self, blk, i, u):
        O, P = _port(), self.params
        p = f"L{i}.mamba."
        d_inner, H, d_head, G, N, conv_dim, K = blk["dims"]
        m = blk["m"]
        xv, z, Bv, Cv, dt = m["x"](u), m["z"](u), m["B"](u), m["C"](u), m["dt"](u)
        xBC = O.mamba_conv_step(xv, Bv, Cv, P[p + "conv_w"], P[p + "conv_b"], blk["ring"], K)
        y = O.mamba_ssd_step(xBC, dt, P[p + "A_log"], P[p + "D"], blk["state"], H, d_head, N, G)
        return m["out"](O.row_norm(y, z, P[p + "norm_w"], blk["norm_eps"]))

    def step(self, tokens):
        """tokens: `rows` ids.  Returns (hidden [layers + 1, rows, d_model], logits [rows, vocab])."""
        O, P = _port(), self.params
        h = np.ascontiguousarray(self.embedding[np.asarray(tokens, np.int64)], np.float32)
        trace = [h]
        for i, blk in enumerate(self.blocks):
            p = f"L{i}."
            core = O.row_norm(h, None, blk["core_norm"], blk["eps"])
            if not blk["hybrid"]:
                h = h + self._mamba(blk, i, core)
            else:
                attn_in = O.row_norm(h, None, P[p + "attn_norm"], blk["eps"])
                mamba = self._mamba(blk, i, core)
                nh, nkv, hd, window = blk["adims"]
                a = blk["attn"]
                heads = O.attention_decode(a["q"](attn_in), a["kv"](attn_in), blk["k_cache"], blk["v_cache"],
                                           blk["tokens"], blk["cos"], blk["sin"], nh, nkv, hd, window)
                attn = a["out"](heads)
                res = h + (mamba * P[p + "mamba_gate"] + attn * P[p + "attn_gate"])
                ff_in = O.row_norm(res, None, P[p + "ff_norm"], 1e-5)
                ff = blk["ffn_down"](O.squared_relu(blk["ffn_up"](ff_in)))
                h = res + ff * P[p + "ffn_gate"]
            trace.append(h)
        logits = self.head(O.row_norm(h, None, P["final_norm"], 1e-5))
        return np.stack(trace), logits

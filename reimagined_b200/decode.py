"""Host-side mirror of the reference model's streaming inference surface on top of `tbl_decode_step`.

`DecodeEngine` plays the role of `nsos::JambaModel` for single-token streaming decode
(OXN/nsos/include/jamba.h:577-700: `forward_ids_last`, `reset_session`, `reserve_kv_cache`,
`forward_ids_decode_graph`): it uploads a parameter set, owns the device state of a batch of independent
sequences (positions, conv windows, SSM states, KV caches) and enqueues one step per call through the C ABI;
`capture()` records the step in a CUDA graph that is then replayed per token.  torch only owns device memory
and streams.  The parameter set is a dict of named numpy arrays:

    config            int32 [12]  (num_layers, d_model, vocab, n_heads, n_kv_heads, d_state, expand, conv_kernel,
                                   head_dim, n_groups, attention_period, attention_slot)
    embedding, final_norm, L<i>.core_norm, L<i>.mamba.{A_log,D,conv_w,conv_b,norm_w}, gates, norms, rope tables ...
    <linear>.words / .scale / .magnitude / .bias / .meta   for head, L<i>.mamba.{x,z,B,C,dt,out},
                                                           L<i>.attn.{q,kv,out}, L<i>.ffn.{up,down}
    (meta = in, out, use_bias, rms_input, use_magnitude, activation bits)

`synthetic_params` draws such a set for any configuration (weights N(0, 0.02) packed by the library's packer).

    python -m reimagined_b200.decode --batch 1          # time the D768 / 16-block hybrid, one JSON line
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import math
from typing import Dict, List, Optional

import numpy as np
import torch

from . import capi

CFG_FIELDS = ("num_layers", "d_model", "vocab_size", "n_heads", "n_kv_heads", "mamba_d_state", "mamba_expand",
              "mamba_conv_kernel", "mamba_head_dim", "mamba_n_groups", "attention_period", "attention_slot")

# the benchmark's decode configuration: D768, 16 blocks, every 8th a Mamba-2 + attention + FFN block
D768_L16 = dict(num_layers=16, d_model=768, vocab_size=32000, n_heads=12, n_kv_heads=12, mamba_d_state=16,
                mamba_expand=2, mamba_conv_kernel=4, mamba_head_dim=64, mamba_n_groups=1, attention_period=8,
                attention_slot=7)


def _pack(rng, n: int, k: int):
    L = capi.lib()
    w = rng.standard_normal((n, k), dtype=np.float32)
    w *= np.float32(0.02)
    words = np.zeros(L.tbl_packed_words(n, k), np.uint32)
    scale = np.zeros(1, np.float32)
    capi.check(L.tbl_pack_weights(w.ctypes.data, n, k, words.ctypes.data, scale.ctypes.data), "tbl_pack_weights")
    return words, scale


def synthetic_params(cfg: dict, seed: int = 1, rope_positions: int = 1024) -> Dict[str, np.ndarray]:
    """A random-init parameter set with the reference model's structure and initial value ranges."""
    rng = np.random.default_rng(seed)
    P: Dict[str, np.ndarray] = {}
    D, V = cfg["d_model"], cfg["vocab_size"]
    d_inner = cfg["mamba_expand"] * D
    hd, G, N, K = cfg["mamba_head_dim"], cfg["mamba_n_groups"], cfg["mamba_d_state"], cfg["mamba_conv_kernel"]
    H = d_inner // hd
    conv_dim = d_inner + 2 * G * N

    def linear(name, n, k, bias=False, default_mode=False):
        words, scale = _pack(rng, n, k)
        P[name + ".words"], P[name + ".scale"] = words, scale
        P[name + ".magnitude"] = np.ones(n, np.float32)
        if bias:
            P[name + ".bias"] = (0.01 * rng.standard_normal(n)).astype(np.float32)
        P[name + ".meta"] = np.asarray([k, n, int(bias), int(default_mode), int(default_mode), 8], np.int32)

    P["config"] = np.asarray([cfg[f] for f in CFG_FIELDS], np.int32)
    P["embedding"] = (0.02 * rng.standard_normal((V, D))).astype(np.float32).reshape(-1)
    P["final_norm"] = rng.uniform(0.5, 1.5, D).astype(np.float32)
    linear("head", V, D)
    for i in range(cfg["num_layers"]):
        p = f"L{i}."
        hybrid = i % cfg["attention_period"] == cfg["attention_slot"]
        P[p + "kind"] = np.asarray([int(hybrid), int(not hybrid), 1], np.int32)
        P[p + "core_norm_eps"] = np.asarray([1e-5], np.float32)
        P[p + "core_norm"] = rng.uniform(0.5, 1.5, D).astype(np.float32)
        P[p + "mamba.dims"] = np.asarray([d_inner, H, hd, G, N, conv_dim, K], np.int32)
        P[p + "mamba.norm_eps"] = np.asarray([1e-5], np.float32)
        linear(p + "mamba.x", d_inner, D)
        linear(p + "mamba.z", d_inner, D)
        linear(p + "mamba.B", G * N, D)
        linear(p + "mamba.C", G * N, D)
        linear(p + "mamba.dt", H, D, bias=True)
        dt = np.exp(rng.uniform(math.log(1e-3), math.log(1e-1), H))
        P[p + "mamba.dt.bias"] = (dt + np.log(-np.expm1(-dt))).astype(np.float32)
        linear(p + "mamba.out", D, d_inner)
        P[p + "mamba.A_log"] = np.log(rng.uniform(1.0, 16.0, H)).astype(np.float32)
        P[p + "mamba.D"] = rng.uniform(0.5, 1.5, H).astype(np.float32)
        bound = 1.0 / math.sqrt(K)
        P[p + "mamba.conv_w"] = rng.uniform(-bound, bound, conv_dim * K).astype(np.float32)
        P[p + "mamba.conv_b"] = rng.uniform(-bound, bound, conv_dim).astype(np.float32)
        P[p + "mamba.norm_w"] = rng.uniform(0.5, 1.5, d_inner).astype(np.float32)
        if hybrid:
            nh, nkv = cfg["n_heads"], cfg["n_kv_heads"]
            ahd = D // nh
            for name, init in (("attn_norm", None), ("ff_norm", None), ("mamba_gate", 1.0), ("attn_gate", 0.01),
                               ("ffn_gate", 0.01)):
                P[p + name] = (rng.uniform(0.5, 1.5, D) * (init or 1.0)).astype(np.float32)
            P[p + "attn.dims"] = np.asarray([nh, nkv, ahd, max(nh // nkv, 1), 4096, rope_positions], np.int32)
            pos = np.arange(rope_positions, dtype=np.float32)[:, None]
            freq = (1.0 / np.power(np.float32(10000.0), (2.0 * np.arange(ahd // 2) / ahd).astype(np.float32))).astype(np.float32)
            angle = (pos * freq[None, :]).astype(np.float32)
            P[p + "attn.cos"], P[p + "attn.sin"] = np.cos(angle).reshape(-1), np.sin(angle).reshape(-1)
            linear(p + "attn.q", D, D, bias=True)
            linear(p + "attn.kv", 2 * nkv * ahd, D, bias=True)
            linear(p + "attn.out", D, D, bias=True)
            linear(p + "ffn.up", 4 * D, D, bias=True)
            linear(p + "ffn.down", D, 4 * D, bias=True)
    return P


class DecodeEngine:
    """Streaming decode of `batch` independent sequences (see the module docstring)."""

    def __init__(self, params: Dict[str, np.ndarray], batch: int = 1, capacity: int = 1024):
        if not torch.cuda.is_available():
            raise RuntimeError("the decode step runs on CUDA devices only (no CPU fallback)")
        self.L = capi.lib()
        self.batch, self.capacity = int(batch), int(capacity)
        self._keep: List[torch.Tensor] = []
        P = params
        cfg = P["config"]
        self.n_blocks, self.d_model, self.vocab = int(cfg[0]), int(cfg[1]), int(cfg[2])
        self.ternary_weights = 0
        stream = torch.cuda.current_stream().cuda_stream
        blocks = (capi.DecodeBlock * self.n_blocks)()
        for i in range(self.n_blocks):
            p = f"L{i}."
            b = blocks[i]
            b.hybrid = int(P[p + "kind"][0])
            b.core_norm_w = self._f32(P.get(p + "core_norm"))
            b.core_norm_eps = float(P[p + "core_norm_eps"][0])
            d_inner, H, d_head, G, N, conv_dim, K = [int(v) for v in P[p + "mamba.dims"]]
            m = b.mamba
            for name in ("x", "z", "B", "C", "dt", "out"):
                setattr(m, name, self._view(P, p + "mamba." + name, stream))
            m.A_log, m.D = self._f32(P[p + "mamba.A_log"]), self._f32(P[p + "mamba.D"])
            m.conv_w, m.conv_b = self._f32(P[p + "mamba.conv_w"]), self._f32(P[p + "mamba.conv_b"])
            m.norm_w = self._f32(P[p + "mamba.norm_w"])
            m.d_inner, m.n_heads, m.d_head, m.n_groups, m.d_state, m.conv_kernel = d_inner, H, d_head, G, N, K
            m.norm_eps = float(P[p + "mamba.norm_eps"][0])
            if b.hybrid:
                nh, nkv, hd, _, window, _ = [int(v) for v in P[p + "attn.dims"]]
                b.attn_norm_w, b.ff_norm_w = self._f32(P.get(p + "attn_norm")), self._f32(P.get(p + "ff_norm"))
                b.mamba_gate, b.attn_gate = self._f32(P[p + "mamba_gate"]), self._f32(P[p + "attn_gate"])
                b.ffn_gate = self._f32(P[p + "ffn_gate"])
                a = b.attn
                for name in ("q", "kv", "out"):
                    setattr(a, name, self._view(P, p + "attn." + name, stream))
                a.rope_cos, a.rope_sin = self._f32(P[p + "attn.cos"]), self._f32(P[p + "attn.sin"])
                a.n_heads, a.n_kv_heads, a.head_dim, a.sliding_window = nh, nkv, hd, window
                a.rope_positions = int(P[p + "attn.cos"].size // (hd // 2))
                b.ffn_up, b.ffn_down = self._view(P, p + "ffn.up", stream), self._view(P, p + "ffn.down", stream)
        self._blocks = blocks
        model = capi.DecodeModel()
        model.d_model, model.vocab, model.n_blocks = self.d_model, self.vocab, self.n_blocks
        model.embedding = self._f32(P["embedding"])
        model.blocks = C.cast(blocks, C.POINTER(capi.DecodeBlock))
        model.final_norm_w, model.final_norm_eps = self._f32(P.get("final_norm")), 1e-5
        model.head = self._view(P, "head", stream)
        self.model = model
        state_bytes = self.L.tbl_decode_state_bytes(C.byref(model), self.batch, self.capacity)
        ws_bytes = self.L.tbl_decode_workspace_bytes(C.byref(model), self.batch)
        if state_bytes == 0 or ws_bytes == 0:
            raise ValueError("the library rejected the model description (shapes inconsistent)")
        self.state = torch.empty(state_bytes, dtype=torch.uint8, device="cuda")
        self.workspace = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        self.tokens = torch.zeros(self.batch, dtype=torch.int32, device="cuda")
        self.logits = torch.empty((self.batch, self.vocab), dtype=torch.float32, device="cuda")
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.launches_per_step = 0
        self.reset()

    # ---- uploads ------------------------------------------------------------------------------------
    def _f32(self, a):
        if a is None:
            return None
        t = torch.from_numpy(np.ascontiguousarray(a, np.float32)).cuda()
        self._keep.append(t)
        return t.data_ptr()

    def _view(self, P, name: str, stream) -> capi.LinearView:
        meta = P[name + ".meta"]
        k, n, use_bias, rms, use_mag, bits = [int(v) for v in meta]
        self.ternary_weights += n * k
        words = torch.from_numpy(np.ascontiguousarray(P[name + ".words"]).view(np.int32)).cuda()
        self._keep.append(words)
        strips = None
        nbytes = self.L.tbl_strip_bytes(n, k)
        if nbytes:
            strips = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            capi.check(self.L.tbl_relayout_strips(words.data_ptr(), n, k, strips.data_ptr(), stream), "tbl_relayout_strips")
            self._keep.append(strips)
        v = capi.LinearView()
        v.weight = None
        v.packed = words.data_ptr()
        v.magnitude = self._f32(P[name + ".magnitude"]) if use_mag else None
        v.bias = self._f32(P[name + ".bias"]) if use_bias else None
        v.inputs, v.outputs, v.activation_bits, v.rms_input = k, n, bits, rms
        v.weight_scale = float(P[name + ".scale"][0])
        v.strips = strips.data_ptr() if strips is not None else None
        v.w_i8 = None
        return v

    # ---- the reference model's streaming surface ---------------------------------------------------
    def reset(self) -> None:
        """JambaModel::reset_session: empty caches, positions at zero."""
        capi.check(self.L.tbl_decode_state_reset(C.byref(self.model), self.batch, self.capacity, self.state.data_ptr(),
                                                 self.state.numel(), torch.cuda.current_stream().cuda_stream),
                   "tbl_decode_state_reset")

    def _enqueue(self, trace_ptr=None) -> None:
        capi.check(self.L.tbl_decode_step(C.byref(self.model), self.batch, self.capacity, self.state.data_ptr(),
                                          self.tokens.data_ptr(), self.logits.data_ptr(), trace_ptr,
                                          self.workspace.data_ptr(), self.workspace.numel(),
                                          torch.cuda.current_stream().cuda_stream), "tbl_decode_step")

    def step(self, token_ids, trace: bool = False):
        """One token per sequence -> logits [batch, vocab] (device tensor, overwritten by the next step); with
        `trace` also the residual stream [n_blocks + 1, batch, d_model]."""
        ids = torch.as_tensor(token_ids, dtype=torch.int32).reshape(self.batch)
        self.tokens.copy_(ids, non_blocking=True)
        hidden = None
        if trace:
            hidden = torch.empty((self.n_blocks + 1, self.batch, self.d_model), dtype=torch.float32, device="cuda")
        if self.graph is not None and not trace:
            self.graph.replay()
        else:
            self._enqueue(hidden.data_ptr() if trace else None)
        return (self.logits, hidden) if trace else self.logits

    def capture(self) -> int:
        """Records one step in a CUDA graph (JambaModel::forward_ids_decode_graph); returns the number of kernels
        in it.  Call after at least one eager step (one-time kernel attributes are set on first use)."""
        torch.cuda.synchronize()
        before = self.L.tbl_launch_count()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._enqueue(None)
        self.launches_per_step = int(self.L.tbl_launch_count() - before)
        self.graph = graph
        # the capture did not run the step; nothing to undo in the state
        return self.launches_per_step


def main() -> None:
    ap = argparse.ArgumentParser(description="time one decode step of the D768 / 16-block hybrid")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--context", type=int, default=512, help="tokens already in the KV cache when timing starts")
    args = ap.parse_args()
    print(json.dumps(time_decode(args.batch, args.iters, args.context)))


def time_decode(batch: int, iters: int = 50, context: int = 512, cfg: Optional[dict] = None, seed: int = 1) -> dict:
    cfg = cfg or D768_L16
    params = synthetic_params(cfg, seed)
    eng = DecodeEngine(params, batch=batch, capacity=context + iters + 8)
    gen = torch.Generator().manual_seed(seed)
    draw = lambda: torch.randint(0, cfg["vocab_size"], (batch,), generator=gen, dtype=torch.int32).cuda()
    eng.step(draw())
    launches = eng.capture()
    for _ in range(context - 1):             # fill the caches: the timed steps attend over `context` tokens
        eng.step(draw())
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ids = [draw() for _ in range(iters)]
    e0.record()
    for t in ids:
        eng.step(t)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    status = eng.L.tbl_device_status(torch.cuda.current_stream().cuda_stream)
    return {"workload": f"D{cfg['d_model']}/L{cfg['num_layers']} decode step (every op of the step)", "batch": batch,
            "context_tokens": context, "kernel_launches_per_step": launches, "us_per_step": round(us, 1),
            "tokens_per_s": round(batch / us * 1e6, 1), "ternary_weights": eng.ternary_weights,
            "packed_mb": round(eng.ternary_weights / 4 / 1e6, 2), "device_status": status}


if __name__ == "__main__":
    main()

"""Host-side mirror of the reference's ``nsos::BitLinear`` packed-inference surface
(OXN/nsos/include/bitlinear.h:77-212) on top of the C ABI.

Only what the packed inference path needs is mirrored: construction from fp32 weights or from an
exported packed state, ``to(device)``, ``forward``, ``set_exact_linear_mode``,
``export_packed_state`` / ``import_packed_state``, ``prepare_gpu_decode_view``.  Training,
QAT, LoQA, Hadamard and the float reference path are not part of this library.

torch owns device memory and streams here; every computation is a C-ABI call into
libternary_b200.so (there is no PyTorch or CPU fallback).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional

import numpy as np
import torch

from . import capi


@dataclass
class BitLinearPackedState:
    """Mirror of nsos::BitLinearPackedState (OXN/nsos/include/bitlinear.h:37-47)."""
    in_features: int = 0
    out_features: int = 0
    use_bias: bool = True
    weight_scale: float = 1.0
    packed_weights: np.ndarray = field(default_factory=lambda: np.zeros(0, np.uint32))
    magnitude: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    bias: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    # per-input affine of the reference's Hadamard/"flat" option, carried for interchange (ones / zeros when unused)
    flat_alpha: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))
    flat_beta: np.ndarray = field(default_factory=lambda: np.zeros(0, np.float32))


class BitLinear:
    """Packed ternary linear.  Default mode = input RMSNorm(1e-6) + magnitude [+ bias];
    exact-linear mode = none of those (bitlinear.h:99-108)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True):
        if in_features <= 0 or out_features <= 0:
            raise ValueError("BitLinear feature counts must be positive")
        self.in_features = in_features
        self.out_features = out_features
        self.use_bias = bias
        self.precision_bits = 8
        self.exact_linear_mode = False
        self.rms_mode = 1                      # TBL_RMS_FAST; 2 reproduces the CPU sum order bit for bit
        self.weight_scale = 1.0
        self.packed_weights = np.zeros(0, np.uint32)
        self.magnitude = np.ones(out_features, np.float32)
        self.bias = np.zeros(out_features if bias else 0, np.float32)
        self.flat_alpha = np.ones(in_features, np.float32)
        self.flat_beta = np.zeros(in_features, np.float32)
        self._dev = None                       # device buffers after to("cuda")
        self._ws = None

    # ---- construction -------------------------------------------------------------------
    @classmethod
    def from_float(cls, weight: np.ndarray, bias: Optional[np.ndarray] = None) -> "BitLinear":
        """Packs fp32 weights [out,in] with the host packer (== BitLinear::repack_weights)."""
        w = np.ascontiguousarray(weight, np.float32)
        n, k = w.shape
        layer = cls(k, n, bias is not None)
        L = capi.lib()
        words = np.zeros(L.tbl_packed_words(n, k), np.uint32)
        scale = np.zeros(1, np.float32)
        capi.check(L.tbl_pack_weights(w.ctypes.data, n, k, words.ctypes.data, scale.ctypes.data), "tbl_pack_weights")
        layer.packed_weights, layer.weight_scale = words, float(scale[0])
        if bias is not None:
            layer.bias = np.ascontiguousarray(bias, np.float32)
        return layer

    def set_exact_linear_mode(self, enabled: bool) -> None:
        self.exact_linear_mode = bool(enabled)

    def set_precision_mode(self, bits: int) -> None:
        if not 2 <= bits <= 8:
            raise ValueError("activation bits must be in [2,8]")
        self.precision_bits = bits

    def export_packed_state(self) -> BitLinearPackedState:
        return BitLinearPackedState(self.in_features, self.out_features, self.use_bias, self.weight_scale,
                                    self.packed_weights.copy(), self.magnitude.copy(), self.bias.copy(),
                                    self.flat_alpha.copy(), self.flat_beta.copy())

    def import_packed_state(self, state: BitLinearPackedState) -> None:
        """Validate first, install afterwards (a rejected state leaves the layer untouched)."""
        if (state.in_features, state.out_features, state.use_bias) != (self.in_features, self.out_features, self.use_bias):
            raise RuntimeError("BitLinear packed state shape mismatch")
        words = np.ascontiguousarray(state.packed_weights, np.uint32)
        mag = np.ascontiguousarray(state.magnitude, np.float32)
        bias = np.ascontiguousarray(state.bias, np.float32)
        alpha = np.ascontiguousarray(state.flat_alpha, np.float32) if state.flat_alpha.size else np.ones(self.in_features, np.float32)
        beta = np.ascontiguousarray(state.flat_beta, np.float32) if state.flat_beta.size else np.zeros(self.in_features, np.float32)
        if mag.size != self.out_features or bias.size != (self.out_features if self.use_bias else 0) or \
                alpha.size != self.in_features or beta.size != self.in_features:
            raise RuntimeError("BitLinear packed state buffer length mismatch")
        if not (np.isfinite(alpha).all() and np.isfinite(beta).all()):
            raise RuntimeError("BitLinear packed state contains non-finite values")
        rc = capi.lib().tbl_validate_packed(words.ctypes.data, words.size, self.out_features, self.in_features,
                                            float(state.weight_scale), mag.ctypes.data,
                                            bias.ctypes.data if bias.size else None)
        capi.check(rc, "tbl_validate_packed")
        self.packed_weights, self.weight_scale, self.magnitude, self.bias = words, float(state.weight_scale), mag, bias
        self.flat_alpha, self.flat_beta = alpha, beta
        if self._dev is not None:
            self.to("cuda")

    # ---- device residency ---------------------------------------------------------------
    def to(self, device: str = "cuda", with_int8: bool = True) -> "BitLinear":
        """Uploads the canonical words once and derives the two device layouts: strips for the decode
        GEMV (K % 256 == 0) and, if asked, the int8 copy the tcgen05 prefill GEMM reads."""
        if device != "cuda":
            raise ValueError("the ternary linear path runs on CUDA devices only")
        L = capi.lib()
        n, k = self.out_features, self.in_features
        st = torch.cuda.current_stream().cuda_stream
        words = torch.from_numpy(self.packed_weights.view(np.int32)).cuda()
        dev = {"words": words, "strips": None, "w_i8": None,
               "magnitude": torch.from_numpy(self.magnitude).cuda(),
               "bias": torch.from_numpy(self.bias).cuda() if self.use_bias else None}
        nbytes = L.tbl_strip_bytes(n, k)
        if nbytes and k <= 65536:
            dev["strips"] = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            capi.check(L.tbl_relayout_strips(words.data_ptr(), n, k, dev["strips"].data_ptr(), st), "tbl_relayout_strips")
        if with_int8 and k % 16 == 0:
            dev["w_i8"] = torch.empty((n, k), dtype=torch.int8, device="cuda")
            capi.check(L.tbl_expand_weights_i8(words.data_ptr(), n, k, dev["w_i8"].data_ptr(), st), "tbl_expand_weights_i8")
        self._dev = dev
        return self

    def _workspace(self, m: int) -> torch.Tensor:
        need = capi.lib().tbl_linear_workspace_bytes(m, self.in_features, self.out_features)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(max(need, 256), dtype=torch.uint8, device="cuda")
        return self._ws

    # ---- forward ------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x fp32 CUDA [..., in] -> fp32 CUDA [..., out]; enqueued on the current stream, no sync."""
        if self._dev is None:
            raise RuntimeError("call to('cuda') before forward")
        if x.dtype != torch.float32 or not x.is_cuda or not x.is_contiguous():
            raise ValueError("input must be a contiguous fp32 CUDA tensor")
        k, n = self.in_features, self.out_features
        m = x.numel() // k
        y = out if out is not None else torch.empty((m, n), dtype=torch.float32, device="cuda")
        ws = self._workspace(m)
        d = self._dev
        exact = self.exact_linear_mode
        rc = capi.lib().tbl_linear_forward(
            x.data_ptr(), d["words"].data_ptr(), d["strips"].data_ptr() if d["strips"] is not None else None,
            d["w_i8"].data_ptr() if d["w_i8"] is not None else None, self.weight_scale, m, k, n,
            self.precision_bits, 0 if exact else self.rms_mode,
            None if exact else d["magnitude"].data_ptr(), d["bias"].data_ptr() if self.use_bias else None,
            y.data_ptr(), ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        capi.check(rc, "tbl_linear_forward")
        if out is None and x.dim() != 2:
            return y.reshape(*x.shape[:-1], n)
        return y

    def prepare_gpu_decode_view(self) -> capi.LinearView:
        """Borrowed descriptor for the grouped entry points (GpuLinearView of the reference)."""
        if self._dev is None:
            raise RuntimeError("call to('cuda') first")
        d = self._dev
        return capi.LinearView(None, d["words"].data_ptr(),
                               None if self.exact_linear_mode else d["magnitude"].data_ptr(),
                               d["bias"].data_ptr() if self.use_bias else None,
                               self.in_features, self.out_features, self.precision_bits,
                               0 if self.exact_linear_mode else 1, self.weight_scale,
                               d["strips"].data_ptr() if d["strips"] is not None else None)

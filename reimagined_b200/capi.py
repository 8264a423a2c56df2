"""ctypes bindings of every symbol declared in include/ternary_b200.h.

Pointers are passed as integers (``tensor.data_ptr()`` for device memory, ``array.ctypes.data`` for
host memory); nothing here copies, allocates or falls back to a CPU path.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libternary_b200.so")


class TernaryB200Error(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = lib().tbl_status_string(status).decode()
        super().__init__(f"{where}: status {status} ({msg})")


class LinearView(C.Structure):
    """Field-for-field tbl_linear_view (the reference's GpuLinearView)."""

    _fields_ = [("weight", C.c_void_p), ("packed", C.c_void_p), ("magnitude", C.c_void_p),
                ("bias", C.c_void_p), ("inputs", C.c_int), ("outputs", C.c_int),
                ("activation_bits", C.c_int), ("rms_input", C.c_int), ("weight_scale", C.c_float),
                ("strips", C.c_void_p), ("w_i8", C.c_void_p)]


class EdgeLayer(C.Structure):
    """tbl_edge_layer: one layer record of an edge-linear pack (byte offsets into the image)."""

    _fields_ = [("sensitive", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int), ("use_bias", C.c_int),
                ("weight_scale", C.c_float), ("packed_offset", C.c_uint64), ("packed_words", C.c_uint64),
                ("magnitude_offset", C.c_uint64), ("bias_offset", C.c_uint64), ("flat_alpha_offset", C.c_uint64),
                ("flat_beta_offset", C.c_uint64), ("weight_offset", C.c_uint64), ("weight_count", C.c_uint64)]


class EdgeLayerSrc(C.Structure):
    """tbl_edge_layer_src: one layer handed to the pack writer."""

    _fields_ = [("sensitive", C.c_int), ("in_features", C.c_int), ("out_features", C.c_int), ("use_bias", C.c_int),
                ("weight_scale", C.c_float), ("packed", C.c_void_p), ("magnitude", C.c_void_p), ("bias", C.c_void_p),
                ("flat_alpha", C.c_void_p), ("flat_beta", C.c_void_p), ("weight", C.c_void_p)]


class MambaBlock(C.Structure):
    """tbl_mamba_block."""

    _fields_ = [("x", LinearView), ("z", LinearView), ("B", LinearView), ("C", LinearView), ("dt", LinearView),
                ("out", LinearView), ("A_log", C.c_void_p), ("D", C.c_void_p), ("conv_w", C.c_void_p),
                ("conv_b", C.c_void_p), ("norm_w", C.c_void_p), ("d_inner", C.c_int), ("n_heads", C.c_int),
                ("d_head", C.c_int), ("n_groups", C.c_int), ("d_state", C.c_int), ("conv_kernel", C.c_int),
                ("norm_eps", C.c_float)]


class AttentionBlock(C.Structure):
    """tbl_attention_block."""

    _fields_ = [("q", LinearView), ("kv", LinearView), ("out", LinearView), ("rope_cos", C.c_void_p),
                ("rope_sin", C.c_void_p), ("n_heads", C.c_int), ("n_kv_heads", C.c_int), ("head_dim", C.c_int),
                ("sliding_window", C.c_int), ("rope_positions", C.c_int)]


class DecodeBlock(C.Structure):
    """tbl_decode_block."""

    _fields_ = [("hybrid", C.c_int), ("core_norm_w", C.c_void_p), ("core_norm_eps", C.c_float), ("mamba", MambaBlock),
                ("attn_norm_w", C.c_void_p), ("ff_norm_w", C.c_void_p), ("mamba_gate", C.c_void_p),
                ("attn_gate", C.c_void_p), ("ffn_gate", C.c_void_p), ("attn", AttentionBlock), ("ffn_up", LinearView),
                ("ffn_down", LinearView)]


class DecodeModel(C.Structure):
    """tbl_decode_model."""

    _fields_ = [("d_model", C.c_int), ("vocab", C.c_int), ("n_blocks", C.c_int), ("embedding", C.c_void_p),
                ("blocks", C.POINTER(DecodeBlock)), ("final_norm_w", C.c_void_p), ("final_norm_eps", C.c_float),
                ("head", LinearView)]


_vp = C.c_void_p
_SIGNATURES = {
    # name: (restype, argtypes)
    "tbl_status_string": (C.c_char_p, [C.c_int]),
    "tbl_abi_version": (C.c_int, []),
    "tbl_packed_words": (C.c_int64, [C.c_int, C.c_int]),
    "tbl_pack_weights": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp]),
    "tbl_unpack_weights_i8": (C.c_int, [_vp, C.c_int, C.c_int, _vp]),
    "tbl_validate_packed": (C.c_int, [_vp, C.c_int64, C.c_int, C.c_int, C.c_float, _vp, _vp]),
    "tbl_strip_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "tbl_relayout_strips": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp]),
    "tbl_expand_weights_i8": (C.c_int, [_vp, C.c_int, C.c_int, _vp, _vp]),
    "tbl_quantize_rows": (C.c_int, [_vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp, _vp]),
    "tbl_gemv_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "tbl_gemv": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp,
                           C.c_size_t, _vp]),
    "tbl_gemm": (C.c_int, [_vp, _vp, _vp, C.c_float, _vp, _vp, C.c_int, C.c_int, C.c_int, _vp, _vp, _vp]),
    "tbl_linear_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "tbl_linear_forward": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                     _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "tbl_linear_forward_noalloc": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                             _vp, _vp, _vp, _vp]),
    "tbl_grouped_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "tbl_grouped_forward": (C.c_int, [C.POINTER(LinearView), C.c_int, _vp, _vp, C.c_int, C.c_int, _vp,
                                      C.c_size_t, _vp]),
    "tbl_grouped_rows_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "tbl_grouped_forward_rows": (C.c_int, [C.POINTER(LinearView), C.c_int, _vp, C.c_int, _vp, C.c_longlong, C.c_int,
                                           _vp, C.c_size_t, _vp]),
    "tbl_chain_workspace_bytes": (C.c_size_t, [C.POINTER(LinearView), C.c_int, C.c_int]),
    "tbl_chain_forward": (C.c_int, [C.POINTER(LinearView), C.c_int, C.POINTER(C.c_int), _vp, C.c_int, C.c_int, _vp, _vp,
                                    C.c_size_t, _vp]),
    "tbl_embedding_gather": (C.c_int, [_vp, C.c_int, _vp, C.c_int, C.c_int, _vp, _vp]),
    "tbl_mamba_conv_step": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "tbl_mamba_ssd_step": (C.c_int, [_vp, _vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp]),
    "tbl_attention_decode": (C.c_int, [_vp, _vp, _vp, _vp, C.c_int, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                       C.c_int, C.c_int, _vp, _vp]),
    "tbl_gated_residual": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int, C.c_int, _vp, _vp]),
    "tbl_decode_state_bytes": (C.c_size_t, [C.POINTER(DecodeModel), C.c_int, C.c_int]),
    "tbl_decode_state_reset": (C.c_int, [C.POINTER(DecodeModel), C.c_int, C.c_int, _vp, C.c_size_t, _vp]),
    "tbl_decode_workspace_bytes": (C.c_size_t, [C.POINTER(DecodeModel), C.c_int]),
    "tbl_decode_step": (C.c_int, [C.POINTER(DecodeModel), C.c_int, C.c_int, _vp, _vp, _vp, _vp, _vp, C.c_size_t, _vp]),
    "tbl_retile_columns": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, _vp, _vp]),
    "tbl_router_topk": (C.c_int, [_vp, C.c_int, C.c_int, C.c_int, _vp, _vp]),
    "tbl_row_norm": (C.c_int, [_vp, _vp, _vp, C.c_int, C.c_int, C.c_float, _vp, C.c_int, _vp, _vp, _vp, _vp]),
    "tbl_moe_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tbl_moe_forward": (C.c_int, [C.POINTER(LinearView), _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_int,
                                  C.c_int, C.c_int, C.c_int, _vp, _vp, C.c_size_t, _vp]),
    "tbl_edge_pack_open": (C.c_int, [_vp, C.c_size_t, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tbl_edge_pack_layer": (C.c_int, [_vp, C.c_size_t, C.c_int, C.POINTER(EdgeLayer)]),
    "tbl_edge_pack_layers": (C.c_int, [_vp, C.c_size_t, C.POINTER(EdgeLayer), C.c_int, C.POINTER(C.c_int),
                                       C.POINTER(C.c_int)]),
    "tbl_edge_pack_bytes": (C.c_size_t, [C.POINTER(EdgeLayerSrc), C.c_int]),
    "tbl_edge_pack_write": (C.c_int, [C.POINTER(EdgeLayerSrc), C.c_int, _vp, C.c_size_t, C.POINTER(C.c_size_t)]),
    "tbl_sha256_hex": (None, [_vp, C.c_size_t, C.c_char_p]),
    "tbl_selftest_bounded_wait": (C.c_int, [_vp, _vp]),
    "tbl_linear_forward_scatter": (C.c_int, [_vp, _vp, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _vp, _vp,
                                             C.POINTER(C.c_void_p), C.c_int, C.c_longlong, C.c_longlong, _vp, C.c_size_t, _vp]),
    "tbl_device_status": (C.c_int, [_vp]),
    "tbl_set_kernel_events": (None, [_vp, _vp]),
    "tbl_set_chain_trace": (None, [_vp, C.c_size_t]),
    "tbl_launch_count": (C.c_uint64, []),
}

EXPORTED_SYMBOLS = tuple(_SIGNATURES)

_lib = None


def lib() -> C.CDLL:
    """Loads libternary_b200.so (once).  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python -m reimagined_b200.build` "
                "(the ternary linear path has no CPU or PyTorch fallback)")
        handle = C.CDLL(LIB_PATH)
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status: int, where: str) -> None:
    if status != 0:
        raise TernaryB200Error(status, where)

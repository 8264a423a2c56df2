"""Edge-linear packs ("DGE1" v3): read and write the file in which the reference ships a model's packed linears.

Mirror of `JambaModel::load_edge_linear_pack` / `save_edge_linear_pack` (OXN/nsos/src/jamba.cpp:1325-1663) for
the part that concerns this library: every layer comes back as the fields of the reference's
`BitLinearPackedState` (include/bitlinear.h:37-47), ready for `BitLinear.import_packed_state`.  Parsing,
validation (lengths, finite values, reserved codes, SHA-256 trailer) and serialisation are done by the C
library (`tbl_edge_pack_*`); this module only moves bytes between files and numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import tempfile
from typing import Dict, List

import numpy as np

from . import capi


def _array(image: bytes, offset: int, count: int, dtype) -> np.ndarray:
    # payloads are not aligned inside the file: copy
    return np.frombuffer(image, dtype=np.uint8, count=count * np.dtype(dtype).itemsize, offset=offset).copy().view(dtype)


def loads(image: bytes) -> List[Dict]:
    """Parse and validate a pack held in memory; raises capi.TernaryB200Error with the library's status."""
    L = capi.lib()
    version, layers = C.c_int(0), C.c_int(0)
    # the layer count sits in the header; one pass then hashes, validates and returns every record
    count = int.from_bytes(image[8:12], "little") if len(image) >= 12 else 0
    records = (capi.EdgeLayer * max(count, 1))()
    capi.check(L.tbl_edge_pack_layers(image, len(image), records, count, C.byref(version), C.byref(layers)),
               "tbl_edge_pack_layers")
    out = []
    for index in range(layers.value):
        rec = records[index]
        n, k = rec.out_features, rec.in_features
        out.append({
            "sensitive": bool(rec.sensitive), "in_features": k, "out_features": n, "use_bias": bool(rec.use_bias),
            "weight_scale": np.float32(rec.weight_scale),
            "packed_weights": _array(image, rec.packed_offset, rec.packed_words, np.uint32),
            "magnitude": _array(image, rec.magnitude_offset, n, np.float32),
            "bias": _array(image, rec.bias_offset, n if rec.use_bias else 0, np.float32),
            "flat_alpha": _array(image, rec.flat_alpha_offset, k, np.float32),
            "flat_beta": _array(image, rec.flat_beta_offset, k, np.float32),
            "weight": _array(image, rec.weight_offset, rec.weight_count, np.float32).reshape(n, k) if rec.sensitive else None,
            "version": version.value,
        })
    return out


def load(path: str) -> List[Dict]:
    with open(path, "rb") as f:
        return loads(f.read())


def dumps(layers: List[Dict]) -> bytes:
    """Serialise layers (dicts as returned by `loads`) into a version-3 pack with its SHA-256 trailer."""
    L = capi.lib()
    keep = []

    def ptr(a, dtype):
        if a is None:
            return None
        a = np.ascontiguousarray(a, dtype=dtype)
        keep.append(a)
        return a.ctypes.data if a.size else None

    src = (capi.EdgeLayerSrc * len(layers))()
    for rec, layer in zip(src, layers):
        rec.sensitive = int(bool(layer.get("sensitive", False)))
        rec.in_features, rec.out_features = int(layer["in_features"]), int(layer["out_features"])
        rec.use_bias = int(bool(layer.get("use_bias", False)))
        rec.weight_scale = float(layer["weight_scale"])
        rec.packed = ptr(layer["packed_weights"], np.uint32)
        rec.magnitude = ptr(layer["magnitude"], np.float32)
        rec.bias = ptr(layer.get("bias"), np.float32) if rec.use_bias else None
        rec.flat_alpha = ptr(layer["flat_alpha"], np.float32)
        rec.flat_beta = ptr(layer["flat_beta"], np.float32)
        rec.weight = ptr(layer.get("weight"), np.float32) if rec.sensitive else None
    size = L.tbl_edge_pack_bytes(src, len(layers))
    if size == 0:
        raise ValueError("edge pack: a layer is missing a required array")
    buf = C.create_string_buffer(size)
    written = C.c_size_t(0)
    capi.check(L.tbl_edge_pack_write(src, len(layers), buf, size, C.byref(written)), "tbl_edge_pack_write")
    return buf.raw[: written.value]


def save(path: str, layers: List[Dict]) -> None:
    """Write to a temporary file in the same directory, flush, then replace (the reference's atomic_replace)."""
    image = dumps(layers)
    directory = os.path.dirname(os.path.abspath(path))
    os.makedirs(directory, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix=".edge_pack_", dir=directory)
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(image)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def sha256_hex(data: bytes) -> str:
    out = C.create_string_buffer(65)
    capi.lib().tbl_sha256_hex(data, len(data), out)
    return out.value.decode()


def to_bitlinear(layer: Dict):
    """A non-sensitive pack layer as a `BitLinear` (import_packed_state re-validates before installing).
    Sensitive layers stay on the reference's fp32 path and have no ternary linear to build."""
    from .bitlinear import BitLinear, BitLinearPackedState

    if layer["sensitive"]:
        raise ValueError("a quantisation-sensitive layer runs in fp32 in the reference; it has no packed linear")
    lin = BitLinear(layer["in_features"], layer["out_features"], bias=layer["use_bias"])
    lin.import_packed_state(BitLinearPackedState(
        in_features=layer["in_features"], out_features=layer["out_features"], use_bias=layer["use_bias"],
        weight_scale=float(layer["weight_scale"]), packed_weights=layer["packed_weights"],
        magnitude=layer["magnitude"], bias=layer["bias"], flat_alpha=layer["flat_alpha"], flat_beta=layer["flat_beta"]))
    return lin


def from_bitlinear(lin) -> Dict:
    """The pack record of a `BitLinear` (the inverse of `to_bitlinear`)."""
    st = lin.export_packed_state()
    return {"sensitive": False, "in_features": st.in_features, "out_features": st.out_features, "use_bias": st.use_bias,
            "weight_scale": np.float32(st.weight_scale), "packed_weights": st.packed_weights, "magnitude": st.magnitude,
            "bias": st.bias, "flat_alpha": st.flat_alpha, "flat_beta": st.flat_beta, "weight": None}

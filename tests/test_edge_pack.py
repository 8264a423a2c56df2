"""Edge-linear pack ("DGE1") reader / writer against an independent restatement of the format and, for the
digest, against hashlib and the reference's own SHA-256 (OXN/nsos/src/sha256.cpp through oracle/_ref)."""
import ctypes as C
import hashlib
import struct

import numpy as np
import pytest

MAGIC, TRAILER_MAGIC = 0x31454744, 0x33494745


def _vec(arr, fmt_dtype):
    arr = np.ascontiguousarray(arr, dtype=fmt_dtype)
    return struct.pack("<Q", arr.size) + arr.tobytes()


def restate_pack(layers, version=3):
    """The format, written out independently of the library (jamba.cpp:1345-1439 read as a specification)."""
    body = struct.pack("<III", MAGIC, version, len(layers))
    for L in layers:
        body += struct.pack("<B", int(L["sensitive"])) + struct.pack("<ii", L["in_features"], L["out_features"])
        body += struct.pack("<B", int(L["use_bias"])) + struct.pack("<f", float(L["weight_scale"]))
        body += _vec(L["packed_weights"], np.uint32) + _vec(L["magnitude"], np.float32)
        body += _vec(L["bias"] if L["use_bias"] else [], np.float32)
        body += _vec(L["flat_alpha"], np.float32) + _vec(L["flat_beta"], np.float32)
        if L["sensitive"]:
            body += _vec(np.asarray(L["weight"]).reshape(-1), np.float32)
    if version >= 3:
        body += struct.pack("<IQ", TRAILER_MAGIC, len(body)) + hashlib.sha256(body).hexdigest().encode()
    return body


def make_layers(port, seed=0):
    rng = np.random.default_rng(seed)
    layers = []
    for (n, k, bias, sensitive) in [(24, 48, True, False), (7, 33, False, False), (5, 16, True, True), (1, 1, False, False)]:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        words, scale, *_ = port.pack_weights(w)
        layers.append({"sensitive": sensitive, "in_features": k, "out_features": n, "use_bias": bias,
                       "weight_scale": np.float32(scale), "packed_weights": np.asarray(words, np.uint32),
                       "magnitude": (1 + 0.1 * rng.standard_normal(n)).astype(np.float32),
                       "bias": rng.standard_normal(n).astype(np.float32) if bias else np.zeros(0, np.float32),
                       "flat_alpha": np.ones(k, np.float32), "flat_beta": np.zeros(k, np.float32),
                       "weight": w if sensitive else None})
    return layers


SIZES = [0, 1, 55, 56, 57, 63, 64, 65, 119, 120, 1000, 70001]


def test_sha256_matches_hashlib(tbl):
    from reimagined_b200 import edge_pack
    rng = np.random.default_rng(1)
    for size in SIZES:
        data = rng.integers(0, 256, size, dtype=np.uint8).tobytes()
        assert edge_pack.sha256_hex(data) == hashlib.sha256(data).hexdigest()


def test_sha256_matches_the_reference_build(tbl, ref):
    from reimagined_b200 import edge_pack
    rng = np.random.default_rng(2)
    ref.lib.ref_sha256_hex.argtypes = [C.c_char_p, C.c_size_t, C.c_char_p]
    ref.lib.ref_sha256_hex.restype = None
    for size in SIZES:
        data = rng.integers(0, 256, size, dtype=np.uint8).tobytes()
        out = C.create_string_buffer(65)
        ref.lib.ref_sha256_hex(data, len(data), out)
        assert out.value.decode() == edge_pack.sha256_hex(data)


def test_writer_is_byte_identical_to_the_restated_format_and_round_trips(tbl, port, tmp_path):
    from reimagined_b200 import edge_pack
    layers = make_layers(port)
    image = edge_pack.dumps(layers)
    assert image == restate_pack(layers)
    path = tmp_path / "sub" / "model.edge"
    edge_pack.save(str(path), layers)
    back = edge_pack.load(str(path))
    assert len(back) == len(layers)
    for got, want in zip(back, layers):
        for key in ("sensitive", "in_features", "out_features", "use_bias"):
            assert got[key] == want[key]
        assert np.float32(got["weight_scale"]).tobytes() == np.float32(want["weight_scale"]).tobytes()
        for key in ("packed_weights", "magnitude", "bias", "flat_alpha", "flat_beta"):
            assert np.array_equal(got[key], want[key]), key
        if want["sensitive"]:
            assert np.array_equal(got["weight"], want["weight"])
        assert got["version"] == 3


def test_reader_accepts_the_legacy_version_without_trailer(tbl, port):
    from reimagined_b200 import edge_pack
    layers = make_layers(port, seed=2)[:2]
    back = edge_pack.loads(restate_pack(layers, version=2))
    assert [b["version"] for b in back] == [2, 2]
    assert np.array_equal(back[1]["packed_weights"], layers[1]["packed_weights"])


def test_loaded_layers_feed_the_linear(tbl, port):
    """A pack's layer is a BitLinearPackedState: its words and scale give the oracle's outputs."""
    from reimagined_b200 import edge_pack
    layers = make_layers(port, seed=3)
    back = edge_pack.loads(edge_pack.dumps(layers))
    x = np.random.default_rng(4).standard_normal((3, 48)).astype(np.float32)
    a = port.linear_forward(x, layers[0]["packed_weights"], layers[0]["weight_scale"], 24,
                            magnitude=layers[0]["magnitude"], bias=layers[0]["bias"])[0]
    b = port.linear_forward(x, back[0]["packed_weights"], back[0]["weight_scale"], 24,
                            magnitude=back[0]["magnitude"], bias=back[0]["bias"])[0]
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def _status(image):
    from reimagined_b200 import capi
    version, count = C.c_int(0), C.c_int(0)
    return capi.lib().tbl_edge_pack_open(image, len(image), C.byref(version), C.byref(count))


def test_reader_rejects_what_the_reference_rejects(tbl, port):
    """The loader's refusals (jamba.cpp:1459-1616, 546-606), one corruption each."""
    from reimagined_b200 import capi
    L = capi.lib()
    FORMAT, INTEGRITY, SHAPE, SCALE, CODE = -11, -12, -2, -4, -8
    layers = make_layers(port, seed=5)
    good = restate_pack(layers)
    assert _status(good) == 0

    def mutate(fn, version=3):
        ls = [dict(l) for l in layers]
        fn(ls)
        return restate_pack(ls, version)

    assert _status(b"\x00" * 4 + good[4:]) == FORMAT                         # magic
    assert _status(good[:4] + struct.pack("<I", 4) + good[8:]) == FORMAT     # version
    assert _status(good[:40]) == FORMAT                                      # too small for its trailer
    assert _status(good[:-1] + (b"0" if good[-1:] != b"0" else b"1")) == INTEGRITY   # digest
    flipped = bytearray(good); flipped[100] ^= 1
    assert _status(bytes(flipped)) == INTEGRITY                              # payload changed under the digest
    assert _status(good[:-76] + struct.pack("<IQ", TRAILER_MAGIC, 5) + good[-64:]) == INTEGRITY   # trailer length
    assert _status(restate_pack(layers, 2) + b"\x00") == FORMAT              # legacy pack with trailing bytes

    def bad_code(ls): w = ls[0]["packed_weights"].copy(); w[1] |= 3 << 6; ls[0]["packed_weights"] = w
    assert _status(mutate(bad_code)) == CODE
    def nan_mag(ls): m = ls[1]["magnitude"].copy(); m[0] = np.nan; ls[1]["magnitude"] = m
    assert _status(mutate(nan_mag)) == FORMAT
    def inf_weight(ls): w = ls[2]["weight"].copy(); w[0, 0] = np.inf; ls[2]["weight"] = w
    assert _status(mutate(inf_weight)) == FORMAT
    def zero_scale(ls): ls[0]["weight_scale"] = np.float32(0)
    assert _status(mutate(zero_scale)) == SCALE
    def short_alpha(ls): ls[0]["flat_alpha"] = ls[0]["flat_alpha"][:-1]
    assert _status(mutate(short_alpha)) == SHAPE
    def long_words(ls): ls[1]["packed_weights"] = np.concatenate([ls[1]["packed_weights"], np.zeros(1, np.uint32)])
    assert _status(mutate(long_words)) == SHAPE
    def bad_dims(ls): ls[0]["in_features"] = 0
    assert _status(mutate(bad_dims)) == FORMAT
    # a sensitivity flag of 2: patch the first layer's flag byte and re-seal the trailer
    body = bytearray(good[:-76]); body[12] = 2
    sealed = bytes(body) + struct.pack("<IQ", TRAILER_MAGIC, len(body)) + hashlib.sha256(bytes(body)).hexdigest().encode()
    assert _status(sealed) == FORMAT
    # codes in the unused tail of the last word are not weights: layer 1 has 7*33 = 231 weights, 15 words, 7 live fields
    def tail_bits(ls): w = ls[1]["packed_weights"].copy(); w[-1] |= 3 << 30; ls[1]["packed_weights"] = w
    assert _status(mutate(tail_bits)) == 0
    rec = capi.EdgeLayer()
    assert L.tbl_edge_pack_layer(good, len(good), 99, C.byref(rec)) == -1
    assert L.tbl_edge_pack_layer(good, len(good), 2, C.byref(rec)) == 0 and rec.sensitive == 1 and rec.weight_count == 80


def test_writer_refuses_what_would_not_load(tbl, port):
    from reimagined_b200 import capi, edge_pack
    layers = make_layers(port, seed=6)
    layers[0]["magnitude"] = layers[0]["magnitude"].copy()
    layers[0]["magnitude"][3] = np.inf
    with pytest.raises(capi.TernaryB200Error):
        edge_pack.dumps(layers)


def test_loading_a_pack_of_many_layers_hashes_it_once(tbl, port):
    """120 layers: one digest and one scan of the file, not one per layer."""
    import time
    from reimagined_b200 import edge_pack
    rng = np.random.default_rng(5)
    layers = []
    for i in range(120):
        n, k = 256, 512
        words = rng.integers(0, 3, (n * k,), dtype=np.uint32).reshape(-1, 16)
        packed = (words << (2 * np.arange(16, dtype=np.uint32))).sum(axis=1).astype(np.uint32)
        layers.append({"sensitive": False, "in_features": k, "out_features": n, "use_bias": False,
                       "weight_scale": np.float32(0.016), "packed_weights": packed, "magnitude": np.ones(n, np.float32),
                       "bias": np.zeros(0, np.float32), "flat_alpha": np.ones(k, np.float32),
                       "flat_beta": np.zeros(k, np.float32), "weight": None})
    image = edge_pack.dumps(layers)
    t0 = time.perf_counter()
    back = edge_pack.loads(image)
    one_pass = time.perf_counter() - t0
    t0 = time.perf_counter()
    edge_pack.sha256_hex(image)
    one_hash = time.perf_counter() - t0
    assert len(back) == 120 and np.array_equal(back[77]["packed_weights"], layers[77]["packed_weights"])
    assert one_pass < 6 * one_hash + 0.5, f"loading took {one_pass:.2f}s for a file that hashes in {one_hash:.2f}s"
    # the per-layer call still works and agrees
    rec = __import__("reimagined_b200.capi", fromlist=["EdgeLayer"]).EdgeLayer()
    assert tbl.tbl_edge_pack_layer(image, len(image), 119, C.byref(rec)) == 0 and rec.packed_words == 256 * 512 // 16
    assert tbl.tbl_edge_pack_layer(image, len(image), 120, C.byref(rec)) == -1

"""CPU-only checks of the product library: it loads, exports every declared symbol, its host-side
packer is bit-identical to the oracle and the golden vectors, and validation rejects bad calls
before anything is launched."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from conftest import ROOT, golden_cases, load_golden


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "ternary_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tbl_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(tbl):
    from reimagined_b200 import capi
    names = declared_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(tbl, n), f"{n} declared in include/ternary_b200.h but not exported"
    assert set(names) == set(capi.EXPORTED_SYMBOLS), "capi.py bindings out of sync with the header"
    assert tbl.tbl_abi_version() == 3
    assert tbl.tbl_status_string(0) == b"ok"


def host_pack(tbl, w):
    N, K = w.shape
    n = tbl.tbl_packed_words(N, K)
    words = np.zeros(n, np.uint32)
    scale = np.zeros(1, np.float32)
    rc = tbl.tbl_pack_weights(w.ctypes.data, N, K, words.ctypes.data, scale.ctypes.data)
    assert rc == 0
    return words, scale[0]


@pytest.mark.parametrize("path", [p for p in golden_cases() if "moe_" not in p],
                         ids=lambda p: p.split("/")[-1][:-4])
def test_host_packer_matches_golden(tbl, path):
    g = load_golden(path)
    words, scale = host_pack(tbl, np.ascontiguousarray(g["w"]))
    assert np.array_equal(words, g["words"])
    assert np.float32(scale).view(np.uint32) == np.float32(g["weight_scale"]).view(np.uint32)


@pytest.mark.parametrize("N,K", [(1, 16), (3, 5), (17, 33), (64, 768), (5, 1)])
def test_host_packer_matches_oracle_and_roundtrips(tbl, port, N, K):
    rng = np.random.default_rng(N * 1000 + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    words, scale = host_pack(tbl, w)
    owords, oscale, t, _ = port.pack_weights(w)
    assert np.array_equal(words, owords)
    assert np.float32(scale).view(np.uint32) == oscale.view(np.uint32)
    back = np.zeros((N, K), np.int8)
    assert tbl.tbl_unpack_weights_i8(words.ctypes.data, N, K, back.ctypes.data) == 0
    assert np.array_equal(back, t)
    assert set(np.unique(back)).issubset({-1, 0, 1})
    assert tbl.tbl_validate_packed(words.ctypes.data, words.size, N, K, float(scale), None, None) == 0


def test_packer_all_zero_and_constant(tbl, port):
    w = np.zeros((4, 16), np.float32)
    words, scale = host_pack(tbl, w)
    assert scale == np.float32(1e-8) and np.all(words == 0x55555555)  # every code is 1 (zero weight)
    w[:] = 0.3
    words, scale = host_pack(tbl, w)
    assert np.all(words == 0xAAAAAAAA)  # every weight rounds to +1
    assert np.array_equal(words, port.pack_weights(w)[0])


def test_validate_packed_rejects(tbl):
    from reimagined_b200 import capi as A
    C3 = -8
    words = np.full(4, 0x55555555, np.uint32)
    ok = lambda *a: tbl.tbl_validate_packed(*a)
    assert ok(words.ctypes.data, 4, 4, 16, 0.5, None, None) == 0
    assert ok(words.ctypes.data, 3, 4, 16, 0.5, None, None) == -2          # wrong word count
    assert ok(words.ctypes.data, 4, 4, 16, 0.0, None, None) == -4          # scale must be > 0
    assert ok(words.ctypes.data, 4, 4, 16, float("nan"), None, None) == -4
    bad = words.copy(); bad[2] |= 0x3 << 10
    assert ok(bad.ctypes.data, 4, 4, 16, 0.5, None, None) == C3            # reserved code 0b11
    mag = np.array([1, 2, np.inf, 4], np.float32)
    assert ok(words.ctypes.data, 4, 4, 16, 0.5, mag.ctypes.data, None) == -1
    assert ok(None, 4, 4, 16, 0.5, None, None) == -1


def test_device_entry_points_validate_before_launching(tbl):
    """Bad arguments are refused with a status and nothing is enqueued (no GPU needed).
    The non-null 'pointers' are dummies that validation never dereferences."""
    P = 0x1000  # 16-byte aligned dummy
    before = tbl.tbl_launch_count()
    lf = tbl.tbl_linear_forward
    assert lf(P, P, None, None, 0.5, 1, 24, 8, 8, 0, None, None, P, None, 0, None) == -2     # K % 16
    assert lf(P, P, None, None, 0.5, 0, 32, 8, 8, 0, None, None, P, None, 0, None) == -1     # M <= 0
    assert lf(P, P, None, None, -1.0, 1, 32, 8, 8, 0, None, None, P, None, 0, None) == -4    # scale
    assert lf(P, P, None, None, 0.5, 1, 32, 8, 9, 0, None, None, P, None, 0, None) == -5     # bits
    assert lf(P, P, None, None, 0.5, 1, 32, 8, 1, 0, None, None, P, None, 0, None) == -5
    assert lf(P, P, None, None, 0.5, 1, 8454672, 8, 8, 0, None, None, P, None, 0, None) == -3  # K > INT_MAX/254
    assert lf(P, P, None, None, 0.5, 65536, 32, 65536, 8, 0, None, None, P, None, 0, None) == -2  # M*N > INT_MAX
    assert lf(None, P, None, None, 0.5, 1, 32, 8, 8, 0, None, None, P, None, 0, None) == -1
    assert lf(P + 4, P, None, None, 0.5, 1, 32, 8, 8, 0, None, None, P, None, 0, None) == -6  # alignment
    assert lf(P, P, None, None, 0.5, 8, 32, 8, 8, 0, None, None, P, None, 0, None) == -7      # needs workspace
    assert tbl.tbl_gemv(P, P, P, None, 0.5, None, None, 65, 32, 8, P, None, None, 0, None) == -2  # M > 64
    assert tbl.tbl_quantize_rows(P, None, 1, 32, 8, 2, 0, P, P, None, None) == -1
    from reimagined_b200 import capi
    v = capi.LinearView(P, None, None, None, 32, 8, 8, 0, 0.5, None)   # fp32-weight view: not implemented
    arr = (capi.LinearView * 1)(v)
    assert tbl.tbl_grouped_forward(arr, 1, P, P, 8, 0, P, 1 << 20, None) == -10
    assert tbl.tbl_launch_count() == before
    assert tbl.tbl_linear_workspace_bytes(8, 1024, 64) >= 2 * 8 * 1024


def test_header_is_plain_c_and_links(tbl, tmp_path):
    """A C99 program built with gcc against the header and the shared library runs the host packer."""
    import subprocess
    from reimagined_b200 import capi
    exe = tmp_path / "abi_check"
    lib_dir = os.path.dirname(capi.LIB_PATH)
    subprocess.run(["/usr/bin/gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "abi_check.c"), "-o", str(exe),
                    "-L", lib_dir, "-lternary_b200", "-Wl,-rpath," + lib_dir, "-lm"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, f"abi_check exited {out.returncode}: {out.stdout} {out.stderr}"
    assert "abi ok" in out.stdout


def test_cpp_shim_maps_status_codes_to_the_reference_exceptions(tbl, tmp_path):
    """The header-only C++ shim compiles as C++17, links, and throws the reference's exception types."""
    import subprocess
    from reimagined_b200 import capi
    exe = tmp_path / "shim_check"
    lib_dir = os.path.dirname(capi.LIB_PATH)
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "shim_check.cpp"), "-o", str(exe),
                    "-L", lib_dir, "-lternary_b200", "-Wl,-rpath," + lib_dir], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0, f"shim_check exited {out.returncode}: {out.stdout} {out.stderr}"
    assert "shim ok" in out.stdout


def test_graft_entry_build_runs(tbl):
    """The build hook (extension + oracle checkers) completes and imports the package on a machine without a GPU."""
    import importlib
    entry = importlib.import_module("__graft_entry__")
    entry.build()


def test_new_entry_points_validate_before_touching_a_device(tbl):
    """Argument errors of the batched grouped call, the router and the pack reader come back as status codes
    on a machine without a GPU (nothing is enqueued)."""
    import ctypes as C
    from reimagined_b200 import capi
    view = capi.LinearView(None, 0x1000, None, None, 256, 16, 8, 0, 1.0, None, None)
    arr = (capi.LinearView * 1)(view)
    assert tbl.tbl_grouped_forward_rows(arr, 1, 0x1000, 65, 0x2000, 65 * 16, 0, 0x3000, 1 << 20, None) == -2   # rows > 64
    assert tbl.tbl_grouped_forward_rows(arr, 1, 0x1000, 4, 0x2000, 8, 0, 0x3000, 1 << 20, None) == -2         # stride too small
    assert tbl.tbl_grouped_forward_rows(arr, 0, 0x1000, 4, 0x2000, 64, 0, 0x3000, 1 << 20, None) == -1
    assert tbl.tbl_grouped_rows_workspace_bytes(5, 8, 768) >= 2 * 8 * 768
    assert tbl.tbl_router_topk(None, 4, 8, 2, 0x1000, None) == -1
    assert tbl.tbl_router_topk(0x1000, 4, 33, 2, 0x1000, None) == -1                                          # > TBL_MAX_GROUPS
    version, layers = C.c_int(0), C.c_int(0)
    assert tbl.tbl_edge_pack_open(b"DGE1", 4, C.byref(version), C.byref(layers)) == -11
    assert tbl.tbl_status_string(-11).decode().startswith("edge pack")
    assert tbl.tbl_status_string(-12).decode().startswith("edge pack")


def test_workspace_sizes_cover_the_plane_major_codes(tbl):
    """Mid-size batches keep a second copy of the codes with every row padded to 512 (the widening GEMM's layout):
    the workspace queries must account for the padding when K % 512 == 256, for the grouped call, the MoE block and
    the single layer alike (pure host arithmetic)."""
    for M, K in ((64, 768), (200, 1280), (33, 256), (64, 16384)):
        padded = (K + 511) // 512 * 512
        assert tbl.tbl_linear_workspace_bytes(M, K, 128) >= M * K + M * padded + 3 * 4 * M
    assert tbl.tbl_grouped_rows_workspace_bytes(5, 64, 768) >= 64 * 768 + 64 * 1024
    rows, D, Hd, E, top = 256, 768, 1280, 8, 2
    need = rows * top * (1024 + 1536) + 4 * rows * top * (Hd + D)      # both stages' codes + hidden + contributions
    assert tbl.tbl_moe_workspace_bytes(rows, D, Hd, E, top) >= need
    # sizes are monotonic in the row count
    assert tbl.tbl_linear_workspace_bytes(65, 768, 128) > tbl.tbl_linear_workspace_bytes(64, 768, 128)

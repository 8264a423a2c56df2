"""A C++ host on the GPU: tests/cpp/linear_gpu_check.cpp drives ternary_b200::TernaryLinear (transactional import,
forward, export, grouped view) with outputs of the reference's own BitLinear as the expected values; plus the
self-test of the bounded device-side waits."""
import os
import subprocess

import numpy as np
import pytest

from conftest import GOLDEN_DIR, ROOT, load_golden

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fixture", ["c1_exact_768", "mid_96x512_m24", "gemm_160x256_m130"])
def test_cpp_layer_object_on_the_gpu(cuda, tbl, tmp_path, fixture):
    from reimagined_b200 import capi
    g = load_golden(os.path.join(GOLDEN_DIR, fixture + ".npz"))
    N, K, M, exact = int(g["N"]), int(g["K"]), int(g["M"]), bool(g["exact_linear"])
    (tmp_path / "meta.txt").write_text(f"{N} {K} {M} {int(exact)}\n")
    for name in ("w", "x", "y") + (() if exact else ("magnitude", "bias")):
        np.ascontiguousarray(g[name], np.float32).tofile(tmp_path / f"{name}.bin")
    exe = tmp_path / "linear_gpu_check"
    lib_dir = os.path.dirname(capi.LIB_PATH)
    subprocess.run(["/usr/bin/g++", "-std=c++17", "-O1", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    "-I", "/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", "linear_gpu_check.cpp"), "-o", str(exe),
                    "-L", lib_dir, "-lternary_b200", "-Wl,-rpath," + lib_dir, "-L", "/usr/local/cuda/lib64", "-lcudart"],
                   check=True)
    out = subprocess.run([str(exe), str(tmp_path)], capture_output=True, text=True)
    assert out.returncode == 0, f"{out.stdout}\n{out.stderr}"
    assert "linear gpu ok" in out.stdout


def test_a_wait_that_nobody_answers_gives_up_and_reports(cuda, tbl):
    """The kernel returns by itself, says so, and the status word carries TBL_DEV_WAIT_TIMEOUT once."""
    import gpu_helpers as H
    torch = cuda
    assert H.device_status() == 0
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert tbl.tbl_selftest_bounded_wait(H.ptr(flag), H.stream_ptr()) == 0
    assert H.device_status() == 1           # TBL_DEV_WAIT_TIMEOUT
    assert int(flag.item()) == 1
    assert H.device_status() == 0           # read-and-clear; the context is still usable
    x = torch.ones(8, device="cuda")
    assert float(x.sum().item()) == 8.0

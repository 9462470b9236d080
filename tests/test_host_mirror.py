"""The C++ host mirror (oxicuda_b200/host/*.hpp): compiles and links against the C ABI on CPU; on a GPU the
driver program's INT8 per-row results are compared with the oracle bit for bit."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path):
    from oxicuda_b200 import _build
    _build.build()
    exe = str(tmp_path / "host_mirror_test")
    libdir = os.path.join(ROOT, "oxicuda_b200", "lib")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", "host_mirror_test.cpp"),
           "-o", exe, "-L" + libdir, "-loxq_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_host_config_types(tmp_path):
    """The configuration types' validate() rules (the reference's own tests restated in tests/cpp/host_config_test.cpp): host only."""
    from oxicuda_b200 import _build
    _build.build()
    exe = str(tmp_path / "host_config_test")
    libdir = os.path.join(ROOT, "oxicuda_b200", "lib")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", "host_config_test.cpp"),
           "-o", exe, "-L" + libdir, "-loxq_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, f"check {run.returncode} failed: {run.stdout} {run.stderr}"


def test_host_mirror_compiles_and_links(tmp_path):
    exe = _build(tmp_path)
    assert os.path.exists(exe)


@pytest.mark.gpu
def test_host_mirror_runs_and_matches_oracle(tmp_path, orc):
    exe = _build(tmp_path)
    out = str(tmp_path / "out.bin")
    res = subprocess.run([exe, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"rc={res.returncode} {res.stderr}"
    raw = np.fromfile(out, dtype=np.uint8)
    n = 64 * 256
    x = raw[:4 * n].view(np.float32).reshape(64, 256)
    scales = raw[4 * n:4 * n + 256].view(np.float32)
    codes = raw[4 * n + 256:4 * n + 256 + 4 * n].view(np.int32).reshape(64, 256)
    deq = raw[4 * n + 256 + 4 * n:].view(np.float32)
    q_ref, s_ref = orc.spec_int8_quant_rows(x, orc.ROUND_HALF_AWAY)
    assert np.array_equal(scales, s_ref) and np.array_equal(codes, q_ref.astype(np.int32))
    # the reference's own path gives the same codes (calibrate_2d + quantize_grouped)
    sr, zr = orc.ref_minmax_calibrate_2d(x, 64, 256)
    assert np.array_equal(orc.minmax_quantize_grouped(x, sr, zr, 256).reshape(64, 256), codes)
    t = np.array([0.0, 1.0, -1.0, 0.5, 0.0, 2.0, -2.0, 1.5], np.float32).reshape(2, 4)
    qt, st = orc.spec_int8_quant_rows(t, orc.ROUND_HALF_AWAY)
    assert np.array_equal(deq, orc.spec_int8_dequant_rows(qt, st).ravel())

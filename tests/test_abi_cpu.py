"""CPU-only checks of the drop-in boundary: the shared library builds, loads, and exports exactly the
symbols include/oxq.h declares; argument validation mirrors the reference's error variants."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from oxicuda_b200 import _build, _ffi
    _build.build()
    return _ffi.load()


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "oxq.h")).read()
    return sorted(set(re.findall(r"OXQ_API\s+[\w\s\*]+?\b(oxq_\w+)\s*\(", text)))


def test_header_symbols_all_exported(lib):
    from oxicuda_b200 import _ffi
    declared = _declared_symbols()
    assert len(declared) >= 27
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in oxq.h but not exported"
    assert sorted(_ffi.SIGNATURES) == declared          # the ctypes table covers the whole header


def test_every_entry_cites_the_reference_interface_it_replaces():
    """Each section of the header opens with a comment that names the reference source (a .rs path with line numbers) its
    entries stand behind; the handle utilities (version, status words, error strings) are the library's own."""
    text = open(os.path.join(ROOT, "include", "oxq.h")).read()
    own = {"oxq_version", "oxq_status_name", "oxq_last_error_string", "oxq_device_status"}
    section_cites, seen = False, 0
    for m in re.finditer(r"/\*.*?\*/|OXQ_API[^;]*;", text, re.S):
        tok = m.group(0)
        if tok.startswith("/*"):
            if tok.startswith("/* ----"):
                section_cites = False                     # a new section has to cite again
            if re.search(r"\w+\.rs:\d+", tok):
                section_cites = True
            continue
        decl = re.search(r"\b(oxq_\w+)\s*\(", tok)
        if decl is None:                                  # the macro's own definition
            continue
        name = decl.group(1)
        seen += 1
        assert section_cites or name in own, f"{name}: no reference file:line in its comment or its section's"
    assert seen == len(_declared_symbols())


def test_status_names(lib):
    assert lib.oxq_status_name(0) == b"Ok"
    assert lib.oxq_status_name(1) == b"EmptyInput"
    assert lib.oxq_status_name(2) == b"GroupSizeMismatch"
    assert lib.oxq_status_name(10) == b"InvalidDimension"
    assert lib.oxq_status_name(100) == b"DeviceTimeout"
    assert lib.oxq_status_name(1002) == b"Cuda"
    assert lib.oxq_version() >= 100


def test_size_queries(lib):
    assert lib.oxq_sf_mma_bytes(128, 4) == 512
    assert lib.oxq_sf_mma_bytes(129, 5) == 2 * 2 * 512
    assert lib.oxq_sf_mma_bytes(0, 4) == 0
    assert lib.oxq_gemm_w4a16_workspace_bytes(1, 4096, 4096) >= 4096 * 4 + 32 * 4
    assert lib.oxq_gemm_w4a16_workspace_bytes(0, 4096, 4096) == 0


def test_no_device_means_error_not_fallback(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    rc = lib.oxq_handle_create(0, None, C.byref(h))
    assert rc != 0 and not h                             # no device -> an error status, never a CPU path
    from oxicuda_b200 import ops
    with pytest.raises(RuntimeError):
        ops.Handle()


def test_error_mapping():
    from oxicuda_b200.errors import BlasError, QuantError, raise_for_status
    with pytest.raises(QuantError) as e:
        raise_for_status(2, "x")
    assert e.value.variant == "GroupSizeMismatch"
    with pytest.raises(BlasError) as e:
        raise_for_status(10)
    assert e.value.variant == "InvalidDimension"
    with pytest.raises(BlasError) as e:
        raise_for_status(1000 + 700)
    assert e.value.variant == "Cuda"
    raise_for_status(0)


def test_nf4_thresholds_match_the_reference_comparison():
    """The NF4 encoder counts decision thresholds below x instead of searching the level table.  Each threshold must be
    the largest f32 whose nearest level, under the reference's own f32 distance comparison (nf4.rs:186-205), is the
    lower neighbour: the value itself maps to level i, the next f32 up maps to level i + 1 (no GPU involved)."""
    import ctypes as C
    import numpy as np
    from oracle import oracle as orc
    from oxicuda_b200 import _ffi
    orc.build()
    near = orc.lib().orc_ref_nearest_nf4
    near.argtypes, near.restype = [C.c_float], C.c_int
    thr = np.zeros(15, np.float32)
    assert _ffi.load().oxq_nf4_thresholds(thr.ctypes.data_as(C.c_void_p)) == 0
    assert (np.diff(thr) > 0).all()
    for i, t in enumerate(thr):
        up = np.nextafter(t, np.float32(2.0), dtype=np.float32)
        assert near(float(t)) == i and near(float(up)) == i + 1, (i, float(t))
        # and a sweep of 64 ulps around it: the count of thresholds below x equals the reference's index
        v = t
        for _ in range(64):
            v = np.nextafter(v, np.float32(-2.0), dtype=np.float32)
        for _ in range(128):
            assert int((v > thr).sum()) == near(float(v)), float(v)
            v = np.nextafter(v, np.float32(2.0), dtype=np.float32)
    for v in (-2.0, -1.0, 0.0, 1.0, 2.0, float("nan")):
        assert int((np.float32(v) > thr).sum()) == near(v)


def test_package_exports_exist():
    """Everything the package lists in __all__ can be imported (ops and dist_infer load on first use)."""
    import importlib
    pkg = importlib.import_module("oxicuda_b200")
    for name in pkg.__all__:
        assert getattr(pkg, name).__name__ == "oxicuda_b200." + name
    with pytest.raises(AttributeError):
        pkg.no_such_module


def test_integration_stubs_match_the_header():
    """Every `pub fn oxq_*` line of the binding shown in INTEGRATION.md names a declared entry and has its number of arguments."""
    hdr = open(os.path.join(ROOT, "include", "oxq.h")).read()
    decl = {}
    for m in re.finditer(r"OXQ_API\s+[\w\s\*]+?\b(oxq_\w+)\s*\(([^;]*)\);", hdr, re.S):
        args = [a.strip() for a in re.sub(r"\s+", " ", m.group(2)).split(",")]
        decl[m.group(1)] = 0 if args == ["void"] else len(args)
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    stubs = re.findall(r"pub fn (oxq_\w+)\(([^;]*)\)\s*->", text, re.S)
    assert len(stubs) >= 20
    for name, args in stubs:
        assert name in decl, f"{name} is not declared in oxq.h"
        n = len([a for a in re.sub(r"\s+", " ", args).split(",") if a.strip()])
        assert n == decl[name], f"{name}: {n} arguments in INTEGRATION.md, {decl[name]} in oxq.h"


def test_fp4_block_quantizer_host_helper(orc):  # crates/oxicuda-dnn/src/quantize/block_scale.rs:475-610
    from oxicuda_b200 import ops
    from oxicuda_b200.errors import DnnError
    assert ops.Fp4BlockQuantizer.MAX_VALUE == 6.0 and ops.Fp4BlockQuantizer.REQUIRED_BLOCK_SIZE == 32
    for bad in (16, 64):
        with pytest.raises(DnnError) as e:
            ops.Fp4BlockQuantizer(bad)
        assert e.value.variant == "InvalidArgument"
    q = ops.Fp4BlockQuantizer(32)
    assert q.block_size == 32 and [q.num_scales(n) for n in (32, 96, 33, 0)] == [1, 3, 2, 0]
    assert q.compute_scale([0.0] * 32) == 1.0 and abs(q.compute_scale([6.0] * 32) - 1.0) < 1e-6 and abs(q.compute_scale([12.0] * 32) - 2.0) < 1e-6
    assert abs(q.compute_scale([-6.0, 3.0, 1.5] + [0.0] * 29) - 1.0) < 1e-6
    block = orc.gaussian((1, 32), 3.0, 5).ravel()
    assert q.compute_scale(block) == orc.ref_fp4_block_compute_scale(block)            # the oracle's restatement of the same lines

"""The allocation-free W4A16 entry point, called through the C ABI.

Some callers of this library are not allowed to allocate device memory: they run inside another
framework's memory plan, or in a plugin that must not call cudaMalloc after start-up, so they can
neither create a handle nor hand over a workspace.  oxq_gemm_w4a16_static serves them from a scratch
array built into the library.  This test drives it with nothing but a stream and the operand
pointers, twice in a row (the second call finds the first call's leftovers in the shared array and
must clear them itself), and compares each result with the regular entry point's on the same inputs
and with the CPU oracle's product of the dequantised codes, with the GEMM tolerance of the other tests
(max-relative 1e-2 on bf16 outputs).

This file sorts last on purpose: if it fails under `pytest -x`, every other test has already run.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
MAX_REL = 1e-2


def _call_static(lib, x, codes, scales, zeros, y, group=128):
    m, k = x.shape
    n = codes.shape[0]
    stream = torch.cuda.current_stream().cuda_stream
    return lib.oxq_gemm_w4a16_static(C.c_void_p(stream), m, n, k, C.c_void_p(x.data_ptr()), C.c_void_p(codes.data_ptr()),
                                     C.c_void_p(scales.data_ptr()), C.c_void_p(zeros.data_ptr()), group,
                                     C.c_void_p(y.data_ptr()))


def test_static_entry_matches_regular_entry_twice():
    from oracle import oracle as orc
    from oxicuda_b200 import _ffi, ops
    lib = _ffi.load()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(5)
    for (m, n, k) in ((8, 4096, 4096), (32, 1024, 2048)):
        w = torch.randn((n, k), generator=g, device="cuda") * 0.02
        codes, scales, zeros = ops.int4g_quant_pack(w, 128)
        x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
        want = ops.gemm_w4a16(x, codes, scales, zeros, 128).float()
        scale = float(want.abs().max())
        # the regular entry point's result is itself what the CPU oracle gives for these codes (dequantise, then f64 product)
        deq = orc.spec_int4g_dequant(codes.cpu().numpy().view(np.uint32), scales.view(torch.int16).cpu().numpy().view(np.uint16),
                                     zeros.cpu().numpy().view(np.uint32), n, k, 128).astype(np.float64)
        oracle_y = torch.from_numpy((x.float().cpu().numpy().astype(np.float64) @ deq.T).astype(np.float32)).cuda()
        assert float((want - oracle_y).abs().max()) <= MAX_REL * float(oracle_y.abs().max())
        for call in range(2):
            y = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
            assert _call_static(lib, x, codes, scales, zeros, y) == 0
            torch.cuda.synchronize()
            got = y.float()
            assert bool(torch.isfinite(got).all()), f"call {call}: unwritten or non-finite outputs"
            assert float((got - want).abs().max()) <= MAX_REL * scale, f"call {call} shape {(m, n, k)}"
            assert float((got - oracle_y).abs().max()) <= MAX_REL * float(oracle_y.abs().max()), f"call {call} against the oracle"
        # a different, smaller problem right after: stale sums from the larger one must not leak in
        y2 = torch.empty((1, n), dtype=torch.bfloat16, device="cuda")
        assert _call_static(lib, x[:1].contiguous(), codes, scales, zeros, y2) == 0
        torch.cuda.synchronize()
        assert float((y2.float() - want[:1]).abs().max()) <= MAX_REL * scale


def test_static_entry_rejects_shapes_beyond_its_scratch():
    from oxicuda_b200 import _ffi
    lib = _ffi.load()
    torch.cuda.set_device(0)
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    p = C.c_void_p(dummy.data_ptr())
    # 32 x 16512 outputs > 524288: refused before anything is launched
    assert lib.oxq_gemm_w4a16_static(None, 32, 16512, 4096, p, p, p, p, 128, p) == 11     # OXQ_ERR_BUFFER_TOO_SMALL
    assert lib.oxq_gemm_w4a16_static(None, 33, 128, 4096, p, p, p, p, 128, p) == 13        # m > 32: UnsupportedOperation
    assert lib.oxq_gemm_w4a16_static(None, 0, 128, 4096, p, p, p, p, 128, p) == 10         # zero dimension

"""GPU parity of the quantize / dequantize kernels, through the C ABI, against the CPU oracle and the
committed golden vectors.  Integer codes, packed nibbles and E8M0 / E4M3 scale bytes must be
bit-exact; f32 / f16 scales within 1 ulp (they come out identical in practice)."""
import os

import numpy as np
import pytest
import torch

from tests.gpu_util import bf16_bits, bf16_dev, sf_to_mma_layout, to_dev, u16, u32, ulp_diff_f32

pytestmark = pytest.mark.gpu
G = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_golden.npz"))


@pytest.fixture(scope="module")
def ops():
    from oxicuda_b200 import ops
    return ops


# ------------------------------------------------------------------------------------------- INT8

@pytest.mark.parametrize("shape", [(64, 4096), (7, 1000), (5, 333), (3, 8196), (2, 20480), (1, 4)])
@pytest.mark.parametrize("rounding", [0, 1])
def test_int8_quant_rows_bit_exact(ops, orc, shape, rounding):
    x = orc.gaussian(shape, 0.02, 0)
    x[0, 0] = 0.0
    if shape[1] > 8:
        x[-1, 1] = np.nan                                # NaN -> code 0, skipped by the absmax scan
    q_ref, s_ref = orc.spec_int8_quant_rows(x, rounding)
    q, s = ops.int8_quant_rows(to_dev(x), rounding)
    assert ulp_diff_f32(s.cpu().numpy(), s_ref) <= 1
    assert np.array_equal(s.cpu().numpy(), s_ref)
    assert np.array_equal(q.cpu().numpy(), q_ref)
    y = ops.int8_dequant_rows(q, s).cpu().numpy()
    assert np.array_equal(y, orc.spec_int8_dequant_rows(q_ref, s_ref))
    # the same codes come out of the literal reference path (calibrate_2d + quantize_grouped)
    if not np.isnan(x).any():
        sr, zr = orc.ref_minmax_calibrate_2d(x, *shape)
        qr = orc.minmax_quantize_grouped(x, sr, zr, shape[1], 8, orc.SYMMETRIC, rounding, False)
        assert np.array_equal(qr.reshape(shape), q.cpu().numpy().astype(np.int32))


def test_int8_golden(ops):
    for name, r in (("even", 0), ("away", 1)):
        q, s = ops.int8_quant_rows(to_dev(G["int8_x"]), r)
        assert np.array_equal(q.cpu().numpy(), G[f"int8_q_{name}"])
        assert np.array_equal(s.cpu().numpy(), G["int8_scales"])


def test_int8_edge_cases(ops, orc):
    from oxicuda_b200.errors import QuantError
    x = np.zeros((4, 64), np.float32)                    # all-zero rows: scale = 1e-8/127, codes 0
    q, s = ops.int8_quant_rows(to_dev(x))
    assert (q.cpu().numpy() == 0).all() and np.array_equal(s.cpu().numpy(), orc.spec_int8_quant_rows(x)[1])
    x = orc.gaussian((4, 64), 1.0, 3)
    x[1, 5] = np.inf                                     # Inf -> non-finite scale, reported by the host layer
    _, s = ops.int8_quant_rows(to_dev(x))
    assert not np.isfinite(s.cpu().numpy()[1])
    with pytest.raises(QuantError) as e:                 # calibrate_2d: rows == 0 -> EmptyInput
        ops.int8_quant_rows(torch.empty((0, 16), dtype=torch.float32, device="cuda"))
    assert e.value.variant == "EmptyInput"
    with pytest.raises(QuantError) as e:                 # cols == 0 -> DimensionMismatch
        ops.int8_quant_rows(torch.empty((4, 0), dtype=torch.float32, device="cuda"))
    assert e.value.variant == "DimensionMismatch"


def test_int8_run_twice_identical(ops, orc):
    x = to_dev(orc.gaussian((256, 4096), 0.02, 11))
    a = ops.int8_quant_rows(x)
    b = ops.int8_quant_rows(x)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


# ------------------------------------------------------------------------------------------- FP8

@pytest.mark.parametrize("n", [64 * 256, 16, 1000003, 17, 8192 * 4096 + 5])       # the last one takes the single-launch path (>= 48 MB)
@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_fp8_dynamic_bit_exact(ops, orc, n, dtype):
    x = orc.gaussian(n, 1.0, 0)
    if dtype == "bf16":
        xb = orc.f32_to_bf16_bits(x)
        xd, xo = bf16_dev(xb), xb
    else:
        xd, xo = to_dev(x), x
    am = orc.spec_absmax(xo)
    sc = orc.spec_fp8_scale(am)
    q, stats = ops.fp8_quant_dynamic(xd)
    st = stats.cpu().numpy()
    assert st[0] == np.float32(am)
    assert ulp_diff_f32(st[1:2], np.array([sc], np.float32)) <= 1 and st[1] == sc
    q_ref = orc.spec_fp8_quant(xo, float(sc))
    assert np.array_equal(q.cpu().numpy(), q_ref)
    deq = ops.fp8_dequant(q, stats[1:]).cpu().numpy()
    assert np.array_equal(deq, orc.spec_fp8_dequant(q_ref, float(sc)))
    am2 = ops.absmax(xd).cpu().numpy()[0]
    assert am2 == np.float32(am)
    q2, stats2 = ops.fp8_quant_dynamic(xd)                       # the reduction cells are back to zero: a second call agrees
    assert torch.equal(q, q2) and torch.equal(stats, stats2)
    assert ops.handle().device_status() == 0


def test_fp8_golden_and_special_values(ops, orc):
    q, stats = ops.fp8_quant_dynamic(bf16_dev(G["fp8_x_bf16"]))
    assert stats.cpu().numpy()[0] == G["fp8_absmax"] and stats.cpu().numpy()[1] == G["fp8_scale"]
    assert np.array_equal(q.cpu().numpy(), G["fp8_q"])
    # ties, subnormals, saturation, signed zero with scale 1
    x = np.array([0.0, -0.0, 448.0, 449.0, 464.0, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10, 3 * 2.0 ** -10,
                  1.0625, 1.1875, 1.3125, -17.0, 0.0009765], np.float32)
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    q = ops.fp8_quant(to_dev(x), one).cpu().numpy()
    assert np.array_equal(q, orc.e4m3_rne_sat(x))
    z = ops.fp8_quant_dynamic(torch.zeros(64, dtype=torch.bfloat16, device="cuda"))
    assert (z[0].cpu().numpy() == 0).all() and z[1].cpu().numpy()[1] == 1.0


def test_fp8_refcompat_matches_literal_codec(ops, orc):
    """The test-only REFCOMPAT mode reproduces Fp8Codec (truncation, >=256 -> 448, subnormal shift) bit for bit."""
    one = torch.ones(1, dtype=torch.float32, device="cuda")
    x = G["fp8_codec_x"]
    q = ops.fp8_quant(to_dev(x), one, mode=ops.FP8_REFCOMPAT).cpu().numpy()
    assert np.array_equal(q, G["fp8_codec_ref"])
    assert np.array_equal(q, orc.ref_fp8_encode(x))
    allb = torch.arange(256, dtype=torch.int32, device="cuda").to(torch.uint8)
    d = ops.fp8_dequant(allb, one, mode=ops.FP8_REFCOMPAT).cpu().numpy()
    assert np.array_equal(d, G["fp8_codec_ref_decoded"], equal_nan=True)
    d2 = ops.fp8_dequant(allb, one).cpu().numpy()
    assert np.array_equal(d2, orc.e4m3_to_f32(np.arange(256, dtype=np.uint8)), equal_nan=True)
    # how far the literal codec is from RNE on the same data (reported, not gated)
    q_rne = ops.fp8_quant(to_dev(x), one).cpu().numpy()
    assert 0.2 < float((q != q_rne).mean()) < 0.8


# ------------------------------------------------------------------------------------------- INT4

@pytest.mark.parametrize("group", [32, 64, 128, 256])
@pytest.mark.parametrize("shape", [(9, 768), (64, 4096), (1, 256)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_int4g_bit_exact(ops, orc, group, shape, dtype):
    x = orc.gaussian(shape, 0.02, 3)
    if dtype == "bf16":
        xb = orc.f32_to_bf16_bits(x)
        x = orc.bf16_bits_to_f32(xb)
        xd = bf16_dev(xb)
    else:
        xd = to_dev(x)
    for rounding in (0, 1):
        c_ref, s_ref, z_ref = orc.spec_int4g_quant(x, group, rounding)
        c, s, z = ops.int4g_quant_pack(xd, group, rounding)
        assert np.array_equal(u16(s), s_ref)
        assert np.array_equal(u32(z), z_ref)
        assert np.array_equal(u32(c), c_ref)
    y = ops.int4g_dequant(c, s, z, shape[0], shape[1], group).cpu().numpy()
    assert np.array_equal(y, orc.spec_int4g_dequant(c_ref, s_ref, z_ref, shape[0], shape[1], group))
    yb = ops.int4g_dequant(c, s, z, shape[0], shape[1], group, dtype=torch.bfloat16)
    assert np.array_equal(bf16_bits(yb), orc.f32_to_bf16_bits(y))


def test_int4g_golden_and_errors(ops):
    from oxicuda_b200.errors import BlasError, QuantError
    for grp in (32, 64, 128, 256):
        c, s, z = ops.int4g_quant_pack(to_dev(G["int4_x"]), grp)
        assert np.array_equal(u32(c), G[f"int4_codes_g{grp}"])
        assert np.array_equal(u16(s), G[f"int4_scales_g{grp}"])
        assert np.array_equal(u32(z), G[f"int4_zeros_g{grp}"])
    with pytest.raises(QuantError) as e:                 # GroupSizeMismatch, minmax.rs:147-152
        ops.int4g_quant_pack(to_dev(np.ones((2, 192), np.float32)), 128)
    assert e.value.variant == "GroupSizeMismatch"
    with pytest.raises(BlasError):                       # VALID_GROUP_SIZES, int_ops.rs:250-281
        ops.int4g_quant_pack(to_dev(np.ones((2, 192), np.float32)), 48)
    # constant group: range clamps to 1e-8, codes = zp
    c, s, z = ops.int4g_quant_pack(to_dev(np.full((1, 128), 0.5, np.float32)), 128)
    assert u16(s)[0, 0] != 0


# ------------------------------------------------------------------------------------------- block scaled

@pytest.mark.parametrize("shape", [(16, 256), (128, 512), (130, 1024 + 32), (4, 32)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_mxfp8_bit_exact(ops, orc, shape, dtype):
    x = orc.gaussian(shape, 1.0, 5)
    x[0, :32] = 0.0
    if shape[1] >= 128:
        x[1, 32:64] *= np.float32(1e-20)
        x[2, 64:96] *= np.float32(1e20)
    if dtype == "bf16":
        xb = orc.f32_to_bf16_bits(x)
        x = orc.bf16_bits_to_f32(xb)
        xd = bf16_dev(xb)
    else:
        xd = to_dev(x)
    c_ref, sf_ref = orc.spec_mxfp8_quant(x)
    c, sf, sf_mma = ops.mxfp8_quant(xd)
    assert np.array_equal(sf.cpu().numpy(), sf_ref)      # E8M0 exponents bit-exact
    assert np.array_equal(c.cpu().numpy(), c_ref)
    assert np.array_equal(sf_mma.cpu().numpy(), sf_to_mma_layout(sf_ref))
    y = ops.mxfp8_dequant(c, sf).cpu().numpy()
    assert np.array_equal(y, orc.spec_mxfp8_dequant(c_ref, sf_ref))


@pytest.mark.parametrize("shape", [(16, 256), (128, 512), (130, 1024 + 16), (4, 16)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_nvfp4_bit_exact(ops, orc, shape, dtype):
    x = orc.gaussian(shape, 1.0, 7)
    x[0, :16] = 0.0
    if shape[1] >= 64:
        x[1, 16:32] *= np.float32(1e-6)
    if dtype == "bf16":
        xb = orc.f32_to_bf16_bits(x)
        x = orc.bf16_bits_to_f32(xb)
        xd = bf16_dev(xb)
    else:
        xd = to_dev(x)
    g = orc.spec_nvfp4_global_scale(orc.spec_absmax(x))
    p_ref, sf_ref = orc.spec_nvfp4_quant(x, float(g))
    p, sf, sf_mma, stats = ops.nvfp4_quant(xd)
    assert stats.cpu().numpy()[1] == g
    assert np.array_equal(sf.cpu().numpy(), sf_ref)
    assert np.array_equal(p.cpu().numpy(), p_ref)
    assert np.array_equal(sf_mma.cpu().numpy(), sf_to_mma_layout(sf_ref))
    y = ops.nvfp4_dequant(p, sf, stats).cpu().numpy()
    assert np.array_equal(y, orc.spec_nvfp4_dequant(p_ref, sf_ref, float(g), *shape))


def test_block_scaled_golden(ops):
    c, sf, _ = ops.mxfp8_quant(to_dev(G["mx_x"]))
    assert np.array_equal(c.cpu().numpy(), G["mx_codes"]) and np.array_equal(sf.cpu().numpy(), G["mx_sf"])
    p, sf, _, st = ops.nvfp4_quant(to_dev(G["nv_x"]))
    assert st.cpu().numpy()[1] == G["nv_g"]
    assert np.array_equal(p.cpu().numpy(), G["nv_packed"]) and np.array_equal(sf.cpu().numpy(), G["nv_sf"])


# ------------------------------------------------------------------------------------------- full size

def test_full_size_config1_and_2_properties(ops, orc):
    """Benchmark sizes: config 1 (4096x4096 f32 -> INT8) compared with the oracle in full (the oracle
    finishes in well under a second with OpenMP); config 2 (8192x8192 bf16 -> E4M3) through properties:
    decode(encode(x)) is within half an E4M3 step of x/scale and re-encoding the decoded tensor is
    the identity (idempotence)."""
    w = orc.gaussian((4096, 4096), 0.02, 0)
    q, s = ops.int8_quant_rows(to_dev(w))
    q_ref, s_ref = orc.spec_int8_quant_rows(w)
    assert np.array_equal(s.cpu().numpy(), s_ref) and np.array_equal(q.cpu().numpy(), q_ref)
    gen = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((8192, 8192), generator=gen, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    qa, st = ops.fp8_quant_dynamic(a)
    assert float(st[0]) == float(a.float().abs().max())
    deq = ops.fp8_dequant(qa, st[1:])                     # f32
    err = (deq - a.float()).abs()
    step = torch.clamp(a.float().abs(), min=float(st[1]) * 2.0 ** -6) * (2.0 ** -4)   # half ulp of a 3-bit mantissa
    assert bool((err <= step * 1.0001 + float(st[1]) * 2.0 ** -10).all())
    q2 = ops.fp8_quant(deq, st[1:])
    assert torch.equal(q2, qa)
    # a 1M-element slice against the oracle, bit for bit
    sl = bf16_bits(a[:128])
    assert np.array_equal(qa[:128].cpu().numpy(), orc.spec_fp8_quant(sl, float(st[1])))

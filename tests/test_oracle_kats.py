"""Pins the CPU oracle against the known-answer tests the reference carries for this path.

Every case cites the reference test it restates (paths relative to the reference workspace).
"""
import math

import numpy as np
import pytest


# ---- crates/oxicuda-quant/src/scheme/minmax.rs tests -------------------------------------------

def test_symmetric_calibrate_scale(orc):  # minmax.rs:341-349
    s, z = orc.ref_minmax_calibrate([-2.0, -1.0, 0.5, 2.0], 8, orc.SYMMETRIC)
    assert abs(s[0] - 2.0 / 127.0) < 1e-6 and z[0] == 0
    assert s[0] == np.float32(2.0) / np.float32(127.0)


def test_asymmetric_calibrate_scale_zp(orc):  # minmax.rs:351-360
    s, z = orc.ref_minmax_calibrate([0.0, 1.0, 2.0, 3.0], 8, orc.ASYMMETRIC)
    assert abs(s[0] - 3.0 / 255.0) < 1e-5 and z[0] == 0


def test_per_group_calibrate(orc):  # minmax.rs:362-368 (int4_per_group(4) is 4-bit symmetric)
    s, z = orc.ref_minmax_calibrate([-1.0, 0.0, 0.5, 1.0, -2.0, 0.0, 1.0, 2.0], 4, orc.SYMMETRIC, group=4)
    assert len(s) == 2
    assert s[0] == np.float32(1.0) / np.float32(7.0) and s[1] == np.float32(2.0) / np.float32(7.0)


def test_symmetric_round_trip_low_error(orc):  # minmax.rs:370-385
    t = np.array([(i / 127.0) * 2.0 - 1.0 for i in range(128)], np.float32)
    s, z = orc.ref_minmax_calibrate(t, 8, orc.SYMMETRIC)
    codes = orc.minmax_quantize_grouped(t, s, z, t.size, 8, orc.SYMMETRIC)
    deq = orc.ref_minmax_dequantize_grouped(codes, s, z, t.size)
    assert np.abs(t - deq).max() < 0.02


def test_grouped_round_trip(orc):  # minmax.rs:387-402
    t = np.array([i * 0.1 for i in range(64)], np.float32)
    s, z = orc.ref_minmax_calibrate(t, 4, orc.SYMMETRIC, group=16)
    codes = orc.minmax_quantize_grouped(t, s, z, 16, 4, orc.SYMMETRIC)
    deq = orc.ref_minmax_dequantize_grouped(codes, s, z, 16)
    assert np.abs(t - deq).max() < 0.5


def test_empty_input_error(orc):  # minmax.rs:404-408
    with pytest.raises(orc.OracleError) as e:
        orc.ref_minmax_calibrate(np.zeros(0, np.float32))
    assert e.value.name == "EmptyInput"


def test_group_size_mismatch_error(orc):  # minmax.rs:410-418
    with pytest.raises(orc.OracleError) as e:
        orc.ref_minmax_calibrate(np.ones(10, np.float32), 4, orc.SYMMETRIC, group=3)
    assert e.value.name == "GroupSizeMismatch"


def test_q_range_int8(orc):  # minmax.rs:420-426: q_max 127, q_min -128 on the reference path
    s = np.array([1.0], np.float32)
    z = np.array([0], np.int32)
    codes = orc.minmax_quantize_grouped([1e9, -1e9], s, z, 2, 8, orc.SYMMETRIC)
    assert list(codes) == [127, -128]
    codes = orc.minmax_quantize_grouped([1e9, -1e9], s, z, 2, 8, orc.SYMMETRIC, orc.ROUND_HALF_EVEN, True)
    assert list(codes) == [127, -127]


def test_calibrate_2d_per_row(orc):  # minmax.rs:428-439
    t = [0.0, 1.0, -1.0, 0.5, 0.0, 2.0, -2.0, 1.5]
    s, z = orc.ref_minmax_calibrate_2d(t, 2, 4)
    assert len(s) == 2 and s[1] > s[0]
    with pytest.raises(orc.OracleError):
        orc.ref_minmax_calibrate_2d(t, 0, 4)
    with pytest.raises(orc.OracleError) as e:
        orc.ref_minmax_calibrate_2d(t, 2, 0)
    assert e.value.name == "DimensionMismatch"


def test_rounding_modes_and_nonfinite(orc):
    s = np.array([1.0], np.float32)
    z = np.array([0], np.int32)
    x = [0.5, 1.5, 2.5, -0.5, -2.5, float("nan"), float("inf"), float("-inf")]
    away = orc.minmax_quantize_grouped(x, s, z, len(x), 8, orc.SYMMETRIC, orc.ROUND_HALF_AWAY)
    even = orc.minmax_quantize_grouped(x, s, z, len(x), 8, orc.SYMMETRIC, orc.ROUND_HALF_EVEN)
    assert list(away) == [1, 2, 3, -1, -3, 0, 127, -128]    # Rust f32::round; NaN as i32 == 0
    assert list(even) == [0, 2, 2, 0, -2, 0, 127, -128]
    with pytest.raises(orc.OracleError) as e:                # Inf in calibration -> InvalidScale (minmax.rs:234-236)
        orc.ref_minmax_calibrate([1.0, float("inf")])
    assert e.value.name == "InvalidScale"
    sc, zp = orc.ref_minmax_calibrate(np.zeros(8, np.float32))
    assert sc[0] == np.float32(1e-8) / np.float32(127.0)


# ---- crates/oxicuda-quant/src/scheme/fp8.rs tests ----------------------------------------------

def test_e4m3_zero_encodes_to_zero(orc):  # fp8.rs:287-292
    assert list(orc.ref_fp8_encode([0.0, -0.0])) == [0x00, 0x80]


def test_e4m3_round_trip_basic(orc):  # fp8.rs:294-303
    v = np.array([1.0, -1.0, 2.0, 0.5, 0.25, -0.25], np.float32)
    dec = orc.ref_fp8_decode(orc.ref_fp8_encode(v))
    assert (np.abs(v - dec) / np.abs(v) < 0.15).all()


def test_e5m2_round_trip_basic(orc):  # fp8.rs:305-314
    v = np.array([1.0, -1.0, 4.0, 16.0, -8.0], np.float32)
    dec = orc.ref_fp8_decode(orc.ref_fp8_encode(v, e5m2=True), e5m2=True)
    assert (np.abs(v - dec) / np.abs(v) < 0.25).all()


def test_e4m3_saturates_large_values(orc):  # fp8.rs:316-324
    dec = orc.ref_fp8_decode(orc.ref_fp8_encode([1000.0]))
    assert 0.0 < dec[0] <= 449.0


def test_nan_input_errors(orc):  # fp8.rs:326-340
    for bad in (float("nan"), float("inf")):
        with pytest.raises(orc.OracleError) as e:
            orc.ref_fp8_encode([bad])
        assert e.value.name == "NonFiniteFp8"


def test_mse_within_tolerance(orc):  # fp8.rs:342-348
    d = np.array([(i / 128.0) - 1.0 for i in range(256)], np.float32)
    dec = orc.ref_fp8_decode(orc.ref_fp8_encode(d))
    assert float(((d - dec) ** 2).sum() / d.size) < 0.01


def test_ref_fp8_literal_quirks(orc):
    """Behaviour of the literal restatement that the reference tests leave unpinned (fp8.rs:163-261):
    truncation, |v| >= 256 -> 448, subnormal shift, subnormal decode."""
    enc = orc.ref_fp8_encode([1.9375, 256.0, 2.0 ** -7, 1.0])
    assert list(enc) == [0x3F, 0x7E, 0x02, 0x38]            # 0x38 = E4M3 one (blas types.rs:355-357)
    assert orc.ref_fp8_decode([0x3F])[0] == 1.875
    assert orc.ref_fp8_decode([0x02])[0] == np.float32(2.0 ** -6 * 1.25)
    assert orc.ref_fp8_encode([1.0], e5m2=True)[0] == 0x3C  # E5M2 one (blas types.rs:383-385)
    assert math.isnan(orc.ref_fp8_decode([0x7F])[0])


# ---- crates/oxicuda-blas/src/precision/int_ops.rs tests ----------------------------------------

def test_pack_unpack_int4_roundtrip(orc):  # int_ops.rs:1008-1017
    v = [0, 1, -1, 7, -8, 3, -5, 2]
    p = orc.ref_pack_int4(v)
    assert p.size == 1 and list(orc.ref_unpack_int4(p)) == v


def test_pack_int4_errors(orc):  # int_ops.rs:1019-1029
    with pytest.raises(orc.OracleError):
        orc.ref_pack_int4([0, 1, 2])
    with pytest.raises(orc.OracleError):
        orc.ref_pack_int4([0, 1, 2, 3, 4, 5, 6, 10])


def test_unpack_int4_patterns(orc):  # int_ops.rs:1031-1052
    assert list(orc.ref_unpack_int4([0x00000000])) == [0] * 8
    assert list(orc.ref_unpack_int4([0xFFFFFFFF])) == [-1] * 8
    assert list(orc.ref_unpack_int4([0x87878787])) == [7, -8] * 4
    assert list(orc.unpack_uint4([0x87878787])) == [7, 8] * 4
    v = np.arange(16, dtype=np.uint8)
    assert list(orc.unpack_uint4(orc.pack_uint4(v))) == list(v)


# ---- crates/oxicuda-blas/src/precision/fp4_fp6_ops.rs tests ------------------------------------

def test_fp4_e2m1_roundtrip_accuracy(orc):  # fp4_fp6_ops.rs:1681-1697
    for v in [0.0, 1.0, -1.0, 2.0, -2.0, 4.0, -4.0, 6.0]:
        rec = orc.e2m1_to_f32(np.array([orc.ref_e2m1_quantize_one(v)], np.uint8))[0]
        assert abs(v - rec) <= abs(v) * 0.6 + 0.01


def test_ref_e2m1_floor_map(orc):
    """The reference encoder's value map (fp4_fp6_ops.rs:645-661), by interval."""
    table = [(0.3, 0.0), (0.74, 0.0), (0.75, 0.5), (0.99, 0.5), (1.0, 1.0), (1.49, 1.0), (1.5, 1.5), (1.99, 1.5),
             (2.0, 2.0), (2.99, 2.0), (3.0, 3.0), (3.99, 3.0), (4.0, 4.0), (5.99, 4.0), (6.0, 6.0), (100.0, 6.0)]
    for v, want in table:
        got = orc.e2m1_to_f32(np.array([orc.ref_e2m1_quantize_one(v)], np.uint8))[0]
        assert got == want, (v, got, want)
    assert orc.ref_e2m1_quantize_one(-0.1) == 0x8
    assert orc.ref_e2m1_quantize_one(-0.0) == 0x0


def test_micro_scaling_fp4_roundtrip(orc):  # fp4_fp6_ops.rs micro_scaling tests: block scale = absmax/6
    x = np.array([i * 0.25 - 4.0 for i in range(64)], np.float32)
    packed, scales = orc.ref_microscale_fp4(x, 32)
    assert scales[0] == np.float32(np.abs(x[:32]).max()) / np.float32(6.0)
    rec = orc.ref_microscale_fp4_dequant(packed, scales, x.size, 32)
    assert np.abs(x - rec).max() <= np.abs(x).max() * 0.35
    with pytest.raises(orc.OracleError):
        orc.ref_microscale_fp4(x, 16)                      # block_size must be 32/64/128 (fp4_fp6_ops.rs:202-214)
    _, s0 = orc.ref_microscale_fp4(np.zeros(32, np.float32), 32)
    assert s0[0] == 1.0                                    # all-zero block -> scale 1.0 (:773-777)


# ---- adjacent scale KATs -----------------------------------------------------------------------

def test_int8_block_dequant_kat(orc):  # crates/oxicuda-dnn/src/quantize/int8_quantize.rs:619-639
    y = orc.spec_int8_dequant_rows(np.array([[-128, 0, 127]], np.int8), np.array([0.1], np.float32))
    assert np.allclose(y[0], [-12.8, 0.0, 12.7], atol=1e-5)


# ---- tensor-parallel definition ----------------------------------------------------------------

def test_tp_column_then_row_matches_unsharded(orc):  # crates/oxicuda-dist-infer/src/lib.rs:120 (tp=4 e2e)
    rng = np.random.default_rng(0)
    x = rng.standard_normal((3, 8)).astype(np.float32)
    wg = rng.standard_normal((16, 8)).astype(np.float32)
    wu = rng.standard_normal((16, 8)).astype(np.float32)
    wd = rng.standard_normal((8, 16)).astype(np.float32)
    full = orc.ref_swiglu_mlp(x, wg, wu, wd)
    tp = orc.ref_tp_swiglu_mlp(x, wg, wu, wd, 4)
    assert np.allclose(full, tp, rtol=1e-5, atol=1e-5)
    want = (x @ wg.T)
    want = want / (1 + np.exp(-want)) * (x @ wu.T)
    assert np.allclose(full, want @ wd.T, rtol=1e-4, atol=1e-4)


# ---- rows after the hot path: NF4, per-block INT8, per-tensor INT8 ------------------------------------

def test_nf4_lut_kats(orc):  # crates/oxicuda-quant/src/scheme/nf4.rs:213-233
    lut = orc.nf4_levels()
    assert (np.diff(lut) > 0).all()
    assert lut[0] == -1.0 and lut[15] == 1.0 and lut[7] == 0.0
    assert orc.ref_nearest_nf4(-1.0) == 0 and orc.ref_nearest_nf4(1.0) == 15 and orc.ref_nearest_nf4(0.0) == 7
    mid = float((lut[7] + lut[8]) / np.float32(2.0))
    assert orc.ref_nearest_nf4(mid) in (7, 8)
    assert orc.ref_nearest_nf4(-5.0) == 0 and orc.ref_nearest_nf4(5.0) == 15


def test_nf4_round_trip_kats(orc):  # nf4.rs:243-296
    t = (np.arange(128, dtype=np.float32) / np.float32(64.0)) - np.float32(1.0)
    packed, am = orc.ref_nf4_encode(t, 64)
    assert packed.size == 64 and am.size == 2
    dec = orc.ref_nf4_decode(packed, am, 64)
    assert float(((t - dec) ** 2).mean()) < 0.01
    packed, am = orc.ref_nf4_encode(np.zeros(64, np.float32), 64)       # all zeros: absmax floor 1e-8, code 7
    assert am[0] == np.float32(1e-8) and (packed == 0x77).all()
    assert np.abs(orc.ref_nf4_decode(packed, am, 64)).max() < 1e-5
    t = np.tile(2.0 * (np.arange(64, dtype=np.float32) / 64.0) - 1.0, 16)
    packed, am = orc.ref_nf4_encode(t, 64)
    assert float(((t - orc.ref_nf4_decode(packed, am, 64)) ** 2).mean()) < 0.05
    with pytest.raises(orc.OracleError) as e:
        orc.ref_nf4_encode(np.full(65, 0.5, np.float32), 64)
    assert e.value.name == "GroupSizeMismatch"
    with pytest.raises(orc.OracleError) as e:
        orc.ref_nf4_decode(np.zeros(32, np.uint8), np.ones(5, np.float32), 64)
    assert e.value.name == "DimensionMismatch"
    with pytest.raises(orc.OracleError) as e:
        orc.ref_nf4_encode(np.zeros(0, np.float32), 64)
    assert e.value.name == "EmptyInput"


def test_block_int8_kats(orc):  # crates/oxicuda-dnn/src/quantize/int8_quantize.rs:541-704
    x = np.arange(256, dtype=np.float32)
    q, s = orc.ref_block_int8_quant(x, 64)
    assert s.size == 4
    q, s = orc.ref_block_int8_quant(np.arange(100, dtype=np.float32), 64)        # 64 + 36
    assert s.size == 2 and orc.ref_block_int8_dequant(q, s, 64).size == 100
    x = np.array([1e30, -1e30, 0.0, 1e30], np.float32)
    q, s = orc.ref_block_int8_quant(x, 4)
    d = orc.ref_block_int8_dequant(q, s, 4)
    assert d[0] > 0 and d[1] < 0 and d[2] == 0.0 and list(q) == [127, -127, 0, 127]
    assert orc.ref_block_int8_quant(np.arange(256, dtype=np.float32), 128)[1].size == 2
    d = orc.ref_block_int8_dequant(np.array([-128, 0, 127], np.int8), np.array([0.1], np.float32), 3)
    assert np.allclose(d, [-12.8, 0.0, 12.7], atol=1e-4)
    x = np.concatenate([np.full(64, 0.001, np.float32), np.full(64, 100.0, np.float32)])
    _, s = orc.ref_block_int8_quant(x, 64)
    assert s[1] / s[0] > 10.0
    x = (np.arange(300, dtype=np.float32) - np.float32(150.0)) / np.float32(5.0)
    q, s = orc.ref_block_int8_quant(x, 100)
    assert s.size == 3
    assert (np.abs(x - orc.ref_block_int8_dequant(q, s, 100)) <= s.max() * 0.5 + 1e-5).all()
    _, s = orc.ref_block_int8_quant(np.zeros(8, np.float32), 4)                  # all-zero block -> scale 1
    assert (s == 1.0).all()


def test_dnn_int8_tensor_definition(orc):  # int8_quantize.rs:26-29 (the formula its kernels implement)
    x = orc.gaussian((1, 1000), 1.0, 3).ravel()
    q, s = orc.ref_dnn_int8_quant(x)
    assert s[0] == np.float32(np.abs(x).max()) / np.float32(127.0)
    want = np.rint(np.clip(x / s[0], -127, 127)).astype(np.int8)
    assert (q == want).all() and np.abs(q).max() == 127
    q0, s0 = orc.ref_dnn_int8_quant(np.zeros(4, np.float32))
    assert s0[0] == np.float32(1e-12) and (q0 == 0).all()
    assert np.allclose(orc.ref_dnn_int8_dequant(q, s[0]), q.astype(np.float32) * s[0])


def test_smooth_quant_kats(orc):  # crates/oxicuda-quant/src/scheme/smooth_quant.rs:311-440
    assert np.allclose(orc.ref_smooth_scales([4.0, 1.0, 9.0], [1.0, 4.0, 1.0], 0.5), [2.0, 0.5, 3.0], atol=1e-5)
    assert np.allclose(orc.ref_smooth_scales([2.0, 5.0], [3.0, 7.0], 1.0), [2.0, 5.0], atol=1e-5)
    assert np.allclose(orc.ref_smooth_scales([4.0, 1.0], [2.0, 5.0], 0.0), [0.5, 0.2], atol=1e-5)
    assert np.allclose(orc.ref_smooth_col_absmax(np.array([[1.0, -5.0, 2.0], [-3.0, 4.0, 1.0]], np.float32)), [3.0, 5.0, 2.0])
    assert np.allclose(orc.ref_smooth_col_absmax(np.array([[0.5, -2.0, 1.0], [-1.5, 0.3, 3.0]], np.float32)), [1.5, 2.0, 3.0])
    acts = (np.arange(12, dtype=np.float32) * np.float32(0.3) - np.float32(1.0)).reshape(3, 4)
    w = (np.arange(8, dtype=np.float32) * np.float32(0.2) - np.float32(0.5)).reshape(2, 4)
    a2, w2, _ = orc.ref_smooth_layer(acts, w, 0.5)
    assert np.allclose(acts @ w.T, a2 @ w2.T, atol=1e-4)                       # smoothing preserves the layer output
    acts = np.array([100.0, 1.0, -100.0, 1.0, 100.0, -1.0, -100.0, -1.0], np.float32).reshape(4, 2)
    w = np.array([0.5, 0.5, -0.5, 0.5], np.float32).reshape(2, 2)
    a2, _, sc = orc.ref_smooth_layer(acts, w, 0.5)
    assert np.abs(a2[:, 0]).max() / np.abs(a2[:, 1]).max() < 100.0 and sc[0] > 1.0
    with pytest.raises(orc.OracleError) as e:
        orc.ref_smooth_scales(np.ones(3, np.float32), np.ones(4, np.float32), 0.5)
    assert e.value.name == "DimensionMismatch"
    with pytest.raises(orc.OracleError) as e:
        orc.ref_smooth_scales(np.zeros(0, np.float32), np.zeros(0, np.float32), 0.5)
    assert e.value.name == "EmptyInput"


def test_rms_norm_kats(orc):  # crates/oxicuda-lm/src/layer/norm.rs:186-227
    out = orc.ref_rms_norm(np.array([[3.0, 4.0, 0.0, 0.0]], np.float32), np.ones(4, np.float32), 1e-8)
    assert abs(out[0, 0] - 1.2) < 1e-5 and abs(out[0, 1] - 1.6) < 1e-5 and abs(out[0, 2]) < 1e-5      # rms = 2.5
    out = orc.ref_rms_norm(np.ones((1, 2), np.float32), np.array([2.0, 0.5], np.float32), 1e-8)
    assert abs(out[0, 0] - 2.0) < 1e-5 and abs(out[0, 1] - 0.5) < 1e-5
    out = orc.ref_rms_norm(np.array([[1.0, 1.0], [2.0, 2.0]], np.float32), np.ones(2, np.float32), 1e-8)
    assert np.allclose(out, 1.0, atol=1e-5)
    with pytest.raises(orc.OracleError) as e:
        orc.ref_rms_norm(np.ones((2, 3), np.float32), np.ones(4, np.float32), 1e-5)
    assert e.value.name == "DimensionMismatch"


def test_swiglu_ffn_kats(orc):  # crates/oxicuda-lm/src/layer/ffn.rs:279-315, :359-389
    one = np.ones(1, np.float32)
    silu = lambda v: float(orc.ref_silu_mul(np.full(1, v, np.float32), one)[0])
    assert abs(silu(0.0)) < 1e-6 and abs(silu(10.0) - 10.0) < 1e-3 and silu(1.0) > 0.0 and silu(-1.0) < 0.0
    eye, eye2 = np.eye(4, dtype=np.float32), np.eye(2, dtype=np.float32)
    assert np.allclose(orc.ref_linear_f32(np.array([[3.0, 4.0]], np.float32), eye2), [[3.0, 4.0]], atol=1e-6)   # linear_vec_identity
    y = orc.ref_linear_f32(np.array([[1.0, 2.0]], np.float32), eye2, bias=np.array([10.0, 20.0], np.float32))
    assert np.allclose(y, [[11.0, 22.0]], atol=1e-6)                                                 # linear_vec_with_bias
    zeros8 = np.zeros((8, 4), np.float32)
    out = orc.ref_swiglu_mlp(np.ones((1, 4), np.float32), zeros8, zeros8, np.zeros((4, 8), np.float32))
    assert out.shape == (1, 4) and np.all(np.abs(out) < 1e-6)                                        # zero weights -> zero output
    out = orc.ref_swiglu_mlp(np.full((1, 4), 2.0, np.float32), eye, eye, eye)                        # gate = up = down = I
    assert np.allclose(out, 2.0 / (1.0 + math.exp(-2.0)) * 2.0, atol=1e-5)
    out = orc.ref_swiglu_mlp(np.zeros((3, 4), np.float32), zeros8, zeros8, np.zeros((4, 8), np.float32))
    assert out.shape == (3, 4)                                                                       # three tokens at once


def test_fused_dequant_gemv_definition(orc):  # crates/oxicuda-dnn/src/quantize/gptq_awq.rs:867-994 (the arithmetic its kernel states)
    # 4 bits: element `sub` of a word at bit 4 * sub; one group of 8 with scale 0.5; x = 1 -> 0.5 * (0 + 1 + ... + 7)
    y = orc.ref_dnn_fused_dequant_gemv(np.array([0x76543210], np.uint32), np.array([0.5], np.float32), np.ones(8, np.float32), 1, 8, 8, 4)
    assert y.tolist() == [14.0]
    # two rows, two groups of 8 per row, codes unsigned (0xF is 15, not -1), x picks single columns
    w = np.array([0x0000000F, 0xF0000000, 0x00000001, 0x10000000], np.uint32)
    s = np.array([2.0, 3.0, 0.25, 0.5], np.float32)
    x = np.zeros(16, np.float32); x[0] = 1.0; x[15] = 10.0
    assert orc.ref_dnn_fused_dequant_gemv(w, s, x, 2, 16, 8, 4).tolist() == [15 * 2.0 + 15 * 3.0 * 10.0, 0.25 + 0.5 * 10.0]
    # 8 bits: four codes per word; 2 bits: sixteen
    assert orc.ref_dnn_fused_dequant_gemv(np.array([0xFF000102], np.uint32), np.array([1.0], np.float32), np.array([1, 10, 100, 1000], np.float32), 1, 4, 4, 8).tolist() == [2 + 10 + 255000.0]
    assert orc.ref_dnn_fused_dequant_gemv(np.array([0xE4E4E4E4], np.uint32), np.array([1.0], np.float32), np.ones(16, np.float32), 1, 16, 16, 2).tolist() == [24.0]


def test_gptq_kats(orc):  # crates/oxicuda-quant/src/scheme/gptq.rs:341-520
    l = orc.ref_cholesky_lower(np.array([[4.0, 2.0], [2.0, 3.0]], np.float32))          # L = [[2, 0], [1, sqrt 2]]
    assert np.allclose(l, [[2.0, 0.0], [1.0, np.sqrt(2.0)]], atol=1e-6) and np.allclose(l @ l.T, [[4.0, 2.0], [2.0, 3.0]], atol=1e-5)
    assert np.allclose(orc.ref_cholesky_lower(np.eye(4, dtype=np.float32)), np.eye(4), atol=1e-6)
    l3 = np.array([[2.0, 0.0, 0.0], [1.0, 3.0, 0.0], [0.0, 2.0, 4.0]], np.float32)
    assert np.allclose(l3 @ orc.ref_invert_lower(l3), np.eye(3), atol=1e-5)
    with pytest.raises(orc.OracleError) as e:                                               # zero Hessian, no dampening
        orc.ref_gptq_quantize_layer(np.full(4, 0.5, np.float32), 2, 2, np.zeros(4, np.float32), percdamp=0.0)
    assert e.value.name == "SingularHessian"
    with pytest.raises(orc.OracleError) as e:
        orc.ref_gptq_quantize_layer(np.full(3, 0.5, np.float32), 1, 4, np.eye(4, dtype=np.float32))
    assert e.value.name == "DimensionMismatch"
    with pytest.raises(orc.OracleError) as e:
        orc.ref_gptq_quantize_layer(np.full(4, 0.5, np.float32), 2, 2, np.eye(2, dtype=np.float32), bits=0)
    assert e.value.name == "InvalidBitWidth"
    w = (np.arange(32, dtype=np.float32) / np.float32(16.0) - np.float32(1.0)).reshape(4, 8)
    q, sc, zp = orc.ref_gptq_quantize_layer(w, 4, 8, np.eye(8, dtype=np.float32), bits=8)
    assert np.mean((orc.gptq_dequantize(q, sc, zp) - w) ** 2) < 1e-4                       # identity Hessian: round to nearest
    q, sc, zp = orc.ref_gptq_quantize_layer(np.full((3, 6), 0.3, np.float32), 3, 6, np.eye(6, dtype=np.float32), bits=4)
    assert q.shape == (3, 6) and sc.shape == (6,) and zp.shape == (6,)
    w = np.array([-0.6, 0.4, -0.2, 0.8, 0.6, -0.4, 0.2, -0.8], np.float32).reshape(2, 4)
    q, sc, zp = orc.ref_gptq_quantize_layer(w, 2, 4, np.eye(4, dtype=np.float32), bits=4, symmetric=False)
    assert np.mean((orc.gptq_dequantize(q, sc, zp) - w) ** 2) < 0.05 and q.min() >= 0 and q.max() <= 15
    # a diagonal Hessian has a diagonal inverse, so no error propagates: same codes as with the identity
    rng = np.random.default_rng(3)
    w = rng.standard_normal((16, 32)).astype(np.float32)
    hd = np.diag(rng.uniform(0.5, 4.0, 32)).astype(np.float32)
    q, sc, zp = orc.ref_gptq_quantize_layer(w, 16, 32, hd, bits=4)
    qi, sci, zpi = orc.ref_gptq_quantize_layer(w, 16, 32, np.eye(32, dtype=np.float32), bits=4)
    assert np.array_equal(q, qi) and np.array_equal(sc, sci)
    # a dense Hessian does propagate: later columns change
    x = rng.standard_normal((256, 32)).astype(np.float32)
    q2, _, _ = orc.ref_gptq_quantize_layer(w, 16, 32, (2.0 * x.T @ x / 256.0).astype(np.float32), bits=4)
    assert np.array_equal(q2[:, 0], qi[:, 0]) and not np.array_equal(q2, qi)


# --------------------------------------------------------------------------- DNN INT4 / block-scaled (f1)

def test_fp4_block_quantizer_scale_kats(orc):
    """Fp4BlockQuantizer::compute_scale known answers (crates/oxicuda-dnn/src/quantize/block_scale.rs:511-544, :574-590)."""
    assert orc.ref_fp4_block_compute_scale(np.zeros(32, np.float32)) == 1.0
    assert abs(orc.ref_fp4_block_compute_scale(np.full(32, 6.0, np.float32)) - 1.0) < 1e-6
    assert abs(orc.ref_fp4_block_compute_scale(np.full(32, 12.0, np.float32)) - 2.0) < 1e-6
    blk = np.zeros(32, np.float32)
    blk[0], blk[1], blk[2] = -6.0, 3.0, 1.5
    assert abs(orc.ref_fp4_block_compute_scale(blk) - 1.0) < 1e-6


def test_dnn_block_scaled_restatement(orc):
    """quantize_block_scaled's generated arithmetic (block_scale.rs:243-249, :300-333) on hand-checked values:
    scale = absmax / 6, codes = rint(x / scale) + 6, ties to even, a short last block, an all-zero block."""
    x = np.array([6.0, -6.0, 3.0, 2.5, 1.5, 0.5, -0.5, 0.0] + [0.0] * 8 + [0.0] * 16 + [12.0, -3.0], np.float32)
    q, s = orc.ref_dnn_block_scaled_quant(x, 16)
    assert s.tolist() == [1.0, np.float32(1e-12), 2.0]
    assert q[:8].tolist() == [12, 0, 9, 8, 8, 6, 6, 6]               # 2.5 -> 2, 1.5 -> 2, +-0.5 -> 0 (half to even)
    assert q[16:32].tolist() == [6] * 16
    assert q[32:].tolist() == [12, 4]                                 # -3 / 2 = -1.5 -> -2


def test_dnn_int4_restatement(orc):
    """quantize_to_int4's generated arithmetic (int4_quantize.rs:440-468, :518-536, :655-690): symmetric scale = absmax / 7
    with codes trunc(x / scale + 8); asymmetric scale = (max - min) / 15, zero = -min / scale, codes trunc(x / scale) clamped at 0."""
    x = np.array([7.0, -7.0, 3.5, -3.5, 0.0, 1.0, -8.0, 6.9], np.float32)
    p, s, z = orc.ref_dnn_int4_quant(x, 8, True)
    assert s.tolist() == [np.float32(8.0) / np.float32(7.0)] and z is None
    codes = [int(b) & 15 for b in p for _ in (0,)] + []
    lo = [int(b) & 15 for b in p]
    hi = [int(b) >> 4 for b in p]
    got = [v for pair in zip(lo, hi) for v in pair]
    want = [int(min(max(np.float32(v) / s[0], -8.0), 7.0) + 8.0) for v in x]
    assert got == want and got[6] == 1 and got[0] == 14              # -8 / (8/7) = -7 -> 1; 7 / (8/7) = 6.125 -> 14
    y = orc.ref_dnn_int4_dequant(p, s, 8, 8, True)
    assert y[4] == 0.0 and y[6] == np.float32(-7.0) * s[0]
    x = np.arange(16, dtype=np.float32) - 5.0                         # min -5, max 10: scale 1, zero 5; negatives clamp to code 0
    p, s, z = orc.ref_dnn_int4_quant(x, 16, False)
    assert s.tolist() == [1.0] and z.tolist() == [5.0]
    lo = [int(b) & 15 for b in p]
    hi = [int(b) >> 4 for b in p]
    got = [v for pair in zip(lo, hi) for v in pair]
    assert got == [0, 0, 0, 0, 0, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    p, s, z = orc.ref_dnn_int4_quant(np.zeros(5, np.float32), 4, True)   # short last group, all zero: scale floor 1e-12 / 7
    assert len(p) == 3 and s.tolist() == [np.float32(1e-12) / np.float32(7.0)] * 2

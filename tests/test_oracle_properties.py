"""Size-independent properties of the CPU oracle on generated inputs (hypothesis): the relations any correct quantizer of
each kind satisfies, whatever the data.  They guard the oracle itself; the GPU parity tests compare the kernels with it."""
import numpy as np
import pytest

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings  # noqa: E402
from hypothesis import strategies as st  # noqa: E402
from hypothesis.extra import numpy as hnp  # noqa: E402

FINITE = st.floats(min_value=-1e4, max_value=1e4, allow_nan=False, allow_infinity=False, width=32)
SETTINGS = dict(max_examples=60, deadline=None, derandomize=True, database=None)   # the same examples on every run


def _matrix(rows, cols):
    return hnp.arrays(np.float32, (rows, cols), elements=FINITE)


@settings(**SETTINGS)
@given(x=_matrix(4, 64))
def test_int8_per_row_round_trip_within_half_a_step(orc, x):
    """MinMaxQuantizer, 8-bit symmetric per row (minmax.rs:179-324): |dequant(quant(x)) - x| <= scale / 2 and codes in [-127, 127]."""
    scales, zps = orc.ref_minmax_calibrate_2d(x, 4, 64)
    q = orc.minmax_quantize_grouped(x, scales, zps, 64).reshape(4, 64)
    assert q.min() >= -127 and q.max() <= 127 and not zps.any()
    back = orc.ref_minmax_dequantize_grouped(q, scales, zps, 64).reshape(4, 64)
    assert np.all(np.abs(back - x) <= scales[:, None] * 0.5 * (1 + 1e-5) + 1e-30)
    # the element of largest magnitude in a row lands on +-127
    for r in range(4):
        if np.abs(x[r]).max() > 1e-6:
            assert abs(q[r, np.abs(x[r]).argmax()]) == 127


@settings(**SETTINGS)
@given(x=_matrix(2, 128), rounding=st.sampled_from([0, 1]))
def test_spec_int8_rows_agree_with_the_reference_path_off_ties(orc, x, rounding):
    """The per-row form the kernels implement equals calibrate_2d + quantize_grouped; the rounding mode only matters at ties."""
    q, s = orc.spec_int8_quant_rows(x, rounding)
    sr, zr = orc.ref_minmax_calibrate_2d(x, 2, 128)
    assert np.array_equal(s.view(np.uint32), sr.view(np.uint32))
    qr = orc.minmax_quantize_grouped(x, sr, zr, 128, rounding=rounding, clamp_sym_lo127=True).reshape(2, 128)
    assert np.array_equal(q.astype(np.int32), qr)
    other, _ = orc.spec_int8_quant_rows(x, 1 - rounding)
    ratio = x / s[:, None]
    ties = np.abs(np.abs(ratio - np.trunc(ratio)) - 0.5) < 1e-6
    assert np.array_equal(q[~ties], other[~ties])


@settings(**SETTINGS)
@given(x=_matrix(2, 256))
def test_int4_groups_round_trip_within_a_step(orc, x):
    """uint4 per group of 128, asymmetric (minmax.rs:146-167, :226-232): codes in [0, 15].  The zero-point is clamped to [0, 15]
    as in the reference, so only a group whose range contains zero is representable; there the reconstruction is within one
    step (zero-point rounding adds up to half a step to the half step of the code, the f16 scale a little more)."""
    codes, scales, zeros = orc.spec_int4g_quant(x, 128, orc.ROUND_HALF_AWAY)
    nib = orc.unpack_uint4(codes)
    assert nib.min() >= 0 and nib.max() <= 15
    back = orc.spec_int4g_dequant(codes, scales, zeros, 2, 256, 128)
    s = np.repeat(orc.f16_bits_to_f32(scales).reshape(2, 2), 128, axis=1)
    g = x.reshape(2, 2, 128)
    spans_zero = np.repeat((g.min(axis=2) <= 0) & (g.max(axis=2) >= 0), 128, axis=1).reshape(2, 256)
    ok = np.isfinite(s) & (s > 1e-6) & spans_zero
    assert np.all(np.abs(back - x)[ok] <= s[ok] * 1.05 + 1e-6)


@settings(**SETTINGS)
@given(v=hnp.arrays(np.int8, 64, elements=st.integers(-8, 7)))
def test_pack_int4_round_trip(orc, v):
    """pack_int4 / unpack_int4 (int_ops.rs:375-428): eight signed nibbles per word, element j at bits [4j, 4j + 4)."""
    words = orc.ref_pack_int4(v)
    assert words.size == 8 and np.array_equal(orc.ref_unpack_int4(words), v)
    for j in range(8):
        assert ((int(words[0]) >> (4 * j)) & 0xF) == (int(v[j]) & 0xF)


@settings(**SETTINGS)
@given(x=hnp.arrays(np.float32, 64, elements=st.floats(min_value=-448, max_value=448, allow_nan=False, width=32)))
def test_e4m3_encode_is_the_nearest_code(orc, x):
    """RNE, saturating E4M3: no other finite code is closer; decode(encode(x)) is idempotent; the sign is kept."""
    codes = orc.e4m3_rne_sat(x)
    grid = orc.e4m3_to_f32(np.arange(256, dtype=np.uint8))
    finite = np.isfinite(grid)
    back = orc.e4m3_to_f32(codes)
    best = np.abs(grid[finite][None, :] - x[:, None]).min(axis=1)
    assert np.all(np.abs(back - x) <= best * (1 + 1e-6) + 1e-30)
    assert np.array_equal(orc.e4m3_rne_sat(back), codes)
    assert np.all(np.signbit(back) == np.signbit(x))


@settings(**SETTINGS)
@given(x=_matrix(4, 64))
def test_mxfp8_block_scale_rule(orc, x):
    """MXFP8 (E8M0 per 32, OCP MX v1.0): the scale is 2^(floor(log2 max) - 8), so the block maximum lands in [256, 512) and the
    part of a block above 448 scales (the top eighth of its binade) saturates to 448; everything else is rounded to nearest."""
    codes, sf = orc.spec_mxfp8_quant(x)
    back = orc.spec_mxfp8_dequant(codes, sf)
    scale = np.repeat(np.exp2(sf.astype(np.float64) - 127.0).reshape(4, 2), 32, axis=1)
    blk = np.repeat(np.abs(x).reshape(4, 2, 32).max(axis=2), 32, axis=1).reshape(4, 64)
    big = blk > 1e-30
    assert np.all((blk / scale)[big] >= 256.0) and np.all((blk / scale)[big] < 512.0)
    clipped = big & (np.abs(x) / scale > 448.0)
    assert np.all(np.abs(back[clipped]) == (448.0 * scale)[clipped]) and np.all(np.sign(back[clipped]) == np.sign(x[clipped]))
    rounded = big & ~clipped
    # relative step of E4M3 is 2^-3 for normals (half of it the error); below 2^-6 scales the grid is uniform with step 2^-9 scales
    assert np.all(np.abs(back - x)[rounded] <= np.maximum(np.abs(x) * 2.0 ** -4, scale * 2.0 ** -10)[rounded] * (1 + 1e-6))


@settings(**SETTINGS)
@given(x=_matrix(2, 64))
def test_nvfp4_error_is_within_half_the_widest_step(orc, x):
    """NVFP4 (E2M1 codes, a UE4M3 scale per 16, one f32 tensor scale g): with s the decoded block scale times g, every element is
    reconstructed within s (half of E2M1's widest step, 2), including the few at the top of a block that clip at 6 s when the
    block scale rounded down; the scale itself is within E4M3's rounding (2^-4 relative) of max / 6."""
    g = float(orc.spec_nvfp4_global_scale(float(np.abs(x).max())))
    packed, sf = orc.spec_nvfp4_quant(x, g)
    back = orc.spec_nvfp4_dequant(packed, sf, g, 2, 64)
    s = np.repeat(orc.e4m3_to_f32(sf).astype(np.float64) * g, 16, axis=1)
    # where the block scale is a subnormal E4M3 number its grid is uniform (step 2^-9): the scale may be short of max / 6 by half
    # a step, down to zero for a block 2^-10 g and less in size, and the elements above 6 s clip
    slack = np.where(np.repeat(orc.e4m3_to_f32(sf), 16, axis=1) >= 2.0 ** -6, 0.0, 6.0 * g * 2.0 ** -10)
    assert np.all(np.abs(back - x) <= (s + slack) * (1 + 1e-6) + 1e-30)
    assert np.all(np.abs(back) <= 6.0 * s * (1 + 1e-6))
    blk = np.abs(x).reshape(2, 4, 16).max(axis=2).astype(np.float64)
    normal = orc.e4m3_to_f32(sf) >= 2.0 ** -6
    assert np.all(np.abs(s[:, ::16] * 6.0 - blk)[normal] <= blk[normal] * 2.0 ** -4 * (1 + 1e-6))


@settings(**SETTINGS)
@given(x=hnp.arrays(np.float32, 128, elements=st.floats(min_value=-100, max_value=100, allow_nan=False, width=32)))
def test_nf4_codes_are_nearest_levels(orc, x):
    """Nf4Quantizer (nf4.rs:93-155): each code is a nearest level of x / absmax; decode(encode(x)) re-encodes to the same codes."""
    packed, absmax = orc.ref_nf4_encode(x, 64)
    levels = orc.nf4_levels()
    nib = np.stack([packed & 0xF, packed >> 4], axis=1).ravel()
    am = np.repeat(np.maximum(absmax, np.float32(1e-8)), 64)
    norm = np.clip(x / am, -1.0, 1.0)
    dist = np.abs(levels[None, :] - norm[:, None])
    assert np.all(dist[np.arange(128), nib] <= dist.min(axis=1) + 1e-7)
    back = orc.ref_nf4_decode(packed, absmax, 64)
    p2, a2 = orc.ref_nf4_encode(back, 64)
    assert np.all(a2 <= absmax * (1 + 1e-6) + 1e-8)
    assert np.allclose(orc.ref_nf4_decode(p2, a2, 64), back, rtol=1e-5, atol=1e-7) or np.array_equal(p2, packed)


@settings(**SETTINGS)
@given(a=_matrix(3, 16), b=_matrix(3, 16), w=_matrix(5, 16))
def test_reference_linear_is_linear_to_rounding(orc, a, b, w):
    """Y = X W^T in the reference's sequential f32 order (ffn.rs:72-110): additive in X up to f32 rounding of the sums."""
    ya, yb, yab = orc.ref_linear_f32(a, w), orc.ref_linear_f32(b, w), orc.ref_linear_f32(a + b, w)
    mag = (np.abs(a) + np.abs(b)) @ np.abs(w).T
    assert np.all(np.abs(yab - (ya + yb)) <= 1e-5 * mag + 1e-30)


@settings(**SETTINGS)
@given(w=hnp.arrays(np.float32, (6, 8), elements=st.floats(min_value=-4, max_value=4, allow_nan=False, width=32)),
       bits=st.sampled_from([3, 4, 8]), symmetric=st.booleans(), diag=st.floats(min_value=0.5, max_value=8.0))
def test_gptq_with_a_diagonal_hessian_is_round_to_nearest_per_column(orc, w, bits, symmetric, diag):
    """GptqQuantizer::quantize_layer (gptq.rs:133-257): a diagonal Hessian has a diagonal inverse, so no column's error reaches a later
    column and the codes are plain per-column round-to-nearest with the column's own parameters (col_quant_params, :242-276)."""
    h = np.eye(8, dtype=np.float32) * np.float32(diag)
    q, sc, zp = orc.ref_gptq_quantize_layer(w, 6, 8, h, bits=bits, symmetric=symmetric, percdamp=0.01)
    if symmetric:
        q_min, q_max = -(1 << (bits - 1)), (1 << (bits - 1)) - 1
        am = np.maximum(np.abs(w).max(axis=0), np.float32(1e-8))
        scale = (am / np.float32(q_max)).astype(np.float32)
        zero = np.zeros(8, np.int32)
    else:
        q_min, q_max = 0, (1 << bits) - 1
        lo, hi = w.min(axis=0), w.max(axis=0)
        scale = (np.maximum(hi - lo, np.float32(1e-8)) / np.float32(q_max)).astype(np.float32)
        t = (-lo / scale).astype(np.float32)
        zero = np.clip(np.sign(t) * np.floor(np.abs(t) + np.float32(0.5)), q_min, q_max).astype(np.int32)
    assert np.array_equal(sc.view(np.uint32), scale.view(np.uint32)) and np.array_equal(zp, zero)
    t = (w / scale[None, :]).astype(np.float32) + zero[None, :].astype(np.float32)
    want = np.clip(np.sign(t) * np.floor(np.abs(t) + np.float32(0.5)), q_min, q_max).astype(np.int32)
    assert np.array_equal(q, want)
    assert np.all(np.abs(orc.gptq_dequantize(q, sc, zp) - w)[(want > q_min) & (want < q_max)] <= scale[None, :].repeat(6, axis=0)[(want > q_min) & (want < q_max)] * 0.5 * (1 + 1e-5) + 1e-7)

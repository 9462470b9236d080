"""Checks the oracle's format conversions against independent implementations (numpy float16,
torch float8_e4m3fn / bfloat16 on CPU, brute-force nearest-grid search, ml_dtypes' float4_e2m1fn /
float8_e4m3fn / float8_e8m0fnu) and the spec quantizers against plain numpy restatements of their
stated formulas (the block-scaled ones rebuilt from ml_dtypes casts, code for code)."""
import numpy as np
import pytest
import torch


def _all_interesting_f32():
    rng = np.random.default_rng(1)
    a = rng.standard_normal(20000).astype(np.float32) * np.float32(30.0)
    b = (rng.standard_normal(20000).astype(np.float32) * np.float32(0.01))
    grid = np.arange(-520, 520, dtype=np.float32) * np.float32(0.5)
    ties = np.array([0.0009765625 * k for k in range(0, 64)], np.float32)        # multiples of 2^-10
    return np.concatenate([a, b, grid, ties, -ties, np.array([448.0, 449.0, 463.9, 464.0, 480.0, 1e9, -1e9,
                                                             2.0 ** -9, 2.0 ** -10, 1.5 * 2.0 ** -10], np.float32)])


def test_e4m3_rne_matches_torch(orc):
    x = _all_interesting_f32()
    got = orc.e4m3_rne_sat(x)
    xc = np.clip(x, -448.0, 448.0)                       # torch's cast does not saturate; clip first
    want = torch.from_numpy(xc).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert (got == want).all(), np.nonzero(got != want)[0][:10]
    assert orc.e4m3_rne_sat([float("inf")])[0] == 0x7E and orc.e4m3_rne_sat([float("-inf")])[0] == 0xFE
    assert orc.e4m3_rne_sat([float("nan")])[0] == 0x7F


def test_e4m3_decode_all_bytes(orc):
    b = np.arange(256, dtype=np.uint8)
    got = orc.e4m3_to_f32(b)
    want = torch.from_numpy(b).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    assert np.array_equal(got, want, equal_nan=True)


def test_f16_bf16_helpers(orc):
    x = np.concatenate([_all_interesting_f32(), np.array([65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8,
                                                          2.9802322e-08, 6.1e-5], np.float32)])
    got = np.array([orc.lib().orc_f32_to_f16(float(v)) & 0xFFFF for v in x], np.uint16)
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    assert (got == want).all(), x[got != want][:10]
    gotb = orc.f32_to_bf16_bits(x)
    wantb = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert (gotb == wantb).all()
    gotc = np.array([orc.lib().orc_f32_to_bf16(float(v)) & 0xFFFF for v in x[:2000]], np.uint16)
    assert (gotc == wantb[:2000]).all()


def test_e2m1_rne_brute_force(orc):
    grid = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], np.float64)
    xs = np.concatenate([np.linspace(-7, 7, 5601), np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 100.0])])
    got = orc.e2m1_rne_sat(xs.astype(np.float32))
    for x, c in zip(xs.astype(np.float32), got):
        a = abs(float(x))
        d = np.abs(grid - min(a, 6.0))
        best = np.nonzero(d == d.min())[0]
        code = best[0] if len(best) == 1 else [b for b in best if b % 2 == 0][0]
        assert (c & 7) == code, (x, c, code)
        assert (c >> 3) == (1 if np.signbit(x) else 0)


def test_spec_int8_rows(orc):
    x = orc.gaussian((16, 512), 0.02, 0)
    for rounding, rnd in ((orc.ROUND_HALF_EVEN, np.rint), (orc.ROUND_HALF_AWAY, lambda v: np.sign(v) * np.floor(np.abs(v) + 0.5))):
        q, s = orc.spec_int8_quant_rows(x, rounding)
        s_want = (np.maximum(np.abs(x).max(axis=1), np.float32(1e-8)) / np.float32(127.0)).astype(np.float32)
        assert np.array_equal(s, s_want)
        q_want = np.clip(rnd((x / s_want[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
        assert np.array_equal(q, q_want)
        # agrees with the reference path (calibrate_2d + quantize_grouped) on calibrated data
        sr, zr = orc.ref_minmax_calibrate_2d(x, 16, 512)
        assert np.array_equal(sr, s)
        qr = orc.minmax_quantize_grouped(x, sr, zr, 512, 8, orc.SYMMETRIC, rounding, False)
        assert np.array_equal(qr.reshape(16, 512), q.astype(np.int32))
    assert np.array_equal(orc.spec_int8_dequant_rows(q, s), q.astype(np.float32) * s[:, None])


def test_spec_fp8_per_tensor(orc):
    x = orc.gaussian((64, 256), 1.0, 0)
    xb = orc.f32_to_bf16_bits(x)
    am = orc.spec_absmax(xb)
    assert am == np.abs(orc.bf16_bits_to_f32(xb)).max()
    sc = orc.spec_fp8_scale(am)
    assert sc == np.float32(am) / np.float32(448.0)
    q = orc.spec_fp8_quant(xb, sc)
    want = torch.from_numpy((orc.bf16_bits_to_f32(xb) / sc).astype(np.float32)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(q, want)
    assert q.max() >= 0x7E or (q & 0x7F).max() == 0x7E     # the absmax element lands on 448
    assert np.array_equal(orc.spec_fp8_dequant(q, sc), orc.e4m3_to_f32(q) * sc)


def test_spec_fp8_reference_properties(orc):  # crates/oxicuda-dnn/src/quantize/fp8_quantize.rs:494-655
    """The properties the reference asserts of its absmax-scaled FP8 arithmetic (clamp at 448, tiny values to zero,
    scale = absmax / 448, round trip within a step, odd symmetry) hold for the spec oracle as well."""
    f = lambda v, sc=1.0: orc.spec_fp8_dequant(orc.spec_fp8_quant(np.asarray(v, np.float32), np.float32(sc)), np.float32(sc))
    assert abs(f([1000.0])[0] - 448.0) < 1.0 and abs(f([-1000.0])[0] + 448.0) < 1.0                  # :494-509
    assert abs(f([1e-10])[0]) < 1.0 / 8.0                                                             # :529-538
    vals = np.array([10.0, -50.0, 30.0, -20.0, 5.0], np.float32)                                      # :555-575
    am = orc.spec_absmax(vals)
    sc = orc.spec_fp8_scale(am)
    assert abs(am - 50.0) < 1e-6 and abs(float(sc) - 50.0 / 448.0) < 1e-6
    assert abs(f([am], sc)[0] - am) < float(sc) * 0.5
    orig = np.array([1.0, -2.0, 0.5, -0.25, 4.0, -3.75], np.float32)                                  # :579-598
    sc = max(np.float32(4.0) / np.float32(448.0), np.float32(1e-12))
    back = f(orig, sc)
    # the reference's model has a fixed step of scale / 8; real E4M3 has a relative step of 2^-3 per binade, so the
    # bound that holds for it is half a step of the value's own binade: |x| / 16
    assert np.all(np.abs(back - orig) <= np.abs(orig) / 16.0 + 1e-6)
    for x in (0.5, 1.0, 2.0, 5.0, 10.0, 100.0):                                                       # :622-633
        assert abs(f([x])[0] + f([-x])[0]) < 1e-5


def test_spec_int4g(orc):
    x = orc.gaussian((8, 512), 0.02, 3)
    codes, sc, zp = orc.spec_int4g_quant(x, 128, orc.ROUND_HALF_AWAY)
    xs = x.reshape(8, 4, 128)
    mn, mx = xs.min(axis=2), xs.max(axis=2)
    s32 = (np.maximum(mx - mn, np.float32(1e-8)) / np.float32(15.0)).astype(np.float32)
    s16 = s32.astype(np.float16)
    assert np.array_equal(sc.view(np.float16), s16)
    s = s16.astype(np.float32)
    away = lambda v: np.sign(v) * np.floor(np.abs(v) + np.float32(0.5))
    z = np.clip(away((-mn / s).astype(np.float32)), 0, 15).astype(np.uint8)
    assert np.array_equal(orc.unpack_uint4(zp)[:32], z.ravel())
    q = np.clip(away((xs / s[..., None]).astype(np.float32) + z[..., None].astype(np.float32)), 0, 15).astype(np.uint8)
    assert np.array_equal(orc.unpack_uint4(codes), q.ravel())
    deq = orc.spec_int4g_dequant(codes, sc, zp, 8, 512, 128)
    want = (q.astype(np.int32) - z[..., None].astype(np.int32)).astype(np.float32) * s[..., None]
    assert np.array_equal(deq, want.reshape(8, 512))
    assert np.abs(deq - x).max() <= s.max() * 0.51 + 1e-7
    # f32-scale reference path differs only through the scale dtype: same formula with refcompat calibrate
    rs, rz = orc.ref_minmax_calibrate(x.ravel(), 4, orc.ASYMMETRIC, group=128)
    assert np.array_equal(rs, s32.ravel())


def test_spec_mxfp8(orc):
    x = orc.gaussian((8, 256), 1.0, 5)
    x[0, :32] = 0.0
    x[1, 32:64] *= 1e-30
    x[2, :32] *= 1e30
    codes, sf = orc.spec_mxfp8_quant(x)
    xb = x.reshape(8, 8, 32)
    am = np.abs(xb).max(axis=2)
    assert sf[0, 0] == 0 and (codes[0, :32] == 0).all()
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(am.astype(np.float64))) - 8
    want_sf = np.where(am == 0, 0, np.clip(e + 127, 0, 254)).astype(np.uint8)
    assert np.array_equal(sf, want_sf)
    scaled = (xb.astype(np.float64) * np.exp2(-(want_sf.astype(np.float64) - 127))[..., None]).astype(np.float32)
    want_codes = torch.from_numpy(np.clip(scaled, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(codes.reshape(8, 8, 32), want_codes)
    assert (sf != 255).all()
    # every nonzero block uses the top binade: max |code value| in [256, 448]
    vals = np.abs(orc.e4m3_to_f32(codes)).reshape(8, 8, 32).max(axis=2)
    assert ((vals[am > 0] >= 256) & (vals[am > 0] <= 448)).all()
    deq = orc.spec_mxfp8_dequant(codes, sf)
    err = np.abs(deq - x).reshape(8, 8, 32).max(axis=2)
    assert (err <= am / 8.0).all()          # values in (448, 512) * 2^e saturate to 448 * 2^e


def test_spec_nvfp4(orc):
    x = orc.gaussian((8, 256), 1.0, 7)
    x[0, :16] = 0.0
    x[1, 16:32] *= 1e-6
    g = orc.spec_nvfp4_global_scale(orc.spec_absmax(x))
    assert g == np.float32(np.abs(x).max()) / np.float32(448.0 * 6.0)
    packed, sf = orc.spec_nvfp4_quant(x, g)
    xb = x.reshape(8, 16, 16)
    am = np.abs(xb).max(axis=2)
    want_sf = orc.e4m3_rne_sat((am / (np.float32(6.0) * g)).astype(np.float32).ravel()).reshape(8, 16)
    assert np.array_equal(sf, want_sf)
    assert sf.max() == 0x7E and sf[0, 0] == 0 and sf[1, 1] == 0
    d = (g * orc.e4m3_to_f32(sf)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        scaled = (xb / d[..., None]).astype(np.float32)
    want = orc.e2m1_rne_sat(np.where(d[..., None] == 0, np.copysign(0.0, xb), scaled).ravel()).reshape(8, 128, 2)
    assert np.array_equal(packed.reshape(8, 128), want[..., 0] | (want[..., 1] << 4))
    deq = orc.spec_nvfp4_dequant(packed, sf, g, 8, 256)
    err = np.abs(deq - x).reshape(8, 16, 16).max(axis=2)
    assert (err <= np.maximum(am * 0.2, 1e-5)).all()


def test_linear_order_and_threads(orc):
    x = orc.gaussian((4, 333), 1.0, 1)
    w = orc.gaussian((17, 333), 0.02, 0)
    y1 = orc.ref_linear_f32(x, w, threads=1)
    y8 = orc.ref_linear_f32(x, w, threads=4)
    assert np.array_equal(y1, y8)                         # threading splits outputs, not the k-sum
    acc = np.float32(0.0)
    for i in range(333):
        acc = np.float32(acc + np.float32(x[2, i] * w[5, i]))
    assert y1[2, 5] == acc


# ---- against ml_dtypes (Google's reference implementation of the narrow float types): element conversions, then the two
#      block-scaled quantizers rebuilt from its casts and compared code for code -------------------------------------------

def test_element_conversions_match_ml_dtypes(orc):
    ml = pytest.importorskip("ml_dtypes")
    x = _all_interesting_f32()
    inside = x[np.abs(x) <= 448.0]                                       # beyond 448 ml_dtypes gives NaN, the quantizers saturate
    assert np.array_equal(orc.e4m3_rne_sat(inside), inside.astype(ml.float8_e4m3fn).view(np.uint8))
    assert np.array_equal(orc.e4m3_to_f32(np.arange(256, dtype=np.uint8)), np.arange(256, dtype=np.uint8).view(ml.float8_e4m3fn).astype(np.float32),
                          equal_nan=True)
    small = np.concatenate([x[np.abs(x) <= 8.0], np.arange(-64, 65, dtype=np.float32) * np.float32(0.125), np.array([6.0, 7.0, 100.0, -1e9], np.float32)])
    assert np.array_equal(orc.e2m1_rne_sat(small) & 0xF, small.astype(ml.float4_e2m1fn).view(np.uint8) & 0xF)        # saturating, ties to even
    assert np.array_equal(orc.e2m1_to_f32(np.arange(16, dtype=np.uint8)), np.arange(16, dtype=np.uint8).view(ml.float4_e2m1fn).astype(np.float32))
    # E8M0: byte b is 2^(b - 127) (0xFF is NaN and never written by the quantizer)
    b = np.arange(255, dtype=np.uint8)
    x8 = orc.gaussian((1, 32), 1.0, 3)
    for byte in (1, 60, 127, 128, 200, 246):                                     # 246: a block maximum in the last f32 binade
        scaled = (x8 * np.exp2(np.float32(byte - 127 + 8) - np.floor(np.log2(np.abs(x8).max())))).astype(np.float32)
        _, sf = orc.spec_mxfp8_quant(scaled)
        assert sf[0, 0] == byte and float(b[byte:byte + 1].view(ml.float8_e8m0fnu).astype(np.float32)[0]) == 2.0 ** (byte - 127)


def _mxfp8_with_ml_dtypes(ml, x):
    rows, k = x.shape
    blocks = x.reshape(rows, k // 32, 32)
    amax = np.abs(blocks).max(axis=2)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(amax.astype(np.float64))).astype(np.int64) - 8   # shared exponent of OCP MX v1.0: floor(log2 max) - emax
    byte = np.where(amax > 0, np.clip(e + 127, 0, 254), 0).astype(np.uint8)
    scale = byte.view(ml.float8_e8m0fnu).astype(np.float32)
    scaled = np.clip(blocks / scale[:, :, None], -448.0, 448.0).astype(np.float32)      # saturating conversion
    codes = scaled.astype(ml.float8_e4m3fn).view(np.uint8)
    return codes.reshape(rows, k), byte


def test_mxfp8_quantizer_matches_a_restatement_over_ml_dtypes(orc):
    ml = pytest.importorskip("ml_dtypes")
    x = orc.gaussian((32, 256), 1.0, 5)
    x[1, 32:64] *= np.float32(1e-12)
    x[2, 64:96] *= np.float32(1e12)
    x[3] = np.abs(x[3]) * np.float32(0.999) + np.float32(1e-3)           # no zeros in the row: every element is a normal code
    codes, sf = orc.spec_mxfp8_quant(x)
    want_codes, want_sf = _mxfp8_with_ml_dtypes(ml, x)
    assert np.array_equal(sf, want_sf)
    assert np.array_equal(codes & 0x7F, want_codes & 0x7F) and np.array_equal((codes >> 7)[(codes & 0x7F) != 0], (want_codes >> 7)[(codes & 0x7F) != 0])


def test_nvfp4_quantizer_matches_a_restatement_over_ml_dtypes(orc):
    ml = pytest.importorskip("ml_dtypes")
    x = orc.gaussian((16, 256), 1.0, 7)
    x[1, 16:32] *= np.float32(1e-3)
    g = np.float32(orc.spec_nvfp4_global_scale(float(np.abs(x).max())))
    assert g == np.float32(np.abs(x).max()) / (np.float32(448.0) * np.float32(6.0))
    packed, sf = orc.spec_nvfp4_quant(x, float(g))
    blocks = x.reshape(16, 16, 16)
    amax = np.abs(blocks).max(axis=2)
    want_sf = np.minimum(amax / (np.float32(6.0) * g), np.float32(448.0)).astype(np.float32).astype(ml.float8_e4m3fn)
    assert np.array_equal(sf, want_sf.view(np.uint8))
    d = g * want_sf.astype(np.float32)
    live = d > 0
    q = np.zeros(blocks.shape, np.uint8)
    q[live] = (blocks[live] / d[live][:, None]).astype(np.float32).astype(ml.float4_e2m1fn).view(np.uint8) & 0xF
    nib = np.stack([packed & 0xF, packed >> 4], axis=2).reshape(16, 16, 16)
    assert np.array_equal(nib[live] & 0x7, q[live] & 0x7)                                                     # magnitudes code for code
    nz = live[:, :, None] & ((nib & 0x7) != 0)
    assert np.array_equal((nib >> 3)[nz], (q >> 3)[nz])                                                       # signs wherever the code is not a zero


def test_nvfp4_packing_matches_compressed_tensors(orc):
    """The byte layout of packed E2M1 codes (which nibble holds the even element, how the 16 codes are numbered) is the one
    NVFP4 checkpoints use: compressed_tensors packs the oracle's decoded values into the oracle's own bytes and unpacks the
    oracle's bytes into the same values; its tensor scale is the reciprocal of the oracle's g = max / (448 * 6)."""
    helpers = pytest.importorskip("compressed_tensors.compressors.nvfp4.helpers")
    from compressed_tensors.quantization.utils.helpers import generate_gparam
    x = orc.gaussian((8, 128), 1.0, 9)
    x[0, :16] = 0.0
    g = float(orc.spec_nvfp4_global_scale(float(np.abs(x).max())))
    packed, _ = orc.spec_nvfp4_quant(x, g)
    nib = np.stack([packed & 0xF, packed >> 4], axis=2).reshape(8, 128)
    vals = orc.e2m1_to_f32(nib)
    repacked = helpers.pack_fp4_to_uint8(torch.from_numpy(vals)).numpy()
    same = (nib & 0x7) != 0                                              # a zero may be packed with either sign
    same_bytes = same.reshape(8, 64, 2).all(axis=2)
    assert np.array_equal(repacked[same_bytes], packed[same_bytes]) and np.array_equal(repacked & 0x77, packed & 0x77)
    unpacked = helpers.unpack_fp4_from_uint8(torch.from_numpy(packed), 8, 128, dtype=torch.float32).numpy()
    assert np.array_equal(unpacked, vals)
    gs = generate_gparam(torch.tensor([float(x.min())]), torch.tensor([float(x.max())]))
    assert abs(float(gs) * g - 1.0) < 1e-6


def test_tiled_scale_factor_layout_is_the_128x4_interleave():
    """The tiled order the GEMMs read scale factors in (tests/gpu_util.py: sf_to_mma_layout, the checker of the quantizers' second
    output) is the block-scaled layout CUTLASS, cuBLASLt and the NVFP4 serving stacks use: rows padded to 128 and columns to 4,
    viewed as [row tile][4][32][column tile][4] and permuted to [row tile][column tile][32][4][4]."""
    from tests.gpu_util import sf_to_mma_layout
    rng = np.random.default_rng(0)
    for rows, cols in ((128, 4), (256, 8), (300, 10), (1, 1), (129, 5)):
        sf = rng.integers(1, 255, size=(rows, cols), dtype=np.uint8)
        mp, kp = -(-rows // 128) * 128, -(-cols // 4) * 4
        padded = np.zeros((mp, kp), np.uint8)
        padded[:rows, :cols] = sf
        want = padded.reshape(mp // 128, 4, 32, kp // 4, 4).transpose(0, 3, 2, 1, 4).ravel()
        assert np.array_equal(sf_to_mma_layout(sf), want)

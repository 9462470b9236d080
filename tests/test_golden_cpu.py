"""The committed golden vectors must be reproduced bit for bit by the oracle as built today."""
import os

import numpy as np

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "quant_golden.npz"))


def test_int8_golden(orc):
    for name, r in (("even", orc.ROUND_HALF_EVEN), ("away", orc.ROUND_HALF_AWAY)):
        q, s = orc.spec_int8_quant_rows(G["int8_x"], r)
        assert np.array_equal(q, G[f"int8_q_{name}"]) and np.array_equal(s, G["int8_scales"])
    assert (G["int8_q_even"] != G["int8_q_away"]).sum() >= 0


def test_fp8_golden(orc):
    am = orc.spec_absmax(G["fp8_x_bf16"])
    assert np.float32(am) == G["fp8_absmax"]
    assert orc.spec_fp8_scale(am) == G["fp8_scale"]
    assert np.array_equal(orc.spec_fp8_quant(G["fp8_x_bf16"], float(G["fp8_scale"])), G["fp8_q"])
    assert np.array_equal(orc.ref_fp8_encode(G["fp8_codec_x"]), G["fp8_codec_ref"])
    assert np.array_equal(orc.ref_fp8_decode(np.arange(256, dtype=np.uint8)), G["fp8_codec_ref_decoded"], equal_nan=True)


def test_int4_golden(orc):
    for grp in (32, 64, 128, 256):
        c, s, z = orc.spec_int4g_quant(G["int4_x"], grp, orc.ROUND_HALF_AWAY)
        assert np.array_equal(c, G[f"int4_codes_g{grp}"])
        assert np.array_equal(s, G[f"int4_scales_g{grp}"])
        assert np.array_equal(z, G[f"int4_zeros_g{grp}"])


def test_block_scaled_golden(orc):
    c, sf = orc.spec_mxfp8_quant(G["mx_x"])
    assert np.array_equal(c, G["mx_codes"]) and np.array_equal(sf, G["mx_sf"])
    p, sf = orc.spec_nvfp4_quant(G["nv_x"], float(G["nv_g"]))
    assert np.array_equal(p, G["nv_packed"]) and np.array_equal(sf, G["nv_sf"])


R = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_golden.npz"))


def _same(a, b):
    a, b = np.asarray(a), np.asarray(b)
    return a.shape == b.shape and a.dtype == b.dtype and np.array_equal(a.view(np.uint8) if a.dtype.kind == "f" else a, b.view(np.uint8) if b.dtype.kind == "f" else b)


def test_reference_quantizer_golden(orc):
    """The reference's own arithmetic (MinMaxQuantizer per group, micro-scaled FP4, the DNN layer's INT8 / INT4 / block-scaled forms, NF4)."""
    x = R["x"]
    sc, zp = orc.ref_minmax_calibrate(x, bits=4, scheme=orc.ASYMMETRIC, group=128)
    assert _same(sc, R["mm_scales"]) and _same(zp, R["mm_zps"])
    codes = orc.minmax_quantize_grouped(x, sc, zp, 128, bits=4, scheme=orc.ASYMMETRIC)
    assert _same(codes, R["mm_codes"]) and _same(orc.ref_minmax_dequantize_grouped(codes, sc, zp, 128), R["mm_back"])
    v = x.ravel()[:1000]
    p, s = orc.ref_microscale_fp4(v, 32)
    assert _same(p, R["ms_packed"]) and _same(s, R["ms_scales"]) and _same(orc.ref_microscale_fp4_dequant(p, s, v.size, 32), R["ms_back"])
    q, s = orc.ref_dnn_int8_quant(x)
    assert _same(q, R["dnn_i8_q"]) and _same(s, R["dnn_i8_scale"])
    q, s = orc.ref_block_int8_quant(v, 64)
    assert _same(q, R["blk_i8_q"]) and _same(s, R["blk_i8_scales"])
    for name, sym in (("sym", True), ("asym", False)):
        p4, s4, z4 = orc.ref_dnn_int4_quant(v, 128, sym)
        assert _same(p4, R[f"dnn_i4_{name}_packed"]) and _same(s4, R[f"dnn_i4_{name}_scales"])
        assert z4 is None or _same(z4, R[f"dnn_i4_{name}_zeros"])
    c, s = orc.ref_dnn_block_scaled_quant(v, 32)
    assert _same(c, R["dnn_bs_codes"]) and _same(s, R["dnn_bs_scales"])
    p, a = orc.ref_nf4_encode(x.ravel(), 64)
    assert _same(p, R["nf4_packed"]) and _same(a, R["nf4_absmax"])


def test_reference_weight_preparation_golden(orc):
    """SmoothQuant scales, GPTQ codes (both schemes) and the fused dequantise + GEMV in the reference's sequential order."""
    acts, w, h = R["sq_acts"], R["sq_w"], R["gptq_h"]
    sq = orc.ref_smooth_scales(orc.ref_smooth_col_absmax(acts), orc.ref_smooth_col_absmax(w), 0.5)
    assert np.abs(sq.view(np.int32).astype(np.int64) - R["sq_scales"].view(np.int32)).max() <= 4      # two powf: a few ulp between C libraries
    for name, sym in (("sym", True), ("asym", False)):
        q, gs, gz = orc.ref_gptq_quantize_layer(w, 12, 16, h, bits=4, symmetric=sym, percdamp=0.01)
        assert _same(q, R[f"gptq_{name}_q"]) and _same(gs, R[f"gptq_{name}_scales"]) and _same(gz, R[f"gptq_{name}_zps"])
    assert _same(orc.ref_dnn_fused_dequant_gemv(R["gemv_w"], R["gemv_scales"], R["gemv_x"], 6, 256, 64, 4), R["gemv_y"])

"""Generates tests/golden/quant_golden.npz (the formats of the benchmark configurations) and tests/golden/ref_golden.npz (the
reference's own arithmetic: quantizers in its parameter types, NF4, GPTQ, SmoothQuant, the fused GEMV) from the CPU oracle on
small seeded inputs.

Run from the repository root:  python tests/golden/make_golden.py
The reference is a Rust workspace that cannot be built or imported here, so these vectors come from
the C restatement (oracle/oxq_oracle.c), which is itself pinned by the reference's known-answer
tests (tests/test_oracle_kats.py).  The file pins the oracle against accidental change and gives the
GPU tests fixed vectors that do not depend on the oracle being rebuilt identically.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402


def main():
    out = {}
    w = orc.gaussian((24, 512), 0.02, 0)
    w[3, 7] = np.float32(0.0)
    out["int8_x"] = w
    for name, r in (("even", orc.ROUND_HALF_EVEN), ("away", orc.ROUND_HALF_AWAY)):
        q, s = orc.spec_int8_quant_rows(w, r)
        out[f"int8_q_{name}"] = q
        out["int8_scales"] = s
    a = orc.gaussian((32, 256), 1.0, 1)
    ab = orc.f32_to_bf16_bits(a)
    out["fp8_x_bf16"] = ab
    am = orc.spec_absmax(ab)
    sc = orc.spec_fp8_scale(am)
    out["fp8_absmax"] = np.float32(am)
    out["fp8_scale"] = np.float32(sc)
    out["fp8_q"] = orc.spec_fp8_quant(ab, sc)
    codec_in = np.concatenate([orc.gaussian(2048, 40.0, 2), np.array([0.0, -0.0, 1.9375, 256.0, 2.0 ** -7, 448.0, -1000.0], np.float32)])
    out["fp8_codec_x"] = codec_in
    out["fp8_codec_ref"] = orc.ref_fp8_encode(codec_in)
    out["fp8_codec_ref_decoded"] = orc.ref_fp8_decode(np.arange(256, dtype=np.uint8))
    g = orc.gaussian((9, 768), 0.02, 3)
    out["int4_x"] = g
    for grp in (32, 64, 128, 256):
        c, s, z = orc.spec_int4g_quant(g, grp, orc.ROUND_HALF_AWAY)
        out[f"int4_codes_g{grp}"] = c
        out[f"int4_scales_g{grp}"] = s
        out[f"int4_zeros_g{grp}"] = z
    m = orc.gaussian((16, 256), 1.0, 5)
    m[0, :32] = 0.0
    m[1, 32:64] *= np.float32(1e-20)
    m[2, 64:96] *= np.float32(1e20)
    out["mx_x"] = m
    c, sf = orc.spec_mxfp8_quant(m)
    out["mx_codes"], out["mx_sf"] = c, sf
    n = orc.gaussian((16, 256), 1.0, 7)
    n[0, :16] = 0.0
    n[1, 16:32] *= np.float32(1e-6)
    out["nv_x"] = n
    gs = orc.spec_nvfp4_global_scale(orc.spec_absmax(n))
    p, sf = orc.spec_nvfp4_quant(n, gs)
    out["nv_g"], out["nv_packed"], out["nv_sf"] = np.float32(gs), p, sf
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "quant_golden.npz"), **out)
    print("wrote", len(out), "arrays")
    ref_main()


def ref_main():
    """The reference-defined forms (every function here restates reference lines and is pinned by its known-answer tests)."""
    out = {}
    x = orc.gaussian((4, 256), 0.05, 11)
    x[1, 128:] = 0.0
    x[2, 5] = np.float32(-1e-30)
    out["x"] = x
    # MinMaxQuantizer per group, asymmetric, f32 scales and i32 zero-points (minmax.rs:146-167, :226-324)
    sc, zp = orc.ref_minmax_calibrate(x, bits=4, scheme=orc.ASYMMETRIC, group=128)
    out["mm_scales"], out["mm_zps"] = sc, zp
    out["mm_codes"] = orc.minmax_quantize_grouped(x, sc, zp, 128, bits=4, scheme=orc.ASYMMETRIC)
    out["mm_back"] = orc.ref_minmax_dequantize_grouped(out["mm_codes"], sc, zp, 128)
    # MicroScalingQuantizer::quantize_fp4 (fp4_fp6_ops.rs:763-897), ragged length
    v = x.ravel()[:1000]
    p, s = orc.ref_microscale_fp4(v, 32)
    out["ms_packed"], out["ms_scales"] = p, s
    out["ms_back"] = orc.ref_microscale_fp4_dequant(p, s, v.size, 32)
    # oxicuda-dnn: per-tensor INT8, per-block INT8, INT4 (both schemes), block-scaled (int8_quantize.rs, int4_quantize.rs, block_scale.rs)
    out["dnn_i8_q"], out["dnn_i8_scale"] = orc.ref_dnn_int8_quant(x)
    out["blk_i8_q"], out["blk_i8_scales"] = orc.ref_block_int8_quant(v, 64)
    for name, sym in (("sym", True), ("asym", False)):
        p4, s4, z4 = orc.ref_dnn_int4_quant(v, 128, sym)
        out[f"dnn_i4_{name}_packed"], out[f"dnn_i4_{name}_scales"] = p4, s4
        if z4 is not None:
            out[f"dnn_i4_{name}_zeros"] = z4
    out["dnn_bs_codes"], out["dnn_bs_scales"] = orc.ref_dnn_block_scaled_quant(v, 32)
    # Nf4Quantizer (nf4.rs:93-155)
    out["nf4_packed"], out["nf4_absmax"] = orc.ref_nf4_encode(x.ravel(), 64)
    # SmoothQuantMigrator (smooth_quant.rs:84-254) and GptqQuantizer (gptq.rs:133-257) on a 12 x 16 layer
    acts = orc.gaussian((10, 16), 1.0, 12)
    acts[:, 3] *= 30.0
    w = orc.gaussian((12, 16), 0.1, 13)
    out["sq_acts"], out["sq_w"] = acts, w
    out["sq_scales"] = orc.ref_smooth_scales(orc.ref_smooth_col_absmax(acts), orc.ref_smooth_col_absmax(w), 0.5)
    h = (acts.T.astype(np.float64) @ acts.astype(np.float64) / 10.0).astype(np.float32)
    out["gptq_h"] = h
    for name, sym in (("sym", True), ("asym", False)):
        q, gs, gz = orc.ref_gptq_quantize_layer(w, 12, 16, h, bits=4, symmetric=sym, percdamp=0.01)
        out[f"gptq_{name}_q"], out[f"gptq_{name}_scales"], out[f"gptq_{name}_zps"] = q, gs, gz
    # dnn_fused_dequant_gemv_f32 (gptq_awq.rs:867-994), sequential order
    rng = np.random.Generator(np.random.Philox(14))
    gw = rng.integers(0, 2 ** 32, size=(6, 32), dtype=np.uint64).astype(np.uint32)
    gsc = (0.01 + 0.02 * rng.random((6, 4))).astype(np.float32)
    gx = orc.gaussian((1, 256), 1.0, 15).ravel()
    out["gemv_w"], out["gemv_scales"], out["gemv_x"] = gw, gsc, gx
    out["gemv_y"] = orc.ref_dnn_fused_dequant_gemv(gw, gsc, gx, 6, 256, 64, 4)
    np.savez_compressed(os.path.join(ROOT, "tests", "golden", "ref_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()

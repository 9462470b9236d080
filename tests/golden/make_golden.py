"""Generates tests/golden/quant_golden.npz from the CPU oracle on small seeded inputs.

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


if __name__ == "__main__":
    main()

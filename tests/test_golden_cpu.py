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

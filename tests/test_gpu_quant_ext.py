"""GPU parity of the quantizers next to the hot path (per-tensor INT8, per-block INT8, NF4) against the oracle's
restatement of the reference: codes and scales bit-exact."""
import numpy as np
import pytest
import torch

from gpu_util import to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from oxicuda_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle as _orc
    return _orc


def _bf16_round(x):
    return torch.from_numpy(x).to(torch.bfloat16)


@pytest.mark.parametrize("n", [8, 1000, 4099, 1 << 20])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_quantize_to_int8_tensor(ops, orc, n, dtype):
    x = orc.gaussian((1, n), 1.0, 11).ravel()
    if dtype == "bf16":
        xb = _bf16_round(x)
        x = xb.float().numpy()
        xd = xb.cuda()
    else:
        xd = to_dev(x)
    q, sc = ops.quantize_to_int8(xd)
    q_ref, s_ref = orc.ref_dnn_int8_quant(x)
    assert sc.cpu().numpy()[0] == s_ref[0]
    assert (q.cpu().numpy().ravel() == q_ref).all()
    y = ops.dequantize_from_int8(q, sc).cpu().numpy().ravel()
    assert (y == orc.ref_dnn_int8_dequant(q_ref, s_ref[0])).all()


def test_quantize_to_int8_edges(ops, orc):
    q, sc = ops.quantize_to_int8(torch.zeros(64, device="cuda"))
    assert sc.item() == np.float32(1e-12) and int(q.abs().max()) == 0
    x = np.array([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 127.0, -127.0], np.float32)      # scale 1: ties go to even
    q, sc = ops.quantize_to_int8(to_dev(x))
    assert sc.item() == 1.0 and q.cpu().tolist() == [0, 2, 2, 0, -2, -2, 127, -127]
    q, sc = ops.quantize_to_int8(torch.empty(0, device="cuda"))                       # empty tensor: Ok(())
    assert q.numel() == 0


@pytest.mark.parametrize("n,block", [(256, 64), (100, 64), (300, 100), (4, 4), (1 << 18, 128), (12345, 37)])
def test_block_int8(ops, orc, n, block):
    x = orc.gaussian((1, n), 3.0, 5).ravel()
    q, sc = ops.block_int8_quant(to_dev(x), block)
    q_ref, s_ref = orc.ref_block_int8_quant(x, block)
    assert (sc.cpu().numpy() == s_ref).all()
    assert (q.cpu().numpy() == q_ref).all()
    y = ops.block_int8_dequant(q, sc, block).cpu().numpy()
    assert (y == orc.ref_block_int8_dequant(q_ref, s_ref, block)).all()


def test_block_int8_reference_cases(ops, orc):  # crates/oxicuda-dnn/src/quantize/int8_quantize.rs:561-577
    x = np.array([1e30, -1e30, 0.0, 1e30], np.float32)
    q, sc = ops.block_int8_quant(to_dev(x), 4)
    assert q.cpu().tolist() == [127, -127, 0, 127]
    d = ops.block_int8_dequant(q, sc, 4).cpu().numpy()
    assert d[0] > 0 and d[1] < 0 and d[2] == 0.0
    q, sc = ops.block_int8_quant(torch.zeros(8, device="cuda"), 4)
    assert sc.cpu().tolist() == [1.0, 1.0]
    with pytest.raises(ValueError):
        ops.block_int8_quant(torch.zeros(8, device="cuda"), 0)


@pytest.mark.parametrize("n,block", [(128, 64), (64 * 1000, 64), (1 << 20, 64), (4096, 32), (8192, 128), (4096, 256), (600, 6), (900, 100)])
def test_nf4(ops, orc, n, block):
    x = orc.gaussian((1, n), 0.7, 9).ravel()
    x[::97] = 0.0
    packed, am = ops.nf4_quant(to_dev(x), block)
    p_ref, a_ref = orc.ref_nf4_encode(x, block)
    assert (am.cpu().numpy() == a_ref).all()
    assert (packed.cpu().numpy() == p_ref).all()
    y = ops.nf4_dequant(packed, am, block).cpu().numpy()
    assert (y == orc.ref_nf4_decode(p_ref, a_ref, block)).all()


def test_nf4_reference_cases(ops, orc):  # crates/oxicuda-quant/src/scheme/nf4.rs:243-310
    from oxicuda_b200.errors import QuantError
    t = (np.arange(128, dtype=np.float32) / np.float32(64.0)) - np.float32(1.0)
    packed, am = ops.nf4_quant(to_dev(t), 64)
    assert packed.numel() == 64 and am.numel() == 2
    dec = ops.nf4_dequant(packed, am, 64).cpu().numpy()
    assert float(((t - dec) ** 2).mean()) < 0.01
    packed, am = ops.nf4_quant(torch.zeros(64, device="cuda"), 64)
    assert am.item() == np.float32(1e-8) and (packed.cpu().numpy() == 0x77).all()
    # every midpoint between two levels, and values one ulp either side: ties take the lower index
    lut = orc.nf4_levels()
    mids = ((lut[:-1] + lut[1:]) / np.float32(2.0)).astype(np.float32)
    probe = np.concatenate([mids, np.nextafter(mids, np.float32(2.0)), np.nextafter(mids, np.float32(-2.0)), lut, [1.0] * 3]).astype(np.float32)
    assert probe.size == 64
    packed, am = ops.nf4_quant(to_dev(probe), 64)
    p_ref, _ = orc.ref_nf4_encode(probe, 64)
    assert (packed.cpu().numpy() == p_ref).all()
    with pytest.raises(QuantError) as e:
        ops.nf4_quant(torch.full((65,), 0.5, device="cuda"), 64)
    assert e.value.variant == "GroupSizeMismatch"
    with pytest.raises(QuantError) as e:
        ops.nf4_dequant(torch.zeros(32, dtype=torch.uint8, device="cuda"), torch.ones(5, device="cuda"), 64)
    assert e.value.variant == "DimensionMismatch"
    with pytest.raises(QuantError) as e:
        ops.nf4_quant(torch.empty(0, device="cuda"), 64)
    assert e.value.variant == "EmptyInput"


# ---- SmoothQuant migration --------------------------------------------------------------------------

def _ulp_diff(a, b):
    return np.abs(a.view(np.int32).astype(np.int64) - b.view(np.int32).astype(np.int64))


@pytest.mark.parametrize("shape", [(3, 4, 2), (512, 1024, 256), (100, 1030, 77), (2048, 4096, 4096)])
@pytest.mark.parametrize("alpha", [0.5, 0.8])
def test_smooth_quant_layer(ops, orc, shape, alpha):
    n_tok, n_ch, n_out = shape
    acts = orc.gaussian((n_tok, n_ch), 1.0, 1)
    acts[:, ::17] *= 40.0                                             # outlier channels
    w = orc.gaussian((n_out, n_ch), 0.05, 2)
    mig = ops.SmoothQuantMigrator(alpha)
    a_d, w_d = to_dev(acts.copy()), to_dev(w.copy())
    st_a, st_w = mig.compute_act_stats(a_d), mig.compute_weight_stats(w_d)
    assert (st_a.cpu().numpy() == orc.ref_smooth_col_absmax(acts)).all()                 # bit-exact
    assert (st_w.cpu().numpy() == orc.ref_smooth_col_absmax(w)).all()
    sc = mig.compute_migration_scales(st_a, st_w)
    sc_ref = orc.ref_smooth_scales(orc.ref_smooth_col_absmax(acts), orc.ref_smooth_col_absmax(w), alpha)
    assert _ulp_diff(sc.cpu().numpy(), sc_ref).max() <= 4                                 # two powf and a division: a few ulp between libms
    # with the same scales the smoothed matrices are bit-exact (one IEEE division / multiplication per element)
    sc_h = sc.cpu().numpy()
    mig.smooth_activations(a_d, sc)
    mig.smooth_weights(w_d, sc)
    assert (a_d.cpu().numpy() == orc.ref_smooth_activations(acts, sc_h)).all()
    assert (w_d.cpu().numpy() == orc.ref_smooth_weights(w, sc_h)).all()
    if n_tok * n_out <= 512 * 256:                                                        # the layer output is preserved
        y0 = acts.astype(np.float64) @ w.astype(np.float64).T
        y1 = a_d.cpu().numpy().astype(np.float64) @ w_d.cpu().numpy().astype(np.float64).T
        assert np.abs(y0 - y1).max() <= 1e-4 * np.abs(y0).max()


def test_smooth_quant_reference_cases(ops, orc):  # crates/oxicuda-quant/src/scheme/smooth_quant.rs:311-440
    from oxicuda_b200.errors import QuantError
    dev = lambda v: to_dev(np.array(v, np.float32))  # noqa: E731
    assert np.allclose(ops.SmoothQuantMigrator(0.5).compute_migration_scales(dev([4.0, 1.0, 9.0]), dev([1.0, 4.0, 1.0])).cpu().numpy(), [2.0, 0.5, 3.0], atol=1e-5)
    assert np.allclose(ops.SmoothQuantMigrator(1.0).compute_migration_scales(dev([2.0, 5.0]), dev([3.0, 7.0])).cpu().numpy(), [2.0, 5.0], atol=1e-5)
    assert np.allclose(ops.SmoothQuantMigrator(0.0).compute_migration_scales(dev([4.0, 1.0]), dev([2.0, 5.0])).cpu().numpy(), [0.5, 0.2], atol=1e-5)
    assert ops.SmoothQuantMigrator.compute_act_stats(dev([[1.0, -5.0, 2.0], [-3.0, 4.0, 1.0]])).cpu().tolist() == [3.0, 5.0, 2.0]
    assert ops.SmoothQuantMigrator.compute_weight_stats(dev([[0.5, -2.0, 1.0], [-1.5, 0.3, 3.0]])).cpu().tolist() == [1.5, 2.0, 3.0]
    with pytest.raises(QuantError) as e:
        ops.SmoothQuantMigrator(0.5).compute_migration_scales(dev([1.0] * 3), dev([1.0] * 4))
    assert e.value.variant == "DimensionMismatch"
    with pytest.raises(QuantError) as e:
        ops.SmoothQuantMigrator(0.5).compute_migration_scales(torch.empty(0, device="cuda"), torch.empty(0, device="cuda"))
    assert e.value.variant == "EmptyInput"
    acts = dev([[100.0, 1.0], [-100.0, 1.0], [100.0, -1.0], [-100.0, -1.0]])
    w = dev([[0.5, 0.5], [-0.5, 0.5]])
    sc = ops.SmoothQuantMigrator(0.5).smooth_layer(acts, w)
    a = acts.cpu().numpy()
    assert np.abs(a[:, 0]).max() / np.abs(a[:, 1]).max() < 100.0 and sc[0].item() > 1.0


# ---- RMSNorm fused with the per-row INT8 quantizer -------------------------------------------------------

@pytest.mark.parametrize("shape", [(1, 8), (7, 4096), (64, 8192), (300, 1000), (5, 16384)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_rmsnorm_int8_rows(ops, orc, shape, dtype):
    rows, cols = shape
    x = orc.gaussian((rows, cols), 2.0, 21)
    w = (1.0 + 0.1 * orc.gaussian((1, cols), 1.0, 22)).ravel().astype(np.float32)
    if dtype == "bf16":
        xb = _bf16_round(x)
        x = xb.float().numpy()
        xd = xb.cuda()
    else:
        xd = to_dev(x)
    q, sc, y = ops.rmsnorm_int8_quant_rows(xd, to_dev(w), 1e-5, want_normed=True)
    # Integer codes are held bit-exact.  The oracle takes the row's sum of squares in the kernel's order (a fixed tree of
    # fused multiply-adds and butterfly sums, restated on the CPU) and is the reference's arithmetic from there on; against
    # the reference's left-to-right sum it agrees to a few ulp of inv_rms, which the second block checks.
    y_ref = orc.spec_rms_norm_blocked(x, w, 1e-5)
    q_ref, s_ref = orc.spec_int8_quant_rows(y_ref, orc.ROUND_HALF_EVEN)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), q_ref)
    yg = y.float().cpu().numpy()
    if dtype == "f32":
        assert np.array_equal(yg.view(np.uint32), y_ref.view(np.uint32))
    else:
        assert np.array_equal(orc.f32_to_bf16_bits(yg), orc.f32_to_bf16_bits(y_ref))
    y_seq = orc.ref_rms_norm(x, w, 1e-5)                                   # the reference's sequential sum of squares
    assert np.abs(y_ref - y_seq).max() <= 1e-5 * np.abs(y_seq).max()


def test_rmsnorm_reference_cases(ops, orc):  # crates/oxicuda-lm/src/layer/norm.rs:186-227
    from oxicuda_b200.errors import OxqError
    x = to_dev(np.array([[3.0, 4.0, 0.0, 0.0, 0.0, 0.0, 0.0, 0.0]], np.float32))     # rms = sqrt(25 / 8)
    q, sc, y = ops.rmsnorm_int8_quant_rows(x, torch.ones(8, device="cuda"), 1e-8, want_normed=True)
    rms = np.sqrt(25.0 / 8.0)
    assert np.allclose(y.cpu().numpy()[0, :3], [3.0 / rms, 4.0 / rms, 0.0], atol=1e-5)
    assert q.cpu().tolist()[0][:3] == [95, 127, 0]
    with pytest.raises(OxqError):
        ops.rmsnorm_int8_quant_rows(x, torch.ones(4, device="cuda"))


def _e4m3_half_ulp(v):
    """Half the spacing of the E4M3 grid around |v| (subnormal spacing 2^-9 below 2^-6; the grid ends at 448)."""
    a = np.minimum(np.abs(v), 448.0)
    e = np.floor(np.log2(np.maximum(a, 2.0 ** -6)))
    return 0.5 * 2.0 ** (e - 3)


def _check_fp8_codes(orc, q, want_f64, what):
    """The code is the nearest E4M3 value of the exact quotient, or its neighbour where the kernel's f32 value sat within a
    few ulp of a rounding boundary."""
    dec = orc.e4m3_to_f32(q.cpu().numpy().ravel()).astype(np.float64)
    want = np.clip(want_f64.ravel(), -448.0, 448.0)
    err = np.abs(dec - want)
    hu = _e4m3_half_ulp(want)
    assert (err <= hu * 1.001 + 1e-12).all(), f"{what}: max excess {(err - hu).max()}"
    exact = orc.e4m3_to_f32(orc.spec_fp8_quant(want.astype(np.float32), 1.0)).astype(np.float64)
    assert (dec != exact).mean() <= 2e-3, what


@pytest.mark.parametrize("shape", [(1, 8), (7, 4096), (64, 8192), (300, 1000)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_rmsnorm_fp8_rows(ops, orc, shape, dtype):
    rows, cols = shape
    x = orc.gaussian((rows, cols), 2.0, 31)
    w = (1.0 + 0.1 * orc.gaussian((1, cols), 1.0, 32)).ravel().astype(np.float32)
    if dtype == "bf16":
        xb = _bf16_round(x)
        x = xb.float().numpy()
        xd = xb.cuda()
    else:
        xd = to_dev(x)
    scale = np.float32(4.0 / 448.0)                                       # a calibrated scale; a few values saturate
    q = ops.rmsnorm_fp8_quant_rows(xd, to_dev(w), to_dev(np.array([scale], np.float32)), 1e-5)
    y_ref = orc.ref_rms_norm(x, w, 1e-5).astype(np.float64)
    _check_fp8_codes(orc, q, y_ref / np.float64(scale), f"rmsnorm+fp8 {shape} {dtype}")


@pytest.mark.parametrize("n", [8, 1000, 4099, 2048 * 3584])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_silu_gate_fp8(ops, orc, n, dtype):
    g = orc.gaussian((n,), 2.0, 41)
    u = orc.gaussian((n,), 1.0, 42)
    if dtype == "bf16":
        gb, ub = _bf16_round(g), _bf16_round(u)
        g, u = gb.float().numpy(), ub.float().numpy()
        gd, ud = gb.cuda(), ub.cuda()
    else:
        gd, ud = to_dev(g), to_dev(u)
    scale = np.float32(6.0 / 448.0)
    q = ops.silu_gate_fp8_quant(gd, ud, to_dev(np.array([scale], np.float32)))
    g64, u64 = g.astype(np.float64), u.astype(np.float64)
    _check_fp8_codes(orc, q, g64 / (1.0 + np.exp(-g64)) * u64 / np.float64(scale), f"silu_gate+fp8 {n} {dtype}")
    if n <= 4099:                                                          # and against the reference's own f32 silu_gate
        h = orc.ref_silu_mul(g, u).astype(np.float64)
        _check_fp8_codes(orc, q, h / np.float64(scale), f"silu_gate+fp8 vs reference f32 {n} {dtype}")


def test_dnn_fp8_names(ops, orc):
    """quantize_to_fp8 / dequantize_from_fp8 of the reference's DNN layer: scale = absmax / 448 in a one-element buffer."""
    x = orc.gaussian((1000,), 1.0, 51)
    q, scale = ops.quantize_to_fp8(to_dev(x))
    assert scale.numel() == 1 and float(scale[0]) == np.float32(np.abs(x).max()) / np.float32(448.0)
    q2, _ = ops.fp8_quant_dynamic(to_dev(x))
    assert torch.equal(q, q2)
    y = ops.dequantize_from_fp8(q, scale)
    assert np.allclose(y.cpu().numpy(), x, atol=float(scale[0]) * 16.0)
    buf = torch.zeros(1, device="cuda")
    ops.quantize_to_fp8(to_dev(x), scale=buf)
    assert float(buf[0]) == float(scale[0])


@pytest.mark.parametrize("mnk", [(1, 16, 128), (1, 4096, 4096), (8, 6144, 4096), (3, 1000, 1024), (5, 4100, 14336), (8, 40, 128)])
@pytest.mark.parametrize("block", [64, 128])
def test_gemm_nf4(ops, orc, mnk, block):
    """The fused NF4 GEMV against dequantise (the reference's decode) then an f64 product; tolerance as for the other GEMMs."""
    m, n, k = mnk
    w = orc.gaussian((n, k), 0.02, 61)
    xb = _bf16_round(orc.gaussian((m, k), 1.0, 62))
    packed, am = ops.nf4_quant(to_dev(w.ravel()), block)
    rp, ra = orc.ref_nf4_encode(w.ravel(), block)
    assert np.array_equal(packed.cpu().numpy(), rp) and np.array_equal(am.cpu().numpy(), ra)
    y = ops.gemm_nf4(xb.cuda(), packed, am, n, block)
    torch.cuda.synchronize()
    wd = orc.ref_nf4_decode(rp, ra, block).reshape(n, k).astype(np.float64)
    ref = xb.float().numpy().astype(np.float64) @ wd.T
    got = y.float().cpu().numpy()
    assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max(), f"nf4 gemv {mnk} block {block}: {np.abs(got - ref).max()} vs {np.abs(ref).max()}"


def test_gemm_nf4_errors(ops):
    from oxicuda_b200.errors import OxqError
    x = torch.zeros((9, 128), dtype=torch.bfloat16, device="cuda")
    packed = torch.zeros(16 * 64, dtype=torch.uint8, device="cuda")
    am = torch.ones(32, device="cuda")
    with pytest.raises(OxqError):
        ops.gemm_nf4(x, packed, am, 16, 64)                               # more than 8 batch rows
    with pytest.raises(OxqError):
        ops.gemm_nf4(x[:2], packed, am, 16, 96)                           # block not a multiple of 64

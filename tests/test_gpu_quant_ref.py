"""GPU parity of the quantizers that keep the reference's own parameter types (f32 scales and i32 zero-points for
INT4 per group; f32 block scales and the floor-type E2M1 encoder for micro-scaled FP4; the DNN layer's INT4 and
block-scaled kernels) against the oracle's literal restatement of the reference: every output bit-exact."""
import numpy as np
import pytest
import torch

from gpu_util import to_dev, u32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from oxicuda_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle as _orc
    return _orc


# ---------------------------------------------------------------- MinMaxQuantizer per group, asymmetric (minmax.rs:146-167, :226-232)

@pytest.mark.parametrize("rows,k,group", [(8, 256, 128), (64, 4096, 128), (3, 96, 32), (5, 512, 64), (16, 1024, 256), (1024, 4096, 128)])
@pytest.mark.parametrize("rounding", [0, 1])
def test_int4g_f32_matches_minmax_quantizer(ops, orc, rows, k, group, rounding):
    x = orc.gaussian((rows, k), 0.02, 3)
    x[0, :group] = 0.0                                            # an all-zero group: range floor 1e-8
    x[-1, -1] = np.nan                                            # a NaN is skipped by the scan and gets code 0
    codes, scales, zps = ops.int4g_quant_pack_f32(to_dev(x), group, rounding)
    s_ref, z_ref = orc.ref_minmax_calibrate(x, bits=4, scheme=orc.ASYMMETRIC, group=group)
    assert np.array_equal(scales.cpu().numpy().ravel().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(zps.cpu().numpy().ravel(), z_ref)
    q_ref = orc.minmax_quantize_grouped(x, s_ref, z_ref, group, bits=4, scheme=orc.ASYMMETRIC, rounding=rounding)
    assert np.array_equal(orc.unpack_uint4(u32(codes).ravel()).astype(np.int32), q_ref)
    y = ops.int4g_dequant_f32(codes, scales, zps, rows, k, group).cpu().numpy().ravel()
    y_ref = orc.ref_minmax_dequantize_grouped(q_ref, s_ref, z_ref, group)
    assert np.array_equal(y.view(np.uint32), y_ref.view(np.uint32))


def test_int4g_f32_reference_known_answers(ops, orc):
    """The reference's own asymmetric known answers (minmax.rs:350-359): zero point of a [0, 15] ramp is 0 with scale 1,
    and codes stay in [0, 15]."""
    x = np.tile(np.arange(16, dtype=np.float32), 2).reshape(1, 32)
    codes, scales, zps = ops.int4g_quant_pack_f32(to_dev(x), 32)
    assert scales.item() == 1.0 and zps.item() == 0
    assert orc.unpack_uint4(u32(codes).ravel()).tolist() == list(range(16)) * 2
    x = (np.arange(32, dtype=np.float32) - 10.0).reshape(1, 32)
    codes, scales, zps = ops.int4g_quant_pack_f32(to_dev(x), 32)
    q = orc.unpack_uint4(u32(codes).ravel())
    assert q.min() >= 0 and q.max() <= 15


def test_int4g_f32_errors(ops):
    from oxicuda_b200.errors import BlasError, QuantError
    with pytest.raises(QuantError) as e:
        ops.int4g_quant_pack_f32(torch.zeros((2, 100), device="cuda"), 32)
    assert e.value.variant == "GroupSizeMismatch"
    with pytest.raises(QuantError) as e:
        ops.int4g_quant_pack_f32(torch.zeros((0, 128), device="cuda"), 128)
    assert e.value.variant == "EmptyInput"
    with pytest.raises(BlasError):
        ops.int4g_quant_pack_f32(torch.zeros((2, 96), device="cuda"), 48)
    x = torch.zeros((1, 128), device="cuda")
    x[0, 5] = float("inf")                                        # calibrate returns InvalidScale (minmax.rs:234-236)
    with pytest.raises(QuantError) as e:
        ops.int4g_quant_pack_f32(x, 128)
    assert e.value.variant == "InvalidScale"


# ---------------------------------------------------------------- MicroScalingQuantizer::quantize_fp4 (fp4_fp6_ops.rs:763-897)

@pytest.mark.parametrize("n,block", [(32, 32), (4096, 32), (1000, 32), (33, 32), (1 << 20, 64), (12345, 128), (7, 32), (129, 64)])
def test_fp4_microscale_matches_reference(ops, orc, n, block):
    x = orc.gaussian((1, n), 1.0, 21).ravel()
    if n >= 64:
        x[32:64] = 0.0                                            # all-zero block: scale 1
        x[3] = -1e-30                                             # tiny negative: sign bit with magnitude code 0
    packed, scales = ops.fp4_microscale_quant(to_dev(x), block)
    p_ref, s_ref = orc.ref_microscale_fp4(x, block)
    assert np.array_equal(scales.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(packed.cpu().numpy(), p_ref)
    y = ops.fp4_microscale_dequant(packed, scales, n, block).cpu().numpy()
    assert np.array_equal(y.view(np.uint32), orc.ref_microscale_fp4_dequant(p_ref, s_ref, n, block).view(np.uint32))


def test_fp4_microscale_interval_boundaries(ops, orc):
    """Every decision point of the floor-type E2M1 encoder and its two f32 neighbours, both signs, at scale 1
    (block maximum 6): the comparison form used on the device against the reference's log2 / powf form."""
    pts = [0.0, 0.25, 0.5, 0.75, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, 5.9999995, 7.0, 100.0, 1e-20]
    vals = []
    for p in pts:
        f = np.float32(p)
        vals += [f, np.nextafter(f, np.float32(np.inf)), np.nextafter(f, np.float32(-np.inf))]
    vals = np.array(vals + [-v for v in vals], np.float32)
    vals = np.clip(vals, -6.0, 6.0)                               # keep the block maximum at 6 so that the scale is exactly 1
    x = np.zeros(((vals.size + 31) // 32) * 32, np.float32)
    x[: vals.size] = vals
    x[31::32] = 6.0
    packed, scales = ops.fp4_microscale_quant(to_dev(x), 32)
    p_ref, s_ref = orc.ref_microscale_fp4(x, 32)
    assert (s_ref == 1.0).all() and np.array_equal(scales.cpu().numpy(), s_ref)
    assert np.array_equal(packed.cpu().numpy(), p_ref)


def test_fp4_microscale_roundtrip_within_tolerance(ops, orc):
    """The reference's round-trip bound (fp4_fp6_ops.rs:1681-1697): error at most half the largest grid step times the scale."""
    x = orc.gaussian((1, 4096), 1.0, 4).ravel()
    packed, scales = ops.fp4_microscale_quant(to_dev(x), 32)
    y = ops.fp4_microscale_dequant(packed, scales, x.size, 32).cpu().numpy()
    s = np.repeat(scales.cpu().numpy(), 32)
    assert (np.abs(y - x) <= 2.0 * s + 1e-6).all()                # floor-type codes: at most one grid step (2 at the top) below


def test_fp4_microscale_errors(ops):
    from oxicuda_b200.errors import BlasError
    with pytest.raises(BlasError):
        ops.fp4_microscale_quant(torch.zeros(64, device="cuda"), 16)
    p, s = ops.fp4_microscale_quant(torch.zeros(0, device="cuda"), 32)
    assert p.numel() == 0 and s.numel() == 0


# ---------------------------------------------------------------- DNN quantize_to_int4 (int4_quantize.rs:132-218)

@pytest.mark.parametrize("n,group", [(256, 32), (1000, 128), (33, 32), (1 << 18, 128), (4097, 100)])
@pytest.mark.parametrize("symmetric", [True, False])
def test_dnn_quantize_to_int4(ops, orc, n, group, symmetric):
    x = orc.gaussian((1, n), 0.5, 9).ravel()
    cfg = ops.Int4QuantConfig(group, symmetric)
    out = torch.zeros(cfg.packed_bytes(n), dtype=torch.uint8, device="cuda")
    sc = torch.zeros(cfg.num_groups(n), device="cuda")
    zs = torch.zeros(cfg.num_groups(n), device="cuda")
    ops.quantize_to_int4(to_dev(x), out, sc, zs, n, cfg)
    p_ref, s_ref, z_ref = orc.ref_dnn_int4_quant(x, group, symmetric)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    if not symmetric:
        assert np.array_equal(zs.cpu().numpy().view(np.uint32), z_ref.view(np.uint32))
    assert np.array_equal(out.cpu().numpy(), p_ref)
    y = torch.zeros(n, device="cuda")
    ops.dequantize_int4(out, sc, y, n, cfg)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), orc.ref_dnn_int4_dequant(p_ref, s_ref, n, group, symmetric).view(np.uint32))


def test_dnn_int4_errors(ops):
    from oxicuda_b200.errors import DnnError
    with pytest.raises(DnnError) as e:
        ops.Int4QuantConfig(0, True)
    assert e.value.variant == "InvalidArgument"
    cfg = ops.Int4QuantConfig(32, True)
    x = torch.zeros(64, device="cuda")
    with pytest.raises(DnnError) as e:                            # BufferTooSmall counts bytes in the DNN layer
        ops.quantize_to_int4(x, torch.zeros(16, dtype=torch.uint8, device="cuda"), torch.zeros(2, device="cuda"), None, 64, cfg)
    assert e.value.variant == "BufferTooSmall" and e.value.expected == 32 and e.value.actual == 16
    with pytest.raises(DnnError) as e:
        ops.quantize_to_int4(x, torch.zeros(32, dtype=torch.uint8, device="cuda"), torch.zeros(1, device="cuda"), None, 64, cfg)
    assert e.value.expected == 8 and e.value.actual == 4
    ops.quantize_to_int4(x, torch.zeros(0, dtype=torch.uint8, device="cuda"), torch.zeros(0, device="cuda"), None, 0, cfg)   # n == 0: Ok(())


# ---------------------------------------------------------------- DNN quantize_block_scaled (block_scale.rs:53-140)

@pytest.mark.parametrize("n,block", [(256, 32), (1000, 16), (33, 32), (1 << 18, 64), (5000, 1024)])
@pytest.mark.parametrize("dtype", ["f32", "bf16"])
def test_dnn_quantize_block_scaled(ops, orc, n, block, dtype):
    x = orc.gaussian((1, n), 2.0, 13).ravel()
    if n >= 64:
        x[32:64] = 0.0                                            # all-zero block: scale floor 1e-12
    if dtype == "bf16":
        xb = torch.from_numpy(x).to(torch.bfloat16)
        x = xb.float().numpy()
        xd = xb.cuda()
    else:
        xd = to_dev(x)
    out = torch.zeros(n, dtype=torch.uint8, device="cuda")
    sc = torch.zeros(-(-n // block), device="cuda")
    ops.quantize_block_scaled(ops.TensorDesc(xd), out, sc, block)
    q_ref, s_ref = orc.ref_dnn_block_scaled_quant(x, block)
    assert np.array_equal(sc.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    assert np.array_equal(out.cpu().numpy(), q_ref)
    assert int(out.max()) <= 12


def test_dnn_block_scaled_errors(ops):
    from oxicuda_b200.errors import DnnError
    x = ops.TensorDesc(torch.zeros(64, device="cuda"))
    out, sc = torch.zeros(64, dtype=torch.uint8, device="cuda"), torch.zeros(4, device="cuda")
    for bad in (0, 24, 8):
        with pytest.raises(DnnError) as e:
            ops.quantize_block_scaled(x, out, sc, bad)
        assert e.value.variant == "InvalidArgument"
    with pytest.raises(DnnError) as e:
        ops.quantize_block_scaled(x, out[:10], sc, 16)
    assert e.value.variant == "BufferTooSmall" and e.value.expected == 64
    with pytest.raises(DnnError) as e:                            # scales: expected / actual in bytes (block_scale.rs:89-94)
        ops.quantize_block_scaled(x, out, sc[:1], 16)
    assert e.value.expected == 16 and e.value.actual == 4

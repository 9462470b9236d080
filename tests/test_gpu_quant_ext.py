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

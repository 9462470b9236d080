"""GPU parity of the GPTQ weight preparation against the oracle's restatement of GptqQuantizer::quantize_layer
(crates/oxicuda-quant/src/scheme/gptq.rs): every stage keeps the reference's order of f32 operations, so the inverse
Hessian, the codes, the scales and the zero points are compared bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from oxicuda_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def orc():
    from oracle import oracle as _orc
    _orc.build()
    return _orc


def _layer(n_rows, n_cols, seed, samples=None):
    rng = np.random.default_rng(seed)
    samples = samples or 2 * n_cols
    x = rng.standard_normal((samples, n_cols)).astype(np.float32)
    x[:, : max(1, n_cols // 16)] *= 6.0                                  # a few dominant input channels
    h = (2.0 * (x.T.astype(np.float64) @ x.astype(np.float64)) / samples).astype(np.float32)
    h = np.maximum(h, h.T)                                               # exactly symmetric
    w = (rng.standard_normal((n_rows, n_cols)) * 0.05).astype(np.float32)
    return w, h


def _run(ops, w, h, **cfg):
    q = ops.GptqQuantizer(ops.GptqConfig(**cfg))
    out = q.quantize_layer(torch.from_numpy(w).cuda(), w.shape[0], w.shape[1], torch.from_numpy(h).cuda())
    torch.cuda.synchronize()
    assert ops.handle().device_status() == 0
    return q, out


@pytest.mark.parametrize("shape", [(2, 2), (3, 6), (16, 32), (40, 97), (130, 192), (300, 257)])
@pytest.mark.parametrize("cfg", [dict(bits=4, symmetric=True), dict(bits=4, symmetric=False), dict(bits=8, symmetric=True),
                                 dict(bits=3, symmetric=False, percdamp=0.1)])
def test_gptq_layer_matches_reference(ops, orc, shape, cfg):
    n_rows, n_cols = shape
    w, h = _layer(n_rows, n_cols, seed=n_rows * 1000 + n_cols)
    q, out = _run(ops, w, h, **cfg)
    rq, rs, rz = orc.ref_gptq_quantize_layer(w, n_rows, n_cols, h, bits=cfg["bits"], symmetric=cfg["symmetric"], percdamp=cfg.get("percdamp", 0.01))
    assert np.array_equal(out.scales.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(out.zero_points.cpu().numpy(), rz)
    assert np.array_equal(out.quantized.cpu().numpy(), rq)


def test_gptq_stages_match_reference(ops, orc):
    """The inverse Hessian and the factor's inverse left in the workspace, bit for bit, at a size that crosses several
    32-wide blocks and ends in a ragged one."""
    n_rows, n_cols = 64, 203
    w, h = _layer(n_rows, n_cols, seed=5)
    q, out = _run(ops, w, h, bits=4)
    ws = q.workspace.view(torch.float32)
    hinv = ws[: n_cols * n_cols].reshape(n_cols, n_cols).cpu().numpy()
    linv = ws[n_cols * n_cols: 2 * n_cols * n_cols].reshape(n_cols, n_cols).cpu().numpy()
    lam = np.float32(0.01) * np.float32(abs(np.float32(np.cumsum(np.diag(h), dtype=np.float32)[-1]) / np.float32(n_cols)))
    hd = h.copy()
    hd[np.diag_indices(n_cols)] += lam
    l = orc.ref_cholesky_lower(hd)
    li = orc.ref_invert_lower(l)
    assert np.array_equal(np.tril(linv).view(np.uint32), li.view(np.uint32))
    iu = np.triu_indices(n_cols)
    assert np.array_equal(hinv[iu].view(np.uint32), orc.ref_hinv_upper(li)[iu].view(np.uint32))


def test_gptq_medium_layer(ops, orc):
    """1024 x 1024: several row chunks per CTA, sixteen column blocks; still bit for bit."""
    w, h = _layer(1024, 1024, seed=11, samples=1536)
    _, out = _run(ops, w, h, bits=4)
    rq, rs, rz = orc.ref_gptq_quantize_layer(w, 1024, 1024, h, bits=4)
    assert np.array_equal(out.scales.cpu().numpy().view(np.uint32), rs.view(np.uint32))
    assert np.array_equal(out.quantized.cpu().numpy(), rq)
    # a diagonal Hessian has a diagonal inverse: nothing propagates, whatever the diagonal holds
    hd = np.diag(np.diag(h)).astype(np.float32)
    _, diag = _run(ops, w, hd, bits=4)
    _, eye = _run(ops, w, np.eye(1024, dtype=np.float32), bits=4)
    assert torch.equal(diag.quantized, eye.quantized) and torch.equal(diag.scales, eye.scales)


def test_gptq_identity_hessian_is_round_to_nearest(ops):
    """Size-independent property at a full layer size: with H = I nothing propagates, so the codes are the per-column
    round-to-nearest codes (reference test identity_hessian_int8_low_mse, gptq.rs:464-482, scaled up)."""
    n_rows, n_cols = 4096, 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    w = torch.randn((n_rows, n_cols), generator=g, device="cuda") * 0.02
    q = ops.GptqQuantizer(ops.GptqConfig(bits=4))
    out = q.quantize_layer(w, n_rows, n_cols, torch.eye(n_cols, device="cuda"))
    torch.cuda.synchronize()
    assert ops.handle().device_status() == 0
    am = np.maximum(w.abs().amax(dim=0).cpu().numpy(), np.float32(1e-8))
    scale = torch.from_numpy(am / np.float32(7.0)).cuda()                # IEEE division (torch turns a division by a Python scalar into a multiplication)
    assert torch.equal(out.scales, scale)
    v = w / scale[None, :]
    t = torch.trunc(v)                                                   # f32::round: half away from zero (v - trunc(v) is exact)
    want = (t + torch.sign(v) * ((v - t).abs() >= 0.5)).clamp(-8, 7).to(torch.int32)
    assert torch.equal(out.quantized, want)
    assert out.reconstruction_mse(w) < float((scale.max() / 2) ** 2)


def test_gptq_errors(ops):
    """singular_hessian_returns_error, dimension_mismatch_weight, invalid_bit_width (gptq.rs:422-462)."""
    from oxicuda_b200.errors import QuantError
    w = torch.full((2, 2), 0.5, device="cuda")
    with pytest.raises(QuantError) as e:
        ops.GptqQuantizer(ops.GptqConfig(percdamp=0.0)).quantize_layer(w, 2, 2, torch.zeros((2, 2), device="cuda"))
    assert e.value.variant == "SingularHessian"
    with pytest.raises(QuantError) as e:
        ops.GptqQuantizer().quantize_layer(torch.full((3,), 0.5, device="cuda"), 1, 4, torch.eye(4, device="cuda"))
    assert e.value.variant == "DimensionMismatch"
    with pytest.raises(QuantError) as e:
        ops.GptqQuantizer(ops.GptqConfig(bits=0)).quantize_layer(w, 2, 2, torch.eye(2, device="cuda"))
    assert e.value.variant == "InvalidBitWidth"
    with pytest.raises(QuantError) as e:
        ops.GptqQuantizer().quantize_layer(torch.zeros(0, device="cuda"), 0, 4, torch.eye(4, device="cuda"))
    assert e.value.variant == "EmptyInput"
    # a later pivot that fails: positive definite leading block, zero rest
    h = torch.zeros((40, 40), device="cuda")
    h[:35, :35] = torch.eye(35, device="cuda")
    with pytest.raises(QuantError) as e:
        ops.GptqQuantizer(ops.GptqConfig(percdamp=0.0)).quantize_layer(torch.ones((4, 40), device="cuda"), 4, 40, h)
    assert e.value.variant == "SingularHessian"

"""GPU parity of the low-precision GEMMs, through the C ABI, against the oracle's
dequantise-then-f32 result.  Tolerance (bf16 output): max |y - ref| <= 1e-2 * max |ref| over the
matrix ("max-relative 1e-2"), plus an elementwise sanity check |y - ref| <= 1e-2 |ref| + 1e-2 max|ref|/2
(entries near zero carry the bf16 rounding of their operands, so they cannot be held to a purely relative bound)."""
import numpy as np
import pytest
import torch

from tests.gpu_util import bf16_bits, bf16_dev, to_dev, u16, u32

pytestmark = pytest.mark.gpu
MAX_REL = 1e-2


@pytest.fixture(scope="module")
def ops():
    from oxicuda_b200 import ops
    return ops


def _check(y: np.ndarray, ref: np.ndarray, tag=""):
    assert y.shape == ref.shape
    assert np.isfinite(y).all(), f"{tag}: non-finite output"
    scale = np.abs(ref).max()
    err = np.abs(y - ref)
    assert err.max() <= MAX_REL * scale, f"{tag}: max err {err.max()} vs {MAX_REL * scale}"
    assert (err <= MAX_REL * np.abs(ref) + MAX_REL * scale / 2).all(), tag


def _bf16_to_np(t):
    return t.float().cpu().numpy()


def _status_clean(ops):
    assert ops.handle().device_status() == 0


# ------------------------------------------------------------------------------------------- FP8

@pytest.mark.parametrize("mnk", [(128, 256, 128), (256, 512, 256), (300, 520, 384), (1024, 1024, 1024), (64, 264, 2048),
                                 (1, 256, 128), (129, 257 * 8, 16)])
def test_gemm_fp8(ops, orc, mnk):
    m, n, k = mnk
    a = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    b = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 1))
    qa, sa = ops.fp8_quant_dynamic(bf16_dev(a))
    qb, sb = ops.fp8_quant_dynamic(bf16_dev(b))
    y = ops.gemm_fp8(qa, qb, sa[1:], sb[1:])
    torch.cuda.synchronize()
    _status_clean(ops)
    # oracle: dequantised codes (exact in f32), f32 GEMM, one f32 scale product, bf16 rounding
    da = orc.e4m3_to_f32(qa.cpu().numpy())
    db = orc.e4m3_to_f32(qb.cpu().numpy())
    s = np.float32(sa.cpu().numpy()[1]) * np.float32(sb.cpu().numpy()[1])
    ref = (da.astype(np.float64) @ db.astype(np.float64).T).astype(np.float32) * s
    _check(_bf16_to_np(y), ref, f"fp8 {mnk}")
    if m * n * k <= 128 * 256 * 128:
        # small case: the reference's left-to-right f32 accumulation, bf16-rounded, agrees to 1 bf16 ulp
        ref_seq = orc.ref_linear_f32(da, db) * s
        yb = bf16_bits(y).astype(np.int32)
        rb = orc.f32_to_bf16_bits(ref_seq).astype(np.int32)
        assert np.abs(yb - rb).max() <= 1


@pytest.mark.parametrize("mnk", [(1, 16, 64), (1, 4096, 4096), (8, 1000, 1040), (3, 520, 384), (5, 28672, 1024), (8, 264, 8192),
                                 (9, 520, 384), (16, 4096, 4096), (31, 1000, 1040), (64, 264, 28672), (40, 8192, 2048)])
def test_gemm_fp8_decode_shapes(ops, orc, mnk):
    """Up to 8 batch rows run the GEMV kernel (mma.sync on the raw E4M3 bytes), more the 128-row kernels: same oracle, ragged N and K, alpha."""
    m, n, k = mnk
    a = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    b = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 1))
    qa, sa = ops.fp8_quant_dynamic(bf16_dev(a))
    qb, sb = ops.fp8_quant_dynamic(bf16_dev(b))
    y = ops.gemm_fp8(qa, qb, sa[1:], sb[1:])
    y2 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.gemm_fp8_ex(-2.0, qa, qb, sa[1:], sb[1:], 0.0, y2)
    torch.cuda.synchronize()
    _status_clean(ops)
    da = orc.e4m3_to_f32(qa.cpu().numpy())
    db = orc.e4m3_to_f32(qb.cpu().numpy())
    s = np.float32(sa.cpu().numpy()[1]) * np.float32(sb.cpu().numpy()[1])
    ref = (da.astype(np.float64) @ db.astype(np.float64).T).astype(np.float32) * s
    _check(_bf16_to_np(y), ref, f"fp8 decode {mnk}")
    # tighter than the GEMM bar: products are exact and sums are kept in f32, so only the bf16 rounding of the output is left
    # (a single running FP8 mma.sync accumulator drifts by 0.7 % over K = 8192 and would fail this)
    assert np.abs(_bf16_to_np(y) - ref).max() <= 4e-3 * np.abs(ref).max()
    assert torch.equal(y2.float(), y.float() * -2.0)                       # alpha is a power of two: exact


@pytest.mark.parametrize("m", [3, 20, 48])
def test_gemm_decode_strided_operands(ops, orc, m):
    """Decode batch sizes with leading dimensions larger than K and an output wider than N: FP8 and W8A8 through the
    weight-streaming kernel (48 rows with 104 row tiles: its 64-column form)."""
    n, k = 13312, 512
    xa = ops.fp8_quant_dynamic(bf16_dev(orc.f32_to_bf16_bits(orc.gaussian((m, 2 * k), 1.0, 3))))
    wb = ops.fp8_quant_dynamic(bf16_dev(orc.f32_to_bf16_bits(orc.gaussian((n, 2 * k), 1.0, 4))))
    qx, qw = xa[0][:, k:], wb[0][:, :k]                      # leading dimension 2k
    ybuf = torch.full((m, n + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm_fp8(qx, qw, xa[1][1:], wb[1][1:], out=ybuf[:, :n])
    torch.cuda.synchronize()
    _status_clean(ops)
    s = float(xa[1][1]) * float(wb[1][1])
    ref = (orc.e4m3_to_f32(qx.cpu().numpy()).astype(np.float64) @ orc.e4m3_to_f32(qw.cpu().numpy()).astype(np.float64).T) * s
    _check(_bf16_to_np(ybuf[:, :n].contiguous()), ref.astype(np.float32), f"fp8 strided decode m={m}")
    assert torch.all(ybuf[:, n:] == 7.0)                     # nothing written past N
    # W8A8: exact integer sums
    xi = torch.randint(-127, 128, (m, 2 * k), dtype=torch.int8, device="cuda")
    wi = torch.randint(-127, 128, (n, 2 * k), dtype=torch.int8, device="cuda")
    sx = torch.rand(m, device="cuda") * 0.01 + 0.001
    sw = torch.rand(n, device="cuda") * 0.01 + 0.001
    yi = torch.full((m, n + 64), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.gemm_w8a8(xi[:, :k], wi[:, k:], sx, sw, out=yi[:, :n])
    torch.cuda.synchronize()
    _status_clean(ops)
    acc = xi[:, :k].double().cpu().numpy() @ wi[:, k:].double().cpu().numpy().T
    want = (acc.astype(np.float32) * (sx.cpu().numpy()[:, None] * sw.cpu().numpy()[None, :])).astype(np.float32)
    got = _bf16_to_np(yi[:, :n].contiguous())
    assert np.array_equal(got, orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(want))), "w8a8 strided decode: exact sums, one bf16 rounding"
    assert torch.all(yi[:, n:] == 7.0)


@pytest.mark.parametrize("mnk", [(1, 512, 256), (8, 1024, 4096), (5, 256, 1040), (12, 512, 2048), (33, 1024, 1024), (64, 7168, 8192),
                                 (4, 512, 8192), (2, 256, 28672), (8, 7168, 8192),    # the last three: K split over clusters of CTAs
                                 (16, 2048, 4096), (17, 512, 2048), (32, 7168, 8192), (32, 57344 // 8, 1024)])
def test_gemm_fp8_swiglu_decode_shapes(ops, orc, mnk):
    """The SwiGLU form at decode batch sizes: gate and up rows of one output column meet in one lane (up to 32 rows: the
    weight-streaming tensor-core kernel with a gate and an up accumulator per CTA)."""
    m, n2, k = mnk
    inter = n2 // 2
    x = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    wg = orc.f32_to_bf16_bits(orc.gaussian((inter, k), 0.05, 1))
    wu = orc.f32_to_bf16_bits(orc.gaussian((inter, k), 0.05, 2))
    w_gu = ops.interleave_gate_up(bf16_dev(wg), bf16_dev(wu))
    qx, sx = ops.fp8_quant_dynamic(bf16_dev(x))
    qw, sw = ops.fp8_quant_dynamic(w_gu)
    h = ops.gemm_fp8_swiglu(qx, qw, sx[1:], sw[1:])
    torch.cuda.synchronize()
    _status_clean(ops)
    dx = orc.e4m3_to_f32(qx.cpu().numpy()).astype(np.float64)
    dw = orc.e4m3_to_f32(qw.cpu().numpy()).astype(np.float64).reshape(inter // 128, 2, 128, k)
    s = float(sx[1]) * float(sw[1])
    gate = (dx @ dw[:, 0].reshape(inter, k).T) * s
    up = (dx @ dw[:, 1].reshape(inter, k).T) * s
    ref = (gate / (1.0 + np.exp(-gate)) * up).astype(np.float32)
    _check(_bf16_to_np(h), ref, f"fp8 swiglu decode {mnk}")


def test_gemm_fp8_strided_and_errors(ops, orc):
    from oxicuda_b200.errors import BlasError
    m, n, k = 128, 256, 256
    big_a = ops.fp8_quant_dynamic(bf16_dev(orc.f32_to_bf16_bits(orc.gaussian((m, 2 * k), 1.0, 0))))
    big_b = ops.fp8_quant_dynamic(bf16_dev(orc.f32_to_bf16_bits(orc.gaussian((n, 2 * k), 1.0, 1))))
    qa, qb = big_a[0][:, :k], big_b[0][:, k:]                # leading dimension 2k, offset k
    y = ops.gemm_fp8(qa, qb, big_a[1][1:], big_b[1][1:])
    da, db = orc.e4m3_to_f32(qa.cpu().numpy()), orc.e4m3_to_f32(qb.cpu().numpy())
    s = float(big_a[1][1]) * float(big_b[1][1])
    _check(_bf16_to_np(y), (da @ db.T) * np.float32(s), "fp8 strided")
    one = torch.ones(1, device="cuda")
    e8 = torch.zeros((0, 64), dtype=torch.uint8, device="cuda")
    with pytest.raises(BlasError) as e:                     # zero dimension -> InvalidDimension (gemm_api.rs:88-92)
        ops.gemm_fp8(e8, big_b[0][:, :64], one, one)
    assert e.value.variant == "InvalidDimension"
    with pytest.raises(BlasError) as e:                     # K not a multiple of 16
        ops.gemm_fp8(big_a[0][:, :24].contiguous(), big_b[0][:, :24].contiguous(), one, one)
    assert e.value.variant == "InvalidArgument"


def test_gemm_fp8_linearity_full_size(ops, orc):
    """Benchmark size 8192^3: a sample of 64 x 64 outputs against the f64 dot product of the dequantised
    codes, plus scale linearity: doubling sx doubles every output exactly (power-of-two scaling)."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((8192, 8192), generator=gen, device="cuda").to(torch.bfloat16)
    b = torch.randn((8192, 8192), generator=gen, device="cuda").to(torch.bfloat16)
    qa, sa = ops.fp8_quant_dynamic(a)
    qb, sb = ops.fp8_quant_dynamic(b)
    y = ops.gemm_fp8(qa, qb, sa[1:], sb[1:])
    y2 = ops.gemm_fp8(qa, qb, sa[1:] * 2, sb[1:])
    torch.cuda.synchronize()
    _status_clean(ops)
    assert torch.equal(y2.float(), y.float() * 2)
    rows = torch.randint(0, 8192, (64,), generator=torch.Generator().manual_seed(1))
    cols = torch.randint(0, 8192, (64,), generator=torch.Generator().manual_seed(2))
    da = orc.e4m3_to_f32(qa[rows.cuda()].cpu().numpy()).astype(np.float64)
    db = orc.e4m3_to_f32(qb[cols.cuda()].cpu().numpy()).astype(np.float64)
    ref = (da @ db.T).astype(np.float32) * (np.float32(float(sa[1])) * np.float32(float(sb[1])))
    got = y[rows.cuda()][:, cols.cuda()].float().cpu().numpy()
    _check(got, ref, "fp8 8192^3 sample")


# ------------------------------------------------------------------------------------------- W8A8 / W8A32

@pytest.mark.parametrize("mnk", [(128, 256, 128), (200, 512, 1024), (33, 264, 4096), (1, 16, 64), (1, 4096, 4096), (8, 1000, 1040), (5, 8192, 28672), (3, 520, 384)])
def test_gemm_w8a8(ops, orc, mnk):
    m, n, k = mnk
    x = orc.gaussian((m, k), 1.0, 1)
    w = orc.gaussian((n, k), 0.02, 0)
    qx, sx = ops.int8_quant_rows(to_dev(x))
    qw, sw = ops.int8_quant_rows(to_dev(w))
    y = ops.gemm_w8a8(qx, qw, sx, sw)
    torch.cuda.synchronize()
    _status_clean(ops)
    acc = qx.cpu().numpy().astype(np.int64) @ qw.cpu().numpy().astype(np.int64).T      # exact integer result
    ref = acc.astype(np.float32) * (sx.cpu().numpy()[:, None] * sw.cpu().numpy()[None, :])
    _check(_bf16_to_np(y), ref, f"w8a8 {mnk}")
    # the s32 accumulator is exact, so the only error is the final bf16 rounding
    assert np.abs(bf16_bits(y).astype(np.int32) - orc.f32_to_bf16_bits(ref).astype(np.int32)).max() <= 1


@pytest.mark.parametrize("mnk", [(8, 4096, 4096), (1, 64, 512), (13, 100, 1040), (32, 256, 2048), (64, 1000, 4096), (20, 17, 16), (9, 4096, 1024)])
def test_gemm_w8a32_config1(ops, orc, mnk):
    """Benchmark configuration 1: INT8 per-channel weights, f32 activations, f32 accumulate and output."""
    m, n, k = mnk
    w = orc.gaussian((n, k), 0.02, 0)
    x = orc.gaussian((m, k), 1.0, 1)
    qw, sw = ops.int8_quant_rows(to_dev(w))
    y = ops.gemm_w8a32(to_dev(x), qw, sw).cpu().numpy()
    deq = orc.spec_int8_dequant_rows(qw.cpu().numpy(), sw.cpu().numpy())
    ref = orc.ref_linear_f32(x, deq, threads=orc.max_threads())     # reference summation order, f32
    scale = np.abs(ref).max()
    assert np.abs(y - ref).max() <= 1e-4 * scale                     # f32 path: only the summation order differs


@pytest.mark.parametrize("mnk", [(128, 256, 128), (300, 520, 384), (1024, 1024, 1024), (16, 264, 2048), (2048, 2304, 512)])
@pytest.mark.parametrize("ab", [(2.0, 0.0), (1.0, 1.0), (-0.5, 0.75)])
def test_gemm_alpha_beta(ops, orc, mnk, ab):
    """gemm's general form: Y = alpha * (X . W^T) * scales + beta * Y, for the FP8 and bf16 kernels (1-CTA, CTA-pair, split tail)."""
    m, n, k = mnk
    alpha, beta = ab
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    wb = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 1))
    y0b = orc.f32_to_bf16_bits(orc.gaussian((m, n), 5.0, 2))
    x, w = bf16_dev(xb), bf16_dev(wb)
    y0 = orc.bf16_bits_to_f32(y0b)
    # bf16
    y = bf16_dev(y0b).clone()
    if beta == 0.0:
        y.fill_(float("nan"))                                 # beta == 0: the old contents must not be read
    ops.gemm_bf16_ex(alpha, x, w, beta, y)
    ref = alpha * (orc.bf16_bits_to_f32(xb).astype(np.float64) @ orc.bf16_bits_to_f32(wb).astype(np.float64).T) + beta * y0
    _check(_bf16_to_np(y), ref.astype(np.float32), f"bf16 alpha/beta {mnk} {ab}")
    # fp8
    xq, sx = ops.fp8_quant_dynamic(x)
    wq, sw = ops.fp8_quant_dynamic(w)
    y = bf16_dev(y0b).clone()
    if beta == 0.0:
        y.fill_(float("nan"))
    ops.gemm_fp8_ex(alpha, xq, wq, sx[1:], sw[1:], beta, y)
    torch.cuda.synchronize()
    _status_clean(ops)
    acc = orc.e4m3_to_f32(xq.cpu().numpy()).astype(np.float64) @ orc.e4m3_to_f32(wq.cpu().numpy()).astype(np.float64).T
    ref = alpha * acc * (float(sx[1]) * float(sw[1])) + beta * y0
    _check(_bf16_to_np(y), ref.astype(np.float32), f"fp8 alpha/beta {mnk} {ab}")


def _mn_major(t):
    """[rows x k] -> the transposed matrix [k x rows] with its leading dimension padded to 16 bytes (a view of the padded buffer)."""
    rows, k = t.shape
    al = 16 // t.element_size()
    ld = (rows + al - 1) // al * al
    buf = torch.zeros((k, ld), dtype=t.dtype, device=t.device)
    buf[:, :rows] = t.t()
    return buf[:, :rows]


@pytest.mark.parametrize("mnk", [(256, 512, 256), (300, 520, 384), (1024, 1024, 1024), (64, 264, 2048), (2048, 2304, 512), (129, 136, 48)])
@pytest.mark.parametrize("majors", [(0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("kind", ["fp8", "bf16"])
def test_gemm_operand_forms(ops, orc, mnk, majors, kind):
    """gemm's trans_a / trans_b / layout forms: A stored [M x K] or [K x M], B stored [N x K] or [K x N] (the reference's default
    NoTrans, NoTrans call on row-major matrices is A K-major, B MN-major), against the same oracle as the K-major form, with
    alpha and beta."""
    m, n, k = mnk
    a_mn, b_mn = majors
    ab = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    bb = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 1))
    y0b = orc.f32_to_bf16_bits(orc.gaussian((m, n), 3.0, 2))
    a, b = bf16_dev(ab), bf16_dev(bb)
    y = bf16_dev(y0b).clone()
    alpha, beta = 0.5, 1.0
    if kind == "fp8":
        qa, sa = ops.fp8_quant_dynamic(a)
        qb, sb = ops.fp8_quant_dynamic(b)
        am = _mn_major(qa) if a_mn else qa                      # [K x M] when MN-major
        bm = _mn_major(qb) if b_mn else qb                      # [K x N] when MN-major
        ops.gemm_fp8_op(m, n, k, alpha, am, a_mn, bm, b_mn, sa[1:], sb[1:], beta, y)
        acc = orc.e4m3_to_f32(qa.cpu().numpy()).astype(np.float64) @ orc.e4m3_to_f32(qb.cpu().numpy()).astype(np.float64).T
        acc *= float(sa[1]) * float(sb[1])
    else:
        am = _mn_major(a) if a_mn else a
        bm = _mn_major(b) if b_mn else b
        ops.gemm_bf16_op(m, n, k, alpha, am, a_mn, bm, b_mn, beta, y)
        acc = orc.bf16_bits_to_f32(ab).astype(np.float64) @ orc.bf16_bits_to_f32(bb).astype(np.float64).T
    torch.cuda.synchronize()
    _status_clean(ops)
    ref = alpha * acc + beta * orc.bf16_bits_to_f32(y0b)
    _check(_bf16_to_np(y), ref.astype(np.float32), f"{kind} operand forms {mnk} {majors}")


def test_gemm_operand_forms_errors(ops):
    from oxicuda_b200.errors import BlasError
    a = torch.zeros((64, 128), dtype=torch.uint8, device="cuda")
    y = torch.zeros((64, 64), dtype=torch.bfloat16, device="cuda")
    one = torch.ones(1, device="cuda")
    with pytest.raises(BlasError) as e:                      # unknown layout flag
        ops.gemm_fp8_op(64, 64, 128, 1.0, a, 2, a, 0, one, one, 0.0, y)
    assert e.value.variant == "InvalidArgument"
    with pytest.raises(BlasError) as e:                      # B said to be [K x N] with N = 256 but only 128 elements per row
        ops.gemm_fp8_op(64, 256, 64, 1.0, a[:, :64].contiguous(), 0, a, 1, one, one, 0.0, torch.zeros((64, 256), dtype=torch.bfloat16, device="cuda"))
    assert e.value.variant == "InvalidDimension"
    with pytest.raises(BlasError) as e:                      # zero dimension (gemm_api.rs:88-92)
        ops.gemm_fp8_op(0, 64, 128, 1.0, a, 0, a, 0, one, one, 0.0, y)
    assert e.value.variant == "InvalidDimension"


# ------------------------------------------------------------------------------------------- W4A16

@pytest.mark.parametrize("m", [1, 8, 32, 5, 17, 9, 16])
@pytest.mark.parametrize("nk", [(256, 512), (4096, 4096), (200, 1024), (6144, 4096), (384, 14336)])
def test_gemm_w4a16_decode(ops, orc, m, nk):
    n, k = nk
    w = orc.gaussian((n, k), 0.02, 0)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 1))
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    ws = ops.gemm_w4a16_workspace(m, n, k, "cuda")
    y = ops.gemm_w4a16(bf16_dev(xb), c, s, z, 128, workspace=ws)
    torch.cuda.synchronize()
    deq = orc.spec_int4g_dequant(u32(c), u16(s), u32(z), n, k, 128)
    ref = (orc.bf16_bits_to_f32(xb).astype(np.float64) @ deq.astype(np.float64).T).astype(np.float32)
    _check(_bf16_to_np(y), ref, f"w4a16 m={m} {nk}")
    assert int(ws.view(torch.int32).abs().max()) == 0               # workspace left zeroed
    y2 = ops.gemm_w4a16(bf16_dev(xb), c, s, z, 128, workspace=ws)   # and therefore reusable
    _check(_bf16_to_np(y2), ref, "w4a16 second call")
    _status_clean(ops)


@pytest.mark.parametrize("nk", [(14336, 4096), (4096, 14336)])
def test_gemm_w4a16_decode_llama8b_mlp_weights(ops, orc, nk):
    """Benchmark configuration 3's two large projection weights at M = 1, 8, 32 (quantised once per weight)."""
    n, k = nk
    w = orc.gaussian((n, k), 0.02, 0)
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    deq = orc.spec_int4g_dequant(u32(c), u16(s), u32(z), n, k, 128).astype(np.float64)
    for m in (1, 8, 32):
        xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 1 + m))
        ws = ops.gemm_w4a16_workspace(m, n, k, "cuda")
        y = ops.gemm_w4a16(bf16_dev(xb), c, s, z, 128, workspace=ws)
        torch.cuda.synchronize()
        ref = (orc.bf16_bits_to_f32(xb).astype(np.float64) @ deq.T).astype(np.float32)
        _check(_bf16_to_np(y), ref, f"w4a16 m={m} {nk}")
        assert int(ws.view(torch.int32).abs().max()) == 0
    _status_clean(ops)


def test_gemm_w4a16_one_workspace_for_prefill_and_decode(ops, orc):
    """One workspace sized for the largest batch, used for a prefill call and then for decode calls: the dequantised weight
    of the prefill call must not sit where the decode kernels expect zeroed partial sums."""
    n, k = 1024, 2048
    w = orc.gaussian((n, k), 0.02, 0)
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    deq = orc.spec_int4g_dequant(u32(c), u16(s), u32(z), n, k, 128).astype(np.float64)
    ws = ops.gemm_w4a16_workspace(128, n, k, "cuda")
    for m in (128, 16, 4, 48, 128, 32, 1):
        xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 10 + m))
        y = ops.gemm_w4a16(bf16_dev(xb), c, s, z, 128, workspace=ws)
        torch.cuda.synchronize()
        ref = (orc.bf16_bits_to_f32(xb).astype(np.float64) @ deq.T).astype(np.float32)
        _check(_bf16_to_np(y), ref, f"w4a16 shared workspace m={m}")
    _status_clean(ops)


def test_gemm_w4a16_scales_at_an_odd_offset(ops, orc):
    """The scales pointer is only promised 2-byte alignment: scales that start 2, 4 or 6 bytes into a buffer take the
    scalar loads and give the same result."""
    n, k, m = 256, 4096, 3
    w = orc.gaussian((n, k), 0.02, 0)
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 1))
    want = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")              # the same kernel (no workspace), aligned scales
    ops.handle().call("oxq_gemm_w4a16", m, n, k, ops._p(bf16_dev(xb)), ops._p(c), ops._p(s), ops._p(z), 128, ops._p(want), ops._p(None), 0)
    for off in (1, 2, 3):
        buf = torch.zeros(s.numel() + 8, dtype=torch.float16, device="cuda")
        shifted = buf[off:off + s.numel()]
        shifted.copy_(s.view(-1))
        assert shifted.data_ptr() % 8 == (2 * off) % 8
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        ops.handle().call("oxq_gemm_w4a16", m, n, k, ops._p(bf16_dev(xb)), ops._p(c), ops._p(shifted), ops._p(z), 128, ops._p(y), ops._p(None), 0)
        torch.cuda.synchronize()
        assert torch.equal(y, want)
    _status_clean(ops)


@pytest.mark.parametrize("m", [33, 48, 64, 100, 128])
@pytest.mark.parametrize("nk", [(4096, 4096), (200, 1024), (14336, 4096)])
def test_gemm_w4a16_mid_batch(ops, orc, m, nk):
    """Batches of 33..64 rows run as one pass of the fused tensor-core kernel with 64 batch columns, larger ones through
    the dequantised weight; a workspace that held something else before (here: ones) must not leak into the result."""
    n, k = nk
    w = orc.gaussian((n, k), 0.02, 0)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 1))
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    ws = ops.gemm_w4a16_workspace(m, n, k, "cuda")
    ws.fill_(1)
    y = ops.gemm_w4a16(bf16_dev(xb), c, s, z, 128, workspace=ws)
    torch.cuda.synchronize()
    _status_clean(ops)
    deq = orc.spec_int4g_dequant(u32(c), u16(s), u32(z), n, k, 128)
    ref = (orc.bf16_bits_to_f32(xb).astype(np.float64) @ deq.astype(np.float64).T).astype(np.float32)
    _check(_bf16_to_np(y), ref, f"w4a16 m={m} {nk}")


@pytest.mark.parametrize("mnk", [(64, 256, 512), (200, 1000, 1024), (2048, 1024, 4096)])
def test_gemm_w4a16_prefill(ops, orc, mnk):
    m, n, k = mnk
    w = orc.gaussian((n, k), 0.02, 0)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 1))
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    y = ops.gemm_w4a16(bf16_dev(xb), c, s, z, 128)
    torch.cuda.synchronize()
    _status_clean(ops)
    deq = orc.spec_int4g_dequant(u32(c), u16(s), u32(z), n, k, 128)
    ref = (orc.bf16_bits_to_f32(xb).astype(np.float64) @ deq.astype(np.float64).T).astype(np.float32)
    _check(_bf16_to_np(y), ref, f"w4a16 prefill {mnk}")


@pytest.mark.parametrize("mnk", [(128, 256, 128), (300, 520, 384), (1024, 1024, 1024), (16, 264, 2048)])
def test_gemm_bf16(ops, orc, mnk):
    m, n, k = mnk
    a = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    b = orc.f32_to_bf16_bits(orc.gaussian((n, k), 0.02, 1))
    y = ops.gemm_bf16(bf16_dev(a), bf16_dev(b))
    torch.cuda.synchronize()
    _status_clean(ops)
    ref = (orc.bf16_bits_to_f32(a).astype(np.float64) @ orc.bf16_bits_to_f32(b).astype(np.float64).T).astype(np.float32)
    _check(_bf16_to_np(y), ref, f"bf16 {mnk}")


@pytest.mark.parametrize("m", [1, 64, 300])
def test_swiglu_fused_gemms(ops, orc, m):
    """gate/up projection with the SwiGLU fused into the epilogue (FP8 and bf16) and the standalone SwiGLU kernel,
    against silu(x) = x / (1 + exp(-x)) of the reference (crates/oxicuda-lm/src/layer/ffn.rs:25-27) in f32."""
    inter, k = 384, 512
    wg = orc.gaussian((inter, k), 0.05, 0)
    wu = orc.gaussian((inter, k), 0.05, 2)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 1))
    w_gu = ops.interleave_gate_up(to_dev(wg), to_dev(wu))
    # fp8: one scale for the fused weight tensor
    qw, sw = ops.fp8_quant_dynamic(w_gu)
    qx, sx = ops.fp8_quant_dynamic(bf16_dev(xb))
    h = ops.gemm_fp8_swiglu(qx, qw, sx[1:], sw[1:])
    torch.cuda.synchronize()
    _status_clean(ops)
    dq = orc.e4m3_to_f32(qw.cpu().numpy()).reshape(inter // 128, 2, 128, k)
    dg, du = dq[:, 0].reshape(inter, k), dq[:, 1].reshape(inter, k)
    dx = orc.e4m3_to_f32(qx.cpu().numpy())
    s = np.float32(float(sx[1])) * np.float32(float(sw[1]))
    ref = orc.ref_silu_mul((dx @ dg.T) * s, (dx @ du.T) * s)
    _check(_bf16_to_np(h), ref, f"fp8 swiglu m={m}")
    # bf16
    wb = w_gu.to(torch.bfloat16)
    h2 = ops.gemm_bf16_swiglu(bf16_dev(xb), wb)
    wbf = wb.float().cpu().numpy().reshape(inter // 128, 2, 128, k)
    xf = orc.bf16_bits_to_f32(xb)
    ref2 = orc.ref_silu_mul(xf @ wbf[:, 0].reshape(inter, k).T, xf @ wbf[:, 1].reshape(inter, k).T)
    _check(_bf16_to_np(h2), ref2, f"bf16 swiglu m={m}")
    # standalone kernel on the un-fused product
    gu = ops.gemm_bf16(bf16_dev(xb), wb)
    h3 = ops.swiglu_interleaved(gu)
    guf = gu.float().cpu().numpy().reshape(m, inter // 128, 2, 128)
    ref3 = orc.ref_silu_mul(guf[:, :, 0].reshape(m, inter), guf[:, :, 1].reshape(m, inter))
    _check(_bf16_to_np(h3), ref3, f"swiglu kernel m={m}")


def test_gemm_w4a16_errors(ops, orc):
    from oxicuda_b200.errors import BlasError
    w = orc.gaussian((128, 256), 0.02, 0)
    c, s, z = ops.int4g_quant_pack(to_dev(w), 128)
    x = torch.zeros((64, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(BlasError) as e:                     # prefill path needs the bf16-weight workspace
        ops.gemm_w4a16(x, c, s, z, 128, workspace=torch.zeros(256, dtype=torch.uint8, device="cuda"))
    assert e.value.variant == "BufferTooSmall"
    with pytest.raises(BlasError) as e:
        ops.gemm_w4a16(x[:1], c, s, z, 48)
    assert e.value.variant == "InvalidArgument"


# ------------------------------------------------------------------------------------------- block scaled

@pytest.mark.parametrize("mnk", [(128, 192, 128), (128, 384, 256), (256, 512, 512), (300, 1000, 1024), (64, 200, 4096), (1024, 1544, 2048)])
def test_gemm_mxfp8(ops, orc, mnk):
    m, n, k = mnk
    a = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    b = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 1))
    ca, sfa, sfa_mma = ops.mxfp8_quant(bf16_dev(a))
    cb, sfb, sfb_mma = ops.mxfp8_quant(bf16_dev(b))
    y = ops.gemm_mxfp8(ca, sfa_mma, cb, sfb_mma)
    torch.cuda.synchronize()
    _status_clean(ops)
    da = orc.spec_mxfp8_dequant(ca.cpu().numpy(), sfa.cpu().numpy()).astype(np.float64)
    db = orc.spec_mxfp8_dequant(cb.cpu().numpy(), sfb.cpu().numpy()).astype(np.float64)
    _check(_bf16_to_np(y), (da @ db.T).astype(np.float32), f"mxfp8 {mnk}")


@pytest.mark.parametrize("mnk", [(128, 192, 256), (128, 384, 512), (256, 512, 1024), (300, 1000, 1024), (64, 200, 4096), (1024, 1544, 2048)])
def test_gemm_nvfp4(ops, orc, mnk):
    m, n, k = mnk
    a = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 0))
    b = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 1))
    pa, sfa, sfa_mma, sta = ops.nvfp4_quant(bf16_dev(a))
    pb, sfb, sfb_mma, stb = ops.nvfp4_quant(bf16_dev(b))
    y = ops.gemm_nvfp4(pa, sfa_mma, sta, pb, sfb_mma, stb)
    torch.cuda.synchronize()
    _status_clean(ops)
    da = orc.spec_nvfp4_dequant(pa.cpu().numpy(), sfa.cpu().numpy(), float(sta[1]), m, k).astype(np.float64)
    db = orc.spec_nvfp4_dequant(pb.cpu().numpy(), sfb.cpu().numpy(), float(stb[1]), n, k).astype(np.float64)
    _check(_bf16_to_np(y), (da @ db.T).astype(np.float32), f"nvfp4 {mnk}")


# Decode shapes: one to 64 batch rows, every batch tile width (16 / 32 / 64), K splits from 1 to 8 CTAs, a ragged last
# weight tile, and the two weight shapes of the Llama-3-8B MLP.
@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("mnk", [(1, 128, 256), (3, 200, 512), (8, 1000, 1024), (16, 4096, 4096), (17, 384, 2048), (32, 14336, 4096),
                                 (33, 256, 8192), (64, 520, 1024), (5, 4096, 14336), (1, 14336, 4096)])
def test_gemm_block_scaled_decode(ops, orc, fmt, mnk):
    m, n, k = mnk
    a = orc.f32_to_bf16_bits(orc.gaussian((m, k), 1.0, 10))
    b = orc.f32_to_bf16_bits(orc.gaussian((n, k), 1.0, 11))
    if fmt == "mxfp8":
        ca, sfa, sfa_mma = ops.mxfp8_quant(bf16_dev(a))
        cb, sfb, sfb_mma = ops.mxfp8_quant(bf16_dev(b))
        y = ops.gemm_mxfp8(ca, sfa_mma, cb, sfb_mma)
        y2 = ops.gemm_mxfp8(ca, sfa_mma, cb, sfb_mma)
        da = orc.spec_mxfp8_dequant(ca.cpu().numpy(), sfa.cpu().numpy()).astype(np.float64)
        db = orc.spec_mxfp8_dequant(cb.cpu().numpy(), sfb.cpu().numpy()).astype(np.float64)
    else:
        pa, sfa, sfa_mma, sta = ops.nvfp4_quant(bf16_dev(a))
        pb, sfb, sfb_mma, stb = ops.nvfp4_quant(bf16_dev(b))
        y = ops.gemm_nvfp4(pa, sfa_mma, sta, pb, sfb_mma, stb)
        y2 = ops.gemm_nvfp4(pa, sfa_mma, sta, pb, sfb_mma, stb)
        da = orc.spec_nvfp4_dequant(pa.cpu().numpy(), sfa.cpu().numpy(), float(sta[1]), m, k).astype(np.float64)
        db = orc.spec_nvfp4_dequant(pb.cpu().numpy(), sfb.cpu().numpy(), float(stb[1]), n, k).astype(np.float64)
    torch.cuda.synchronize()
    _status_clean(ops)
    assert torch.equal(y, y2), "the K split must not depend on scheduling"
    _check(_bf16_to_np(y), (da @ db.T).astype(np.float32), f"{fmt} decode {mnk}")


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_gemm_block_scaled_llama8b_prefill_size(ops, orc, fmt):
    """Benchmark configuration 4 at its real size (M = 4096, N = 14336, K = 4096), operands quantised on the GPU: 64 sampled
    rows of the output, all columns, against the f64 product of the dequantised codes."""
    m, n, k = 4096, 14336, 4096
    gen = torch.Generator(device="cuda").manual_seed(0)
    a = torch.randn((m, k), generator=gen, device="cuda").to(torch.bfloat16)
    b = torch.randn((n, k), generator=gen, device="cuda").to(torch.bfloat16)
    rows = torch.randint(0, m, (64,), generator=torch.Generator().manual_seed(1)).cuda()
    if fmt == "mxfp8":
        ca, sfa, sfa_mma = ops.mxfp8_quant(a)
        cb, sfb, sfb_mma = ops.mxfp8_quant(b)
        y = ops.gemm_mxfp8(ca, sfa_mma, cb, sfb_mma)
        torch.cuda.synchronize()
        da = orc.spec_mxfp8_dequant(ca[rows].cpu().numpy(), sfa[rows].cpu().numpy())
        db = orc.spec_mxfp8_dequant(cb.cpu().numpy(), sfb.cpu().numpy())
    else:
        pa, sfa, sfa_mma, sta = ops.nvfp4_quant(a)
        pb, sfb, sfb_mma, stb = ops.nvfp4_quant(b)
        y = ops.gemm_nvfp4(pa, sfa_mma, sta, pb, sfb_mma, stb)
        torch.cuda.synchronize()
        da = orc.spec_nvfp4_dequant(pa[rows].cpu().numpy(), sfa[rows].cpu().numpy(), float(sta[1]), 64, k)
        db = orc.spec_nvfp4_dequant(pb.cpu().numpy(), sfb.cpu().numpy(), float(stb[1]), n, k)
    _status_clean(ops)
    ref = np.empty((64, n), np.float32)
    da64 = da.astype(np.float64)
    for c0 in range(0, n, 2048):                                  # column blocks keep the f64 copy of the weight small
        ref[:, c0:c0 + 2048] = (da64 @ db[c0:c0 + 2048].astype(np.float64).T).astype(np.float32)
    _check(_bf16_to_np(y[rows]), ref, f"{fmt} 4096x14336x4096 sample")
    # the codes the GEMM consumed are the oracle's codes (bit-exact) on a slice of the activation tensor
    xs = a[:256].float().cpu().numpy()
    if fmt == "mxfp8":
        c_ref, sf_ref = orc.spec_mxfp8_quant(xs)
        assert np.array_equal(ca[:256].cpu().numpy(), c_ref) and np.array_equal(sfa[:256].cpu().numpy(), sf_ref)
    else:
        p_ref, sf_ref = orc.spec_nvfp4_quant(xs, float(sta[1]))
        assert np.array_equal(pa[:256].cpu().numpy(), p_ref) and np.array_equal(sfa[:256].cpu().numpy(), sf_ref)


def test_quantize_then_gemm_back_to_back(ops):
    """A quantizer followed directly by the GEMM that consumes its output, no host synchronisation in between: the decode
    kernels start under the tail of the kernel before them (dependent launch) and must not read the weights early.  The
    result has to equal, bit for bit, the same GEMM repeated after the stream has drained."""
    g = torch.Generator(device="cuda").manual_seed(5)
    n, k = 7168, 8192                                                     # 58 MB of 8-bit weights: the quantizer runs for tens of microseconds
    w = torch.randn((n, k), generator=g, device="cuda") * 0.02
    wb = w.to(torch.bfloat16)
    x1 = torch.randn((1, k), generator=g, device="cuda").to(torch.bfloat16)
    x16 = torch.randn((16, k), generator=g, device="cuda").to(torch.bfloat16)
    xf = x1.float().repeat(8, 1).contiguous()
    xq, sx = ops.fp8_quant_dynamic(x1)
    xi, sxi = ops.int8_quant_rows(xf)
    torch.cuda.synchronize()
    for _ in range(3):
        # FP8 and W8A8 GEMV
        wq, sw = ops.fp8_quant_dynamic(wb)
        y = ops.gemm_fp8(xq, wq, sx[1:], sw[1:])
        wi, swi = ops.int8_quant_rows(w)
        yi = ops.gemm_w8a8(xi, wi, sxi, swi)
        y32 = ops.gemm_w8a32(xf, wi, swi)
        # W4A16 GEMV and tensor-core kernel
        c, s, z = ops.int4g_quant_pack(w, 128)
        y4 = ops.gemm_w4a16(x1, c, s, z, 128)
        c2, s2, z2 = ops.int4g_quant_pack(w, 128)
        y4t = ops.gemm_w4a16(x16, c2, s2, z2, 128)
        # NF4
        pk, am = ops.nf4_quant(w.view(-1), 64)
        yn = ops.gemm_nf4(x1, pk, am, n, 64)
        torch.cuda.synchronize()
        assert torch.equal(y, ops.gemm_fp8(xq, wq, sx[1:], sw[1:]))
        assert torch.equal(yi, ops.gemm_w8a8(xi, wi, sxi, swi))
        assert torch.equal(y32, ops.gemm_w8a32(xf, wi, swi))
        assert torch.equal(y4, ops.gemm_w4a16(x1, c, s, z, 128))
        # the tensor-core kernel adds its K splits with f32 atomics: the order, hence the last bit, varies between calls
        y4r = ops.gemm_w4a16(x16, c2, s2, z2, 128).float()
        assert (y4t.float() - y4r).abs().max() <= 2e-2 * y4r.abs().max()
        assert torch.equal(yn, ops.gemm_nf4(x1, pk, am, n, 64))
        torch.cuda.synchronize()
        del wq, wi, c, s, z, c2, s2, z2, pk, am
    assert ops.handle().device_status() == 0

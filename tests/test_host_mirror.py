"""The C++ host mirror (oxicuda_b200/host/*.hpp): compiles and links against the C ABI on CPU; on a GPU the
driver program's INT8 per-row results are compared with the oracle bit for bit."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(tmp_path, name="host_mirror_test"):
    from oxicuda_b200 import _build
    _build.build()
    exe = str(tmp_path / name)
    libdir = os.path.join(ROOT, "oxicuda_b200", "lib")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", name + ".cpp"),
           "-o", exe, "-L" + libdir, "-loxq_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_host_config_types(tmp_path):
    """The configuration types' validate() rules (the reference's own tests restated in tests/cpp/host_config_test.cpp): host only."""
    from oxicuda_b200 import _build
    _build.build()
    exe = str(tmp_path / "host_config_test")
    libdir = os.path.join(ROOT, "oxicuda_b200", "lib")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I/usr/local/cuda/include", os.path.join(ROOT, "tests", "cpp", "host_config_test.cpp"),
           "-o", exe, "-L" + libdir, "-loxq_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, f"check {run.returncode} failed: {run.stdout} {run.stderr}"


def test_host_dnn_types(tmp_path):
    """Int4QuantConfig, TensorDesc::from_raw and Fp4BlockQuantizer (the reference's tests of int4_quantize.rs:971-996 and
    block_scale.rs:475-610 restated in tests/cpp/host_dnn_test.cpp): host only."""
    exe = _build(tmp_path, "host_dnn_test")
    run = subprocess.run([exe, "host"], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, f"check {run.returncode} failed: {run.stdout} {run.stderr}"


def test_host_lm_types(tmp_path):
    """WeightTensor, silu and SwiGluFfn's argument errors (crates/oxicuda-lm/src/layer/ffn.rs:279-296, :391-395; weights.rs:31-76)
    restated in tests/cpp/host_lm_test.cpp: host only."""
    exe = _build(tmp_path, "host_lm_test")
    run = subprocess.run([exe, "host"], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, f"check {run.returncode} failed: {run.stdout} {run.stderr}"


def test_host_mirror_compiles_and_links(tmp_path):
    exe = _build(tmp_path)
    assert os.path.exists(exe)
    assert os.path.exists(_build(tmp_path, "host_dnn_test"))
    assert os.path.exists(_build(tmp_path, "fused_gemv_test"))


def test_host_dist_infer_types(tmp_path):
    """Rank coordinates, handle accessors and the layers' argument errors (the reference's tests of handle.rs:246-360 and the
    error cases of column_parallel.rs / row_parallel.rs restated in tests/cpp/host_dist_infer_test.cpp): host only."""
    exe = _build(tmp_path, "host_dist_infer_test")
    run = subprocess.run([exe, "host"], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, f"check {run.returncode} failed: {run.stdout} {run.stderr}"


@pytest.mark.gpu
def test_host_mirror_runs_and_matches_oracle(tmp_path, orc):
    exe = _build(tmp_path)
    out = str(tmp_path / "out.bin")
    res = subprocess.run([exe, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"rc={res.returncode} {res.stderr}"
    raw = np.fromfile(out, dtype=np.uint8)
    n = 64 * 256
    x = raw[:4 * n].view(np.float32).reshape(64, 256)
    scales = raw[4 * n:4 * n + 256].view(np.float32)
    codes = raw[4 * n + 256:4 * n + 256 + 4 * n].view(np.int32).reshape(64, 256)
    deq = raw[4 * n + 256 + 4 * n:].view(np.float32)
    q_ref, s_ref = orc.spec_int8_quant_rows(x, orc.ROUND_HALF_AWAY)
    assert np.array_equal(scales, s_ref) and np.array_equal(codes, q_ref.astype(np.int32))
    # the reference's own path gives the same codes (calibrate_2d + quantize_grouped)
    sr, zr = orc.ref_minmax_calibrate_2d(x, 64, 256)
    assert np.array_equal(orc.minmax_quantize_grouped(x, sr, zr, 256).reshape(64, 256), codes)
    t = np.array([0.0, 1.0, -1.0, 0.5, 0.0, 2.0, -2.0, 1.5], np.float32).reshape(2, 4)
    qt, st = orc.spec_int8_quant_rows(t, orc.ROUND_HALF_AWAY)
    assert np.array_equal(deq, orc.spec_int8_dequant_rows(qt, st).ravel())


@pytest.mark.gpu
def test_host_dnn_mirror_runs_and_matches_oracle(tmp_path, orc):
    """oxicuda_dnn.hpp: known answers and buffer checks inside the driver; its 4100-element results against the oracle bit for bit."""
    exe = _build(tmp_path, "host_dnn_test")
    out = str(tmp_path / "dnn.bin")
    res = subprocess.run([exe, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"rc={res.returncode} {res.stderr}"
    raw = np.fromfile(out, dtype=np.uint8)
    n, ng, nb = 4100, (4100 + 127) // 128, (4100 + 31) // 32
    pos = 0

    def take(count, dtype):
        nonlocal pos
        size = count * np.dtype(dtype).itemsize
        v = raw[pos:pos + size].view(dtype)
        pos += size
        return v

    x = take(n, np.float32)
    q8, s8 = take(n, np.int8), take(1, np.float32)
    qf, sf = take(n, np.uint8), take(1, np.float32)
    p4s, s4s = take(n // 2, np.uint8), take(ng, np.float32)
    p4a, s4a, z4a, y4a = take(n // 2, np.uint8), take(ng, np.float32), take(ng, np.float32), take(n, np.float32)
    ob, sb = take(n, np.uint8), take(nb, np.float32)
    assert pos == raw.size
    q_ref, s_ref = orc.ref_dnn_int8_quant(x)
    assert np.array_equal(s8.view(np.uint32), s_ref.view(np.uint32)) and np.array_equal(q8, q_ref)
    sc = orc.spec_fp8_scale(orc.spec_absmax(x))
    assert sf[0] == sc and np.array_equal(qf, orc.spec_fp8_quant(x, sc))
    p_ref, sc_ref, _ = orc.ref_dnn_int4_quant(x, 128, True)
    assert np.array_equal(p4s, p_ref) and np.array_equal(s4s.view(np.uint32), sc_ref.view(np.uint32))
    p_ref, sc_ref, z_ref = orc.ref_dnn_int4_quant(x, 128, False)
    assert np.array_equal(p4a, p_ref) and np.array_equal(s4a.view(np.uint32), sc_ref.view(np.uint32))
    assert np.array_equal(z4a.view(np.uint32), z_ref.view(np.uint32))
    assert np.array_equal(y4a.view(np.uint32), orc.ref_dnn_int4_dequant(p_ref, sc_ref, n, 128, False).view(np.uint32))
    o_ref, sb_ref = orc.ref_dnn_block_scaled_quant(x, 32)
    assert np.array_equal(ob, o_ref) and np.array_equal(sb.view(np.uint32), sb_ref.view(np.uint32))


@pytest.mark.gpu
def test_host_dist_infer_mirror_runs_and_matches_oracle(tmp_path, orc):
    """oxicuda_dist_infer.hpp: the reference's ColumnLinear / RowLinear cases inside the driver (exact small integers); its
    256 -> 512 -> 256 pair at tp = 4 against the f32 oracle on the bf16-rounded operands."""
    exe = _build(tmp_path, "host_dist_infer_test")
    out = str(tmp_path / "dist.bin")
    res = subprocess.run([exe, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"rc={res.returncode} {res.stderr}"
    raw = np.fromfile(out, dtype=np.float32)
    tp, in_f, mid, batch = 4, 256, 512, 5
    sizes = [batch * in_f, mid * in_f, mid, in_f * mid, in_f, batch * mid, batch * in_f]
    raw, mlp_raw = raw[:sum(sizes)], raw[sum(sizes):]
    x, w1, b1, w2, b2, h, y = np.split(raw, np.cumsum(sizes)[:-1])
    rb = lambda a: orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(a))  # noqa: E731
    x, w1, w2 = rb(x).reshape(batch, in_f), rb(w1).reshape(mid, in_f), rb(w2).reshape(in_f, mid)
    h_ref = orc.ref_linear_f32(x, w1, b1)
    h = h.reshape(batch, mid)
    assert np.abs(h - h_ref).max() <= 2.0 ** -6 * np.abs(h_ref).max()          # two bf16 roundings (product, then product + bias): one ulp of the largest value
    # the row layer continues from the gathered h the driver produced: tp partial sums, each rounded to bf16
    y_ref = orc.ref_linear_f32(rb(h), w2, b2)
    assert np.abs(y.reshape(batch, in_f) - y_ref).max() <= 2.0 ** -6 * np.abs(y_ref).max()
    # TpSwiGluMlp (FP8), tp = 2: inside the driver the fused entry equals its four steps bit for bit; here h and the summed
    # partials against the oracle at the tensor-parallel bar of 1e-2 (the oracle's down projection continues from the device's h)
    hid, inter, m, mtp = 512, 2048, 5, 2
    il = inter // mtp
    sizes = [m * hid, inter * hid, inter * hid, hid * inter] + [m * il, m * hid] * mtp + [m * hid]
    assert mlp_raw.size == sum(sizes)
    parts = np.split(mlp_raw, np.cumsum(sizes)[:-1])
    xs, wg, wu, wd = parts[0].reshape(m, hid), parts[1].reshape(inter, hid), parts[2].reshape(inter, hid), parts[3].reshape(hid, inter)
    h_dev = [parts[4 + 2 * r].reshape(m, il) for r in range(mtp)]
    partials = [parts[5 + 2 * r].reshape(m, hid) for r in range(mtp)]
    ysum = parts[-1].reshape(m, hid)
    assert np.array_equal(ysum, partials[0] + partials[1])
    y_bits, own_h = orc.spec_tp_mlp(orc.f32_to_bf16_bits(xs), wg, wu, wd, mtp, variant="fp8",
                                    h_bits_per_rank=[orc.f32_to_bf16_bits(v) for v in h_dev], return_h=True)
    for r in range(mtp):
        h_ref = orc.bf16_bits_to_f32(own_h[r]).reshape(m, il)
        assert np.abs(h_dev[r] - h_ref).max() <= 1e-2 * np.abs(h_ref).max()
    y_ref = orc.bf16_bits_to_f32(y_bits).reshape(m, hid)
    assert np.abs(ysum - y_ref).max() <= 1e-2 * np.abs(y_ref).max()


@pytest.mark.gpu
def test_host_lm_mirror_runs_and_matches_oracle(tmp_path, orc):
    """oxicuda_lm.hpp: the reference's SwiGluFfn cases inside the driver; its 256 / 200 layer on five tokens against the f32
    oracle (SwiGluFfn::forward restated) and against the same arithmetic with h rounded to bf16 as the device holds it."""
    exe = _build(tmp_path, "host_lm_test")
    out = str(tmp_path / "lm.bin")
    res = subprocess.run([exe, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"rc={res.returncode} {res.stderr}"
    raw = np.fromfile(out, dtype=np.float32)
    hidden, inter, tokens = 256, 200, 5
    sizes = [tokens * hidden, inter * hidden, inter * hidden, hidden * inter, tokens * hidden]
    assert raw.size == sum(sizes)
    x, wg, wu, wd, y = np.split(raw, np.cumsum(sizes)[:-1])
    rb = lambda a: orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(a))  # noqa: E731
    x, wg, wu, wd = rb(x).reshape(tokens, hidden), rb(wg).reshape(inter, hidden), rb(wu).reshape(inter, hidden), rb(wd).reshape(hidden, inter)
    y = y.reshape(tokens, hidden)
    y_ref = orc.ref_swiglu_mlp(x, wg, wu, wd)
    scale = np.abs(y_ref).max()
    assert np.isfinite(y).all() and np.abs(y - y_ref).max() <= 2.0 ** -5 * scale     # h and y each rounded to bf16
    h = rb(orc.ref_silu_mul(orc.ref_linear_f32(x, wg), orc.ref_linear_f32(x, wu)))
    assert np.abs(y - rb(orc.ref_linear_f32(h, wd))).max() <= 2.0 ** -6 * scale       # same roundings: what is left is summation order


@pytest.mark.gpu
def test_fused_dequant_gemv_c_abi_matches_oracle(tmp_path, orc):
    """oxq_dnn_fused_dequant_gemv through the C ABI (tests/cpp/fused_gemv_test.cpp: argument errors, four shapes, 2 / 4 / 8 bits)
    against the oracle's sequential restatement of dnn_fused_dequant_gemv_f32.  The device sums a row in another order, so
    the bar is f32 summation error: 2e-6 of the sum of the products' magnitudes (measured: 1.5e-7)."""
    exe = _build(tmp_path, "fused_gemv_test")
    out = str(tmp_path / "gemv.bin")
    res = subprocess.run([exe, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, f"rc={res.returncode} {res.stderr}"
    raw = np.fromfile(out, dtype=np.uint8)
    pos, seen = 0, []
    while pos < raw.size:
        rows, cols, group, bits = (int(v) for v in raw[pos:pos + 32].view(np.int64))
        pos += 32
        words, ngroups = rows * cols * bits // 32, rows * cols // group
        w = raw[pos:pos + 4 * words].view(np.uint32); pos += 4 * words
        s = raw[pos:pos + 4 * ngroups].view(np.float32); pos += 4 * ngroups
        x = raw[pos:pos + 4 * cols].view(np.float32); pos += 4 * cols
        y = raw[pos:pos + 4 * rows].view(np.float32); pos += 4 * rows
        y_ref = orc.ref_dnn_fused_dequant_gemv(w, s, x, rows, cols, group, bits)
        epw = 32 // bits
        mag = np.zeros(rows, np.float64)
        for r0 in range(0, rows, 1024):                                  # in blocks of rows: the large case would need a gigabyte at once
            wb = w.reshape(rows, -1)[r0:r0 + 1024]
            codes = ((wb[:, :, None] >> (np.arange(epw, dtype=np.uint32) * bits)) & ((1 << bits) - 1)).reshape(wb.shape[0], cols).astype(np.float32)
            mag[r0:r0 + 1024] = (codes * np.repeat(s.reshape(rows, -1)[r0:r0 + 1024], group, axis=1) * np.abs(x)[None, :]).sum(axis=1, dtype=np.float64)
        assert np.isfinite(y).all() and np.all(np.abs(y.astype(np.float64) - y_ref) <= 2e-6 * mag + 1e-12), (rows, cols, group, bits)
        seen.append((rows, cols, group, bits))
    assert seen == [(100, 256, 64, 4), (14336, 4096, 128, 4), (67, 512, 128, 8), (33, 1024, 64, 2)]

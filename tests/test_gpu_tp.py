"""GPU parity of the tensor-parallel quantized SwiGLU MLP against the oracle that applies the same
quantization points (oracle.spec_tp_mlp).  Single GPU: the ranks of a tp=2 / tp=4 layer are built one after
the other on cuda:0 and their partials summed in rank order (what RowLinear::all_reduce does on the host).
Two or more GPUs: real processes, NCCL all-reduce."""
import os
import socket

import numpy as np
import pytest
import torch

from tests.gpu_util import bf16_bits, bf16_dev

pytestmark = pytest.mark.gpu
MAX_REL = 1e-2


def _weights(orc, hidden, inter):
    return (orc.gaussian((inter, hidden), 0.05, 0), orc.gaussian((inter, hidden), 0.05, 2), orc.gaussian((hidden, inter), 0.05, 3))


@pytest.mark.parametrize("variant", ["fp8", "w4a16"])
@pytest.mark.parametrize("m", [1, 64, 300])
@pytest.mark.parametrize("tp", [1, 2, 4])
def test_tp_mlp_partials_one_gpu(orc, variant, m, tp):
    from oxicuda_b200.dist_infer import TpSwiGluMlp
    hidden, inter = 512, 2048
    wg, wu, wd = _weights(orc, hidden, inter)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 1))
    x = bf16_dev(xb)
    acc = None
    hs = []
    for r in range(tp):
        layer = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), variant, tp=tp, rank=r)
        layer.keep_h = True
        part = layer.forward_partial(x).float()
        acc = part if acc is None else acc + part
        if variant == "fp8":
            hs.append(bf16_bits(layer.last_h))
    torch.cuda.synchronize()
    from oxicuda_b200 import ops
    assert ops.handle().device_status() == 0
    got = acc.to(torch.bfloat16).float().cpu().numpy()
    _check_against_oracle(orc, got, xb, wg, wu, wd, tp, variant, hs, (variant, m, tp))


def _check_against_oracle(orc, got, xb, wg, wu, wd, tp, variant, hs, tag):
    """Both GEMMs of the layer at the 1e-2 bar.  FP8: h of every rank against the oracle's h, then the layer output against
    the oracle continued from those very h values (the E4M3 codes of h are a step function of h: see spec_tp_mlp)."""
    assert np.isfinite(got).all()
    if variant == "fp8":
        ref_own, own_h = orc.spec_tp_mlp(xb, wg, wu, wd, tp, variant, return_h=True)
        for r in range(tp):
            h_gpu, h_ref = orc.bf16_bits_to_f32(hs[r]), orc.bf16_bits_to_f32(own_h[r])
            assert np.abs(h_gpu - h_ref).max() <= MAX_REL * np.abs(h_ref).max(), (tag, "h", r)
        ref = orc.bf16_bits_to_f32(orc.spec_tp_mlp(xb, wg, wu, wd, tp, variant, h_bits_per_rank=hs))
    else:
        ref = orc.bf16_bits_to_f32(orc.spec_tp_mlp(xb, wg, wu, wd, tp, variant))
    scale = np.abs(ref).max()
    assert np.abs(got - ref).max() <= MAX_REL * scale, (tag, np.abs(got - ref).max() / scale)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _nccl_rank(rank, world, port, variant, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import oracle as orc
    from oxicuda_b200.dist_infer import TpSwiGluMlp
    hidden, inter, m = 512, 2048, 520
    wg, wu, wd = _weights(orc, hidden, inter)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 1))
    x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
    errs = []
    layer = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), variant, tp=world, rank=rank)
    layer.keep_h = True
    y1 = layer.forward(x)
    y1_host = y1.float().cpu().numpy()
    hs = None
    if variant == "fp8":                                    # every rank's h, so that the oracle can continue from the same values
        mine = layer.last_h.contiguous()
        allh = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allh, mine)
        hs = [t.view(torch.int16).cpu().numpy().view(np.uint16) for t in allh]
        ref_own, own_h = orc.spec_tp_mlp(xb, wg, wu, wd, world, variant, return_h=True)
        for r in range(world):
            a, b = orc.bf16_bits_to_f32(hs[r]), orc.bf16_bits_to_f32(own_h[r])
            errs.append(float(np.abs(a - b).max() / np.abs(b).max()))
    ref = orc.bf16_bits_to_f32(orc.spec_tp_mlp(xb, wg, wu, wd, world, variant, h_bits_per_rank=hs))
    errs.append(float(np.abs(y1_host - ref).max() / np.abs(ref).max()))
    # a second call on other activations must leave the first result as it was (eager results do not alias the layer's buffers)
    y2 = layer.forward(x * 0.5)
    torch.cuda.synchronize()
    errs.append(0.0 if np.array_equal(y1.float().cpu().numpy(), y1_host) and not torch.equal(y1, y2) else 1.0)
    # M-chunk pipelining: per-chunk activation scales on both sides, no h hand-over (sanity bound only: the E4M3 codes of h
    # are a step function of h, so this path is not held to the per-GEMM bar)
    layer2 = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), variant, tp=world, rank=rank, overlap_chunks=2)
    y = layer2.forward(x).float().cpu().numpy()
    ref2 = orc.bf16_bits_to_f32(orc.spec_tp_mlp(xb, wg, wu, wd, world, variant, m_chunks=2))
    errs.append(float(np.abs(y - ref2).max() / np.abs(ref2).max()) / (1.0 if variant == "w4a16" else 3.0))
    q.put((rank, errs))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("variant", ["fp8", "w4a16"])
def test_tp_mlp_nccl_two_gpus(variant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_nccl_rank, args=(r, 2, port, variant, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, errs in res:
        for e in errs:
            assert e <= MAX_REL, errs


def _fused_rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["OXQ_TP_FUSED_REDUCE"] = "1"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import oracle as orc
    from oxicuda_b200 import ops
    from oxicuda_b200.dist_infer import TpSwiGluMlp
    errs = []
    for (hidden, inter, ms) in ((512, 2048, (520, 300, 520, 1024)), (2048, 4096, (2048, 2048, 2048))):
        wg, wu, wd = _weights(orc, hidden, inter)
        layer = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), "fp8", tp=world, rank=rank)
        if not layer.fused_reduce:                           # no multicast mapping on this fabric: nothing to test
            q.put((rank, None))
            dist.barrier()
            dist.destroy_process_group()
            return
        plain = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), "fp8", tp=world, rank=rank)
        plain.fused_reduce = False
        plain.split_reduce = False
        for i, m in enumerate(ms):
            xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 20 + i))
            x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
            y = layer.forward(x)
            want = plain.forward(x)                          # GEMM, barrier, in-switch reduce, barrier: the same bf16 partials, the same sum
            torch.cuda.synchronize()
            assert layer._fused_calls == i + 1
            errs.append(float((y.float() - want.float()).abs().max() / want.float().abs().max()))
        m = ms[-1]
        xs, ys, gr = layer.capture(m)                        # replays alternate between the two sets of flag words like host calls do
        for i in range(5):
            xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 80 + i))
            x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
            xs.copy_(x)
            gr.replay()
            got = ys.clone()
            want = plain.forward(x)
            torch.cuda.synchronize()
            errs.append(float((got.float() - want.float()).abs().max() / want.float().abs().max()))
        errs.append(float(ops.handle(torch.cuda.current_device()).device_status()))
    q.put((rank, errs))
    dist.barrier()
    dist.destroy_process_group()


def _sync_rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import oracle as orc
    from oxicuda_b200 import ops
    from oxicuda_b200.dist_infer import TpSwiGluMlp
    hidden, inter = 1024, 2048
    wg, wu, wd = _weights(orc, hidden, inter)
    layer = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), "fp8", tp=world, rank=rank)
    plain = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), "fp8", tp=world, rank=rank)
    if not layer.use_multimem:
        q.put((rank, None))
        dist.barrier()
        dist.destroy_process_group()
        return
    layer.sync_reduce, plain.sync_reduce = True, False
    errs = []
    for i, m in enumerate((1024, 1, 520, 7, 64, 1024)):       # split path, fewer rows than ranks, one block, odd rows
        xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 40 + i))
        x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
        y = layer.forward(x)
        want = plain.forward(x)
        torch.cuda.synchronize()
        errs.append(float((y.float() - want.float()).abs().max() / want.float().abs().max()))
    assert layer._sync_calls >= 6
    # the same launches replayed from a CUDA graph: every replay has to wait for its own generation of signals
    for m in (1024, 64):
        xs, ys, gr = layer.capture(m)
        for i in range(5):
            xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 60 + i))
            x = torch.from_numpy(xb.view(np.int16)).cuda().view(torch.bfloat16)
            xs.copy_(x)
            gr.replay()
            got = ys.clone()
            want = plain.forward(x)
            torch.cuda.synchronize()
            errs.append(float((got.float() - want.float()).abs().max() / want.float().abs().max()))
    errs.append(float(ops.handle(torch.cuda.current_device()).device_status()))
    q.put((rank, errs))
    dist.barrier()
    dist.destroy_process_group()


def test_tp_mlp_sync_reduce_two_gpus():
    """The in-switch reduce that synchronises the ranks through flag words inside the kernel against the same reduce between
    cross-rank barrier kernels: identical sums, over the split path, single blocks and batches smaller than the group."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sync_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, errs in res:
        if errs is None:
            pytest.skip("no multicast mapping")
        for e in errs:
            assert e <= 1e-6, errs


def test_tp_mlp_fused_reduce_two_gpus():
    """The down projection with the all-reduce fused in (tiles summed in the switch under the MMAs of later tiles) against
    the unfused in-switch path: several calls (both sets of flag words, changing tile counts), two layer sizes."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_fused_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for _, errs in res:
        if errs is None:
            pytest.skip("no multicast mapping")
        for e in errs:
            assert e <= 1e-6, errs                           # the same partials through the same reduction: identical results


@pytest.fixture(scope="module")
def llama70b_weights(orc):
    """Gate, up and down weights of the benchmark's layer (hidden 8192, intermediate 28672), N(0, 0.02).  One Gaussian
    matrix is drawn; the other two are a row rotation and a transposed column rotation of it (drawing 705 M samples three
    times over would take longer than everything the GPU does in this file)."""
    hidden, inter = 8192, 28672
    wg = orc.gaussian((inter, hidden), 0.02, 0)
    wu = np.roll(wg, 977, axis=0)
    wd = np.ascontiguousarray(np.roll(wg, 131, axis=1).T)
    return wg, wu, wd


@pytest.mark.parametrize("variant", ["fp8", "w4a16"])
@pytest.mark.parametrize("m", [1, 64])
def test_tp_mlp_llama70b_shape_one_gpu(orc, llama70b_weights, variant, m):
    """The benchmark's layer at its real size (hidden 8192, intermediate 28672), tp = 8 with the ranks emulated one
    after the other on one GPU: every rank's kernels see exactly the shard shapes of the 8-GPU run."""
    from oxicuda_b200.dist_infer import TpSwiGluMlp
    hidden, inter, tp = 8192, 28672, 8
    wg, wu, wd = llama70b_weights
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 1))
    x = bf16_dev(xb)
    sh = inter // tp
    acc, hs = None, []
    for r in range(tp):
        layer = TpSwiGluMlp(torch.from_numpy(wg[r * sh:(r + 1) * sh]), torch.from_numpy(wu[r * sh:(r + 1) * sh]),
                            torch.from_numpy(np.ascontiguousarray(wd[:, r * sh:(r + 1) * sh])), variant, tp=tp, rank=r, already_sharded=True)
        layer.keep_h = True
        part = layer.forward_partial(x).float()
        acc = part if acc is None else acc + part
        if variant == "fp8":
            hs.append(bf16_bits(layer.last_h))
        del layer
    torch.cuda.synchronize()
    from oxicuda_b200 import ops
    assert ops.handle().device_status() == 0
    got = acc.to(torch.bfloat16).float().cpu().numpy()
    _check_against_oracle(orc, got, xb, wg, wu, wd, tp, variant, hs, (variant, m, "llama70b"))


# ---- single column- / row-parallel linears ---------------------------------------------------------

def _fp8_linear_ref(orc, xb, w_shard, bias):
    """Oracle for one shard of the "fp8" linears: per-tensor E4M3 of the bf16 operands, exact product, bf16 output,
    then the f32 bias added and rounded to bf16 once more."""
    x = orc.bf16_bits_to_f32(xb)
    wb = orc.f32_to_bf16_bits(w_shard)
    sx, sw = orc.spec_fp8_scale(orc.spec_absmax(xb)), orc.spec_fp8_scale(orc.spec_absmax(wb))
    xq = orc.spec_fp8_dequant(orc.spec_fp8_quant(xb, sx), 1.0)
    wq = orc.spec_fp8_dequant(orc.spec_fp8_quant(wb, sw), 1.0)
    y = (xq.astype(np.float64) @ wq.astype(np.float64).T).astype(np.float32) * (np.float32(sx) * np.float32(sw))
    y = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(y))
    if bias is not None:
        y = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(y + bias[None, :]))
    del x
    return y


@pytest.mark.parametrize("variant", ["fp8", "bf16"])
@pytest.mark.parametrize("tp", [1, 2, 4])
def test_column_linear_one_gpu(orc, variant, tp):
    from oxicuda_b200.dist_infer import ColumnLinear
    in_f, out_f, batch = 256, 512, 5
    w = orc.gaussian((out_f, in_f), 0.05, 0)
    b = orc.gaussian((1, out_f), 1.0, 4).ravel()
    xb = orc.f32_to_bf16_bits(orc.gaussian((batch, in_f), 1.0, 1))
    x = bf16_dev(xb)
    shards, refs = [], []
    for r in range(tp):
        layer = ColumnLinear.from_full_weight(in_f, out_f, torch.from_numpy(w), torch.from_numpy(b), tp=tp, rank=r, variant=variant)
        shards.append(layer.local_forward(x).float().cpu())
        rows = slice(r * out_f // tp, (r + 1) * out_f // tp)
        if variant == "fp8":
            refs.append(_fp8_linear_ref(orc, xb, w[rows], b[rows]))
        else:
            wr = orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(w[rows]))
            refs.append((orc.bf16_bits_to_f32(xb).astype(np.float64) @ wr.astype(np.float64).T).astype(np.float32) + b[rows][None, :])
    got = ColumnLinear.gather_shards(out_f, batch, shards).numpy()
    ref = np.concatenate(refs, axis=1)
    scale = np.abs(ref).max()
    assert got.shape == (batch, out_f) and np.isfinite(got).all()
    assert np.abs(got - ref).max() <= MAX_REL * scale


@pytest.mark.parametrize("variant", ["fp8", "bf16"])
@pytest.mark.parametrize("tp", [1, 2, 4])
def test_row_linear_one_gpu(orc, variant, tp):
    from oxicuda_b200.dist_infer import RowLinear
    in_f, out_f, batch = 512, 256, 7
    w = orc.gaussian((out_f, in_f), 0.05, 0)
    b = orc.gaussian((1, out_f), 1.0, 4).ravel()
    xb = orc.f32_to_bf16_bits(orc.gaussian((batch, in_f), 1.0, 1))
    x = bf16_dev(xb)
    parts = []
    for r in range(tp):
        layer = RowLinear.from_full_weight(out_f, in_f, torch.from_numpy(w), torch.from_numpy(b), tp=tp, rank=r, variant=variant)
        assert (layer.bias is not None) == (r == 0)                                  # bias on rank 0 only
        parts.append(layer.local_forward(x).float().cpu())
    got = RowLinear.reduce_partials(parts).numpy()
    ref = orc.ref_linear_f32(orc.bf16_bits_to_f32(xb), w, b)
    scale = np.abs(ref).max()
    tol = (4.0 if variant == "fp8" else 1.0) * MAX_REL * scale                       # E4M3 operands: 2^-4 relative steps, averaged over K
    assert np.isfinite(got).all() and np.abs(got - ref).max() <= tol


def _linear_rank(rank, world, port, q):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from oracle import oracle as orc
    from oxicuda_b200.dist_infer import ColumnLinear, RowLinear
    in_f, mid, batch = 256, 512, 9
    w1, w2 = orc.gaussian((mid, in_f), 0.05, 0), orc.gaussian((in_f, mid), 0.05, 2)
    x = torch.from_numpy(orc.gaussian((batch, in_f), 1.0, 1)).to(torch.bfloat16).cuda()
    col = ColumnLinear.from_full_weight(in_f, mid, torch.from_numpy(w1), None, tp=world, rank=rank, variant="bf16")
    row = RowLinear.from_full_weight(in_f, mid, torch.from_numpy(w2), None, tp=world, rank=rank, variant="bf16")
    h = col.forward(x)                                     # all-gather of the column shards
    y = row.forward(h)                                     # slice, partial product, all-reduce
    torch.cuda.synchronize()
    xf = x.float().cpu().numpy()
    h_ref = xf @ w1.T
    y_ref = h_ref @ w2.T
    q.put((rank, float(np.abs(h.float().cpu().numpy() - h_ref).max() / np.abs(h_ref).max()),
           float(np.abs(y.float().cpu().numpy() - y_ref).max() / np.abs(y_ref).max())))
    dist.barrier()
    dist.destroy_process_group()


def test_column_then_row_linear_nccl_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_linear_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, eh, ey in res:
        assert eh <= 1e-2 and ey <= 2e-2


# ---- the layer through the C ABI alone -------------------------------------------------------------------------------

def _nccl_lib_dir():
    import importlib.util
    spec = importlib.util.find_spec("nvidia.nccl")
    if spec is None or not spec.submodule_search_locations:
        return None
    d = os.path.join(list(spec.submodule_search_locations)[0], "lib")
    return d if os.path.exists(os.path.join(d, "libnccl.so.2")) else None


@pytest.mark.parametrize("m", [4, 300])
def test_tp_mlp_c_abi_two_ranks(tmp_path, orc, m):
    """oxq_comm_init + oxq_mlp_swiglu_tp from a C++ program, one process per rank and GPU, no Python in the ranks: each rank's
    partial equals, bit for bit, what the Python layer computes for the same shard (whose parity with the oracle the tests
    above establish), both ranks hold the same reduced result, and it is the bf16 sum of the two partials."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import subprocess
    from oxicuda_b200 import _build
    from oxicuda_b200.dist_infer import TpSwiGluMlp, interleave_gate_up
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "oxicuda_b200", "lib")
    exe = str(tmp_path / "tp_mlp_test")
    cmd = ["/usr/bin/g++", "-std=c++17", "-O1", "-I/usr/local/cuda/include", os.path.join(root, "tests", "cpp", "tp_mlp_test.cpp"),
           "-o", exe, "-L" + libdir, "-loxq_b200", "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath," + libdir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    hidden, inter, tp = 512, 2048, 2
    il = inter // tp
    wg, wu, wd = _weights(orc, hidden, inter)
    xb = orc.f32_to_bf16_bits(orc.gaussian((m, hidden), 1.0, 1))
    xb.tofile(str(tmp_path / "x.bin"))
    x = bf16_dev(xb)
    want_parts = []
    for r in range(tp):
        g, u = torch.from_numpy(wg[r * il:(r + 1) * il]), torch.from_numpy(wu[r * il:(r + 1) * il])
        d = torch.from_numpy(np.ascontiguousarray(wd[:, r * il:(r + 1) * il]))
        bf16_bits(interleave_gate_up(g, u).to(torch.bfloat16)).tofile(str(tmp_path / f"rank{r}_wgu.bin"))
        bf16_bits(d.to(torch.bfloat16)).tofile(str(tmp_path / f"rank{r}_wd.bin"))
        layer = TpSwiGluMlp(g.to(torch.bfloat16), u.to(torch.bfloat16), d.to(torch.bfloat16), "fp8", tp=tp, rank=r, already_sharded=True)
        want_parts.append(bf16_bits(layer.forward_partial(x)))
    env = dict(os.environ)
    nccl_dir = _nccl_lib_dir()
    if nccl_dir:
        env["OXQ_NCCL_LIB"] = os.path.join(nccl_dir, "libnccl.so.2")
    env["NCCL_NVLS_ENABLE"] = "0"
    run = subprocess.run([exe, str(tmp_path), str(tp), str(m), str(hidden), str(il)], capture_output=True, text=True, timeout=600, env=env)
    assert run.returncode == 0, f"rc={run.returncode} {run.stdout[-2000:]} {run.stderr[-2000:]}"
    parts = [np.fromfile(str(tmp_path / f"rank{r}_partial.bin"), np.uint16).reshape(m, hidden) for r in range(tp)]
    ys = [np.fromfile(str(tmp_path / f"rank{r}_y.bin"), np.uint16).reshape(m, hidden) for r in range(tp)]
    for r in range(tp):
        assert np.array_equal(parts[r], want_parts[r]), f"rank {r}: partial differs from the Python layer's"
    assert np.array_equal(ys[0], ys[1])
    total = orc.bf16_bits_to_f32(parts[0]) + orc.bf16_bits_to_f32(parts[1])                  # one addition: the bf16 rounding of the f32 sum
    assert np.array_equal(ys[0], orc.f32_to_bf16_bits(total))
    for r in range(tp):                                                                       # rank-major gather of the first 1024 elements
        gth = np.fromfile(str(tmp_path / f"rank{r}_gather.bin"), np.uint16)
        assert np.array_equal(gth, np.concatenate([parts[q].ravel()[:1024] for q in range(tp)]))

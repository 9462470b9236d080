"""GPU parity of the tensor-parallel quantized SwiGLU MLP against the oracle that applies the same
quantization points (oracle.spec_tp_mlp).  Single GPU: the ranks of a tp=2 / tp=4 layer are built one after
the other on cuda:0 and their partials summed in rank order (what RowLinear::all_reduce does on the host).
Two or more GPUs: real processes, NCCL all-reduce."""
import os
import socket

import numpy as np
import pytest
import torch

from tests.gpu_util import bf16_dev

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
    for r in range(tp):
        layer = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), variant, tp=tp, rank=r)
        part = layer.forward_partial(x).float()
        acc = part if acc is None else acc + part
    torch.cuda.synchronize()
    from oxicuda_b200 import ops
    assert ops.handle().device_status() == 0
    got = acc.to(torch.bfloat16).float().cpu().numpy()
    ref = orc.bf16_bits_to_f32(orc.spec_tp_mlp(xb, wg, wu, wd, tp, variant))
    scale = np.abs(ref).max()
    assert np.isfinite(got).all()
    assert np.abs(got - ref).max() <= MAX_REL * scale * (2.0 if variant == "fp8" else 1.0), (variant, m, tp, np.abs(got - ref).max() / scale)


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
    for chunks in (1, 2):
        layer = TpSwiGluMlp(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), variant, tp=world, rank=rank,
                            overlap_chunks=chunks)
        y = layer.forward(x).float().cpu().numpy()
        ref = orc.bf16_bits_to_f32(orc.spec_tp_mlp(xb, wg, wu, wd, world, variant, m_chunks=chunks))
        errs.append(float(np.abs(y - ref).max() / np.abs(ref).max()))
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
            assert e <= 2 * MAX_REL

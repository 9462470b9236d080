"""Host-side logic of the tensor-parallel MLP on CPU: shard index arithmetic against the reference's
`from_full_weight` rules, and a world_size-2 gloo run in which each rank computes its partial with the
oracle (as a stand-in for the GPU kernels) on the shards the product code cut, then all-reduces."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oxicuda_b200 import dist_infer as di


def test_shard_index_rules():
    assert di.column_shard_rows(28672, 8, 3) == slice(3 * 3584, 4 * 3584)          # column_parallel.rs:115-166
    assert di.row_shard_cols(28672, 8, 7) == slice(7 * 3584, 28672)                # row_parallel.rs:109-168
    with pytest.raises(ValueError):
        di.column_shard_rows(100, 8, 0)                                            # NotDivisible
    with pytest.raises(ValueError):
        di.column_shard_rows(128, 4, 4)                                            # rank outside the world
    wg = torch.arange(8 * 4, dtype=torch.float32).reshape(8, 4)
    wu = wg + 100
    wd = torch.arange(4 * 8, dtype=torch.float32).reshape(4, 8)
    g, u, d = di.shard_mlp_weights(wg, wu, wd, 2, 1)
    assert torch.equal(g, wg[4:]) and torch.equal(u, wu[4:]) and torch.equal(d, wd[:, 4:])


def test_interleave_layout():
    wg = torch.arange(256 * 2, dtype=torch.float32).reshape(256, 2)
    wu = -wg
    w = di.interleave_gate_up(wg, wu)
    assert w.shape == (512, 2)
    assert torch.equal(w[:128], wg[:128]) and torch.equal(w[128:256], wu[:128])
    assert torch.equal(w[256:384], wg[128:]) and torch.equal(w[384:], wu[128:])
    with pytest.raises(ValueError):
        di.interleave_gate_up(wg[:100], wu[:100])


def test_spec_tp_mlp_matches_unsharded_f32(orc):
    """The quantized TP oracle stays close to the reference's f32 SwiGluFfn and is independent of tp up to rounding."""
    x = orc.f32_to_bf16_bits(orc.gaussian((4, 256), 1.0, 1))
    wg, wu, wd = orc.gaussian((512, 256), 0.05, 0), orc.gaussian((512, 256), 0.05, 2), orc.gaussian((256, 512), 0.05, 3)
    full = orc.ref_swiglu_mlp(orc.bf16_bits_to_f32(x), wg, wu, wd)
    for variant, tol in (("fp8", 0.08), ("w4a16", 0.15)):
        y1 = orc.bf16_bits_to_f32(orc.spec_tp_mlp(x, wg, wu, wd, 1, variant))
        y4 = orc.bf16_bits_to_f32(orc.spec_tp_mlp(x, wg, wu, wd, 4, variant))
        scale = np.abs(full).max()
        assert np.abs(y1 - full).max() <= tol * scale
        assert np.abs(y4 - y1).max() <= tol * scale


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import oracle as orc
    x = orc.gaussian((3, 256), 1.0, 1)
    wg, wu, wd = orc.gaussian((512, 256), 0.05, 0), orc.gaussian((512, 256), 0.05, 2), orc.gaussian((256, 512), 0.05, 3)
    g, u, d = di.shard_mlp_weights(torch.from_numpy(wg), torch.from_numpy(wu), torch.from_numpy(wd), world, rank)
    w_gu = di.interleave_gate_up(g, u).numpy()
    gu = orc.ref_linear_f32(x, w_gu)                                   # [3 x 2*inter_local], interleaved blocks
    t = gu.reshape(3, -1, 2, 128)
    h = orc.ref_silu_mul(t[:, :, 0].reshape(3, -1), t[:, :, 1].reshape(3, -1))
    part = torch.from_numpy(orc.ref_linear_f32(h, d.numpy()))
    dist.all_reduce(part, op=dist.ReduceOp.SUM)
    full = orc.ref_swiglu_mlp(x, wg, wu, wd)
    out_q.put((rank, float(np.abs(part.numpy() - full).max()), float(np.abs(full).max())))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_all_reduce_matches_unsharded():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for _, err, scale in res:
        assert err <= 1e-5 * scale

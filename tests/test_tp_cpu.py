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


# ---- ColumnLinear / RowLinear host logic -----------------------------------------------------------

def _shard_outputs_column(orc, x, w, b, tp):
    """What each rank's ColumnLinear computes, with the product's shard indices and the oracle's f32 linear."""
    outs = []
    for r in range(tp):
        rows = di.column_shard_rows(w.shape[0], tp, r)
        outs.append(torch.from_numpy(orc.ref_linear_f32(x, w[rows], None if b is None else b[rows])))
    return outs


def test_column_linear_reference_cases(orc):  # crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:224-290
    w = np.eye(4, dtype=np.float32)
    x = np.array([[1.0, 2.0, 3.0, 4.0]], np.float32)
    out = di.ColumnLinear.gather_shards(4, 1, _shard_outputs_column(orc, x, w, None, 2))
    assert out.tolist() == [[1.0, 2.0, 3.0, 4.0]]
    out = di.ColumnLinear.gather_shards(4, 2, _shard_outputs_column(orc, np.ones((2, 2), np.float32), np.ones((4, 2), np.float32), None, 4))
    assert out.tolist() == [[2.0] * 4, [2.0] * 4]
    out = di.ColumnLinear.gather_shards(2, 1, _shard_outputs_column(orc, np.zeros((1, 2), np.float32), np.zeros((2, 2), np.float32),
                                                                    np.array([10.0, 20.0], np.float32), 2))
    assert out.tolist() == [[10.0, 20.0]]


def test_linear_constructor_errors():  # column_parallel.rs:292-330, row_parallel.rs:109-168
    from oxicuda_b200.errors import DistInferError
    w = torch.zeros(4 * 2)
    with pytest.raises(DistInferError) as e:
        di.ColumnLinear.from_full_weight(2, 4, w, None, tp=3, rank=0)
    assert e.value.variant == "TpFeaturesMisaligned"
    with pytest.raises(DistInferError) as e:
        di.ColumnLinear.from_full_weight(2, 4, torch.zeros(7), None, tp=2, rank=0)
    assert e.value.variant == "DimensionMismatch"
    with pytest.raises(DistInferError) as e:
        di.ColumnLinear.from_full_weight(2, 4, w, torch.zeros(3), tp=2, rank=0)
    assert e.value.variant == "DimensionMismatch"
    with pytest.raises(DistInferError) as e:
        di.RowLinear.from_full_weight(2, 4, w, None, tp=3, rank=0)
    assert e.value.variant == "TpInputMisaligned"
    with pytest.raises(DistInferError) as e:
        di.RowLinear.from_full_weight(2, 4, torch.zeros(9), None, tp=2, rank=1)
    assert e.value.variant == "DimensionMismatch"
    with pytest.raises(DistInferError) as e:
        di.ColumnLinear.gather_shards(4, 1, [])
    assert e.value.variant == "TooFewRanks"
    with pytest.raises(DistInferError) as e:
        di.RowLinear.reduce_partials([])
    assert e.value.variant == "TooFewRanks"
    with pytest.raises(DistInferError) as e:
        di.RowLinear.reduce_partials([torch.zeros(4), torch.zeros(5)])
    assert e.value.variant == "DimensionMismatch"


def test_row_linear_partials_sum_to_full(orc):  # row_parallel.rs: bias on rank 0 only, partials summed in rank order
    x = orc.gaussian((3, 64), 1.0, 1)
    w = orc.gaussian((16, 64), 0.1, 2)
    b = orc.gaussian((1, 16), 1.0, 3).ravel()
    parts = []
    for r in range(4):
        cols = di.row_shard_cols(64, 4, r)
        parts.append(torch.from_numpy(orc.ref_linear_f32(np.ascontiguousarray(x[:, cols]), np.ascontiguousarray(w[:, cols]), b if r == 0 else None)))
    full = orc.ref_linear_f32(x, w, b)
    assert np.allclose(di.RowLinear.reduce_partials(parts).numpy(), full, rtol=1e-5, atol=1e-5)


def _gather_main(rank, world, port, out_q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    local = torch.arange(6, dtype=torch.float32).reshape(2, 3) + 100 * rank          # [batch 2 x local_out 3]
    full = di.gather_columns(local, world)
    out_q.put((rank, full.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_column_gather_layout():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gather_main, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = [[0.0, 1.0, 2.0, 100.0, 101.0, 102.0], [3.0, 4.0, 5.0, 103.0, 104.0, 105.0]]
    for _, full in res:
        assert full == want

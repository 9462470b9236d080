"""Tensor-parallel SwiGLU MLP over the quantized GEMMs: the host-side mirror of ColumnLinear / RowLinear
(crates/oxicuda-dist-infer/src/tensor_parallel/{column_parallel,row_parallel}.rs) and SwiGluFfn
(crates/oxicuda-lm/src/layer/ffn.rs:202-254).

Sharding (identical to the reference's `from_full_weight` constructors):
  * gate and up weights [inter x hidden] are split by output rows, rank r owns rows [r*inter/tp, (r+1)*inter/tp)
    (ColumnLinear::from_full_weight, column_parallel.rs:115-166);
  * the down weight [hidden x inter] is split by input columns, rank r owns columns [r*inter/tp, (r+1)*inter/tp)
    of every row (RowLinear::from_full_weight, row_parallel.rs:109-168);
  * h = silu(gate) * up is local (column shard r of gate/up is exactly the K slice the down shard r needs, so
    ColumnLinear::all_gather is not needed);
  * each rank produces a full [M x hidden] partial and one all-reduce(sum) combines them
    (RowLinear::all_reduce, row_parallel.rs:199-223); the reference sums on the host in rank order, here it
    is one NCCL all-reduce over NVLink, issued through torch.distributed.

One process per GPU.  All arithmetic runs in liboxq_b200.so; torch supplies device memory, streams and the
process group.
"""
from __future__ import annotations

import torch

VARIANTS = ("fp8", "w4a16")


# ------------------------------------------------------------------------------------------------ sharding (host logic)

def column_shard_rows(total_out: int, tp: int, rank: int) -> slice:
    """Rows of a column-parallel weight owned by `rank` (column_parallel.rs:115-166).  total_out must divide."""
    if tp < 1 or not (0 <= rank < tp):
        raise ValueError(f"rank {rank} outside world of {tp}")
    if total_out % tp != 0:
        raise ValueError(f"features {total_out} not divisible by degree {tp}")       # DistInferError::NotDivisible
    sh = total_out // tp
    return slice(rank * sh, (rank + 1) * sh)


def row_shard_cols(total_in: int, tp: int, rank: int) -> slice:
    """Input columns of a row-parallel weight owned by `rank` (row_parallel.rs:109-168)."""
    return column_shard_rows(total_in, tp, rank)


def shard_mlp_weights(w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, tp: int, rank: int):
    """(gate shard [inter/tp x hidden], up shard, down shard [hidden x inter/tp]) of rank `rank`."""
    inter = w_gate.shape[0]
    rows = column_shard_rows(inter, tp, rank)
    return w_gate[rows].contiguous(), w_up[rows].contiguous(), w_down[:, row_shard_cols(inter, tp, rank)].contiguous()


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """Blocks of 128 gate rows followed by the 128 matching up rows: the layout the fused SwiGLU epilogue reads."""
    inter, k = w_gate.shape
    if inter % 128 != 0:
        raise ValueError(f"intermediate shard of {inter} rows is not a multiple of 128")
    return torch.stack([w_gate.reshape(inter // 128, 128, k), w_up.reshape(inter // 128, 128, k)], dim=1).reshape(2 * inter, k).contiguous()


# ------------------------------------------------------------------------------------------------ single linears

LINEAR_VARIANTS = ("fp8", "bf16")


def _dist_error(variant: str, msg: str):
    from .errors import DistInferError
    return DistInferError(variant, msg)


class _ShardedLinear:
    """One rank's weight shard on the GPU: E4M3 with a per-shard scale ("fp8", activations quantised per call)
    or bf16.  y = bf16(x . W_shard^T) (+ bias)."""

    def _load(self, w_shard: torch.Tensor, bias, variant: str):
        from . import ops
        if variant not in LINEAR_VARIANTS:
            raise ValueError(f"variant {variant!r} not in {LINEAR_VARIANTS}")
        self.ops, self.variant = ops, variant
        dev = torch.device("cuda", torch.cuda.current_device())
        w = w_shard.to(dev).contiguous()
        if variant == "fp8":
            self.w_q, st = ops.fp8_quant_dynamic(w.to(torch.bfloat16))
            self.s_w = st[1:].clone()
        else:
            self.w = w.to(torch.bfloat16)
        self.bias = None if bias is None else bias.to(dev, torch.float32).contiguous()

    def _matmul(self, x: torch.Tensor) -> torch.Tensor:
        ops = self.ops
        if self.variant == "fp8":
            xq, sx = ops.fp8_quant_dynamic(x)
            y = ops.gemm_fp8(xq, self.w_q, sx[1:], self.s_w)
        else:
            y = ops.gemm_bf16(x, self.w)
        if self.bias is not None:
            ops.bias_add_(y, self.bias)
        return y


def gather_columns(local: torch.Tensor, tp: int, group=None) -> torch.Tensor:
    """All-gather of column shards: local [batch x local_out] on every rank -> [batch x tp*local_out], rank r's
    columns at [r*local_out, (r+1)*local_out) (ColumnLinear::all_gather, column_parallel.rs:181-204)."""
    import torch.distributed as dist
    if tp == 1:
        return local
    batch, lo = local.shape
    stacked = torch.empty((tp * batch, lo), dtype=local.dtype, device=local.device)     # rank-major concatenation
    dist.all_gather_into_tensor(stacked, local.contiguous(), group=group)
    return stacked.view(tp, batch, lo).permute(1, 0, 2).reshape(batch, tp * lo)


class ColumnLinear(_ShardedLinear):
    """Column-parallel linear: rank r owns output rows [r*total_out/tp, (r+1)*total_out/tp) of W [total_out x in]
    (crates/oxicuda-dist-infer/src/tensor_parallel/column_parallel.rs:103-204)."""

    @classmethod
    def from_full_weight(cls, in_features: int, total_out: int, weight: torch.Tensor, bias: torch.Tensor | None = None,
                         tp: int = 1, rank: int = 0, variant: str = "fp8", group=None):
        if tp < 1 or not (0 <= rank < tp):
            raise _dist_error("TooFewRanks", f"rank {rank} outside a world of {tp}")
        if total_out % tp != 0:
            raise _dist_error("TpFeaturesMisaligned", f"features {total_out} not divisible by degree {tp}")
        if weight.numel() != total_out * in_features:
            raise _dist_error("DimensionMismatch", f"expected {total_out * in_features}, got {weight.numel()}")
        if bias is not None and bias.numel() != total_out:
            raise _dist_error("DimensionMismatch", f"expected {total_out}, got {bias.numel()}")
        self = cls()
        self.in_features, self.total_out, self.tp, self.rank, self.group = in_features, total_out, tp, rank, group
        rows = column_shard_rows(total_out, tp, rank)
        self.local_out, self.col_offset = rows.stop - rows.start, rows.start
        self._load(weight.reshape(total_out, in_features)[rows], None if bias is None else bias.reshape(-1)[rows], variant)
        return self

    def local_forward(self, x: torch.Tensor) -> torch.Tensor:
        """[batch x in] bf16 -> this rank's [batch x local_out] bf16."""
        if x.shape[-1] != self.in_features:
            raise _dist_error("DimensionMismatch", f"expected {self.in_features} input features, got {x.shape[-1]}")
        return self._matmul(x)

    def all_gather(self, local: torch.Tensor) -> torch.Tensor:
        return gather_columns(local, self.tp, self.group)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.all_gather(self.local_forward(x))

    @staticmethod
    def gather_shards(total_out: int, batch: int, shards) -> torch.Tensor:
        """The reference's host-side all_gather over a list of per-rank outputs (column_parallel.rs:181-204)."""
        if len(shards) == 0:
            raise _dist_error("TooFewRanks", "needed 1, world_size 0")
        lo = total_out // len(shards)
        return torch.cat([s.reshape(batch, lo) for s in shards], dim=1)


class RowLinear(_ShardedLinear):
    """Row-parallel linear: rank r owns input columns [r*total_in/tp, (r+1)*total_in/tp) of W [out x total_in]; the
    bias lives on rank 0 only so the all-reduce counts it once
    (crates/oxicuda-dist-infer/src/tensor_parallel/row_parallel.rs:97-223)."""

    @classmethod
    def from_full_weight(cls, out_features: int, total_in: int, weight: torch.Tensor, bias: torch.Tensor | None = None,
                         tp: int = 1, rank: int = 0, variant: str = "fp8", group=None):
        if tp < 1 or not (0 <= rank < tp):
            raise _dist_error("TooFewRanks", f"rank {rank} outside a world of {tp}")
        if total_in % tp != 0:
            raise _dist_error("TpInputMisaligned", f"features {total_in} not divisible by degree {tp}")
        if weight.numel() != out_features * total_in:
            raise _dist_error("DimensionMismatch", f"expected {out_features * total_in}, got {weight.numel()}")
        if bias is not None and rank == 0 and bias.numel() != out_features:
            raise _dist_error("DimensionMismatch", f"expected {out_features}, got {bias.numel()}")
        self = cls()
        self.out_features, self.total_in, self.tp, self.rank, self.group = out_features, total_in, tp, rank, group
        cols = row_shard_cols(total_in, tp, rank)
        self.local_in, self.row_offset = cols.stop - cols.start, cols.start
        self._load(weight.reshape(out_features, total_in)[:, cols], bias.reshape(-1) if (bias is not None and rank == 0) else None, variant)
        return self

    def slice_input(self, full_input: torch.Tensor) -> torch.Tensor:
        if full_input.shape[-1] != self.total_in:
            raise _dist_error("DimensionMismatch", f"expected {self.total_in} input features, got {full_input.shape[-1]}")
        return full_input[:, self.row_offset:self.row_offset + self.local_in].contiguous()

    def forward_partial(self, input_slice: torch.Tensor) -> torch.Tensor:
        if input_slice.shape[-1] != self.local_in:
            raise _dist_error("DimensionMismatch", f"expected {self.local_in} input features, got {input_slice.shape[-1]}")
        return self._matmul(input_slice)

    def local_forward(self, full_input: torch.Tensor) -> torch.Tensor:
        return self.forward_partial(self.slice_input(full_input))

    def all_reduce(self, partial: torch.Tensor) -> torch.Tensor:
        """Sum of the ranks' partials, in place (one collective; RowLinear::all_reduce, row_parallel.rs:199-223)."""
        import torch.distributed as dist
        if self.tp > 1:
            dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=self.group)
        return partial

    def forward(self, full_input: torch.Tensor) -> torch.Tensor:
        return self.all_reduce(self.local_forward(full_input))

    @staticmethod
    def reduce_partials(partials) -> torch.Tensor:
        """The reference's host-side all_reduce over a list of per-rank partials, summed in rank order."""
        if len(partials) == 0:
            raise _dist_error("TooFewRanks", "needed 1, world_size 0")
        acc = partials[0].clone()
        for part in partials[1:]:
            if part.numel() != acc.numel():
                raise _dist_error("DimensionMismatch", f"expected {acc.numel()}, got {part.numel()}")
            acc += part
        return acc


# ------------------------------------------------------------------------------------------------ the layer

class TpSwiGluMlp:
    """One rank's shard of a tensor-parallel SwiGLU MLP with quantized weights.

    variant "fp8":   per-tensor E4M3 weights (one scale for the fused gate/up shard, one for the down shard),
                     activations quantised on the fly per call (x per tensor; h per shard, so no max all-reduce).
    variant "w4a16": uint4 group-128 asymmetric weights with f16 scales, bf16 activations.
    """

    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, variant: str = "fp8",
                 tp: int = 1, rank: int = 0, group=None, reduce_dtype: torch.dtype = torch.bfloat16, overlap_chunks: int = 1,
                 already_sharded: bool = False):
        """w_gate, w_up: [inter x hidden]; w_down: [hidden x inter] (full weights, cut here as the reference's
        from_full_weight does), or this rank's shards when already_sharded is set."""
        from . import ops
        if variant not in VARIANTS:
            raise ValueError(f"variant {variant!r} not in {VARIANTS}")
        self.ops = ops
        self.variant, self.tp, self.rank, self.group = variant, tp, rank, group
        self.reduce_dtype = reduce_dtype
        self.overlap_chunks = max(1, int(overlap_chunks))
        self.hidden = w_gate.shape[1]
        if already_sharded:
            g, u, d = w_gate, w_up, w_down
            self.inter = w_gate.shape[0] * tp
        else:
            self.inter = w_gate.shape[0]
            g, u, d = shard_mlp_weights(w_gate, w_up, w_down, tp, rank)
        self.inter_local = g.shape[0]
        dev = torch.device("cuda", torch.cuda.current_device())
        w_gu = interleave_gate_up(g, u).to(dev)
        d = d.to(dev)
        if variant == "fp8":
            self.w_gu_q, st = ops.fp8_quant_dynamic(w_gu)
            self.s_gu = st[1:].clone()
            self.w_down_q, st = ops.fp8_quant_dynamic(d)
            self.s_down = st[1:].clone()
        else:
            self.gu_codes, self.gu_scales, self.gu_zeros = ops.int4g_quant_pack(w_gu.float(), 128)
            self.d_codes, self.d_scales, self.d_zeros = ops.int4g_quant_pack(d.float(), 128)
            self._ws = {}
        self._comm_stream = torch.cuda.Stream() if self.overlap_chunks > 1 else None
        self._symm = None           # (buffer, handle) of the NVLS all-reduce path, created on first use
        import os
        self.keep_h = False         # tests set this: forward_partial then leaves its h = silu(gate) * up in self.last_h
        self.last_h = None
        self.use_multimem = tp > 1 and reduce_dtype == torch.bfloat16 and os.environ.get("OXQ_TP_NO_MULTIMEM", "0") != "1"
        self.split_reduce = os.environ.get("OXQ_TP_SPLIT_REDUCE", "1") != "0"
        self.split_blocks = max(2, int(os.environ.get("OXQ_TP_SPLIT_BLOCKS", "2")))    # column blocks of the down projection
        # OXQ_TP_FUSED_REDUCE=1: the down projection and the all-reduce as one kernel (oxq_gemm_fp8_all_reduce)
        self.fused_reduce = self.use_multimem and os.environ.get("OXQ_TP_FUSED_REDUCE", "0") == "1"
        self._flags = None
        self._fused_calls = 0
        # The in-switch reduce runs between cross-rank barrier kernels, or (OXQ_TP_SYNC_REDUCE=1) synchronises the ranks itself
        # through flag words in the switch.  Measured per step at M = 2048: 2 GPUs 0.591 / 0.623 ms, 8 GPUs 0.257 / 0.272 ms:
        # the barrier form is the default.
        self.sync_reduce = self.use_multimem and os.environ.get("OXQ_TP_SYNC_REDUCE", "0") == "1"
        self._sflags = None
        self._sync_calls = 0

    # -- NVLS path: symmetric output buffer mapped through the NVSwitch multicast object ----------
    def _symm_buffer(self, m: int):
        """Symmetric [m_cap x hidden] bf16 buffer + its rendezvous handle, or None if multicast is unavailable."""
        if not self.use_multimem:
            return None
        if self._symm is not None and self._symm[0].shape[0] >= m:
            return self._symm
        try:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            cap = max(m, 2048)
            buf = symm_mem.empty((cap, self.hidden), dtype=torch.bfloat16, device=torch.device("cuda", torch.cuda.current_device()))
            hdl = symm_mem.rendezvous(buf, self.group if self.group is not None else dist.group.WORLD)
            if not hdl.multicast_ptr:                  # 0 when the fabric offers no multicast mapping
                raise RuntimeError("no multicast support")
            self._symm = (buf, hdl)
        except Exception:
            self.use_multimem = False       # NCCL all-reduce instead
            self._symm = None
        return self._symm

    def _sync_flags(self):
        """Four symmetric flag words of the self-synchronising reduce kernel (zeroed once, then only touched by the kernels)."""
        if self._sflags is None:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            words = symm_mem.empty((4,), dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
            words.zero_()
            fh = symm_mem.rendezvous(words, self.group if self.group is not None else dist.group.WORLD)
            if not fh.multicast_ptr:
                raise RuntimeError("no multicast support")
            torch.cuda.synchronize()
            fh.barrier(channel=0)                      # every replica is zero before anyone's first signal can land
            torch.cuda.synchronize()
            self._sflags = (words, fh)
        return self._sflags

    def _reduce_block(self, hdl, ptr_offset_bytes: int, m: int, cols: int, first: bool, last: bool, channel: int, ld: int | None = None):
        """In-switch all-reduce of a column block of the symmetric output: either the kernel that synchronises the ranks
        itself, or the plain kernel between cross-rank barriers."""
        ops = self.ops
        ld = self.hidden if ld is None else ld
        if self.sync_reduce:
            try:
                words, fh = self._sync_flags()
            except Exception:
                self.sync_reduce = False
            else:
                self._sync_calls += 1
                ops.multimem_all_reduce_bf16_2d_sync(hdl.multicast_ptr + ptr_offset_bytes, m, cols, ld, self.rank, self.tp, words, fh.multicast_ptr)
                return
        hdl.barrier(channel=channel)
        ops.multimem_all_reduce_bf16_2d(hdl.multicast_ptr + ptr_offset_bytes, m, cols, ld, self.rank, self.tp)
        if last:
            hdl.barrier(channel=channel + 1)

    def _fused_flags(self):
        """Symmetric flag words of the fused GEMM + all-reduce kernel (zeroed once; every call leaves them zero)."""
        if self._flags is None:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            words = symm_mem.empty((2 * 4096 + 1,), dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()))
            words.zero_()
            fh = symm_mem.rendezvous(words, self.group if self.group is not None else dist.group.WORLD)
            if not fh.multicast_ptr:
                raise RuntimeError("no multicast support")
            torch.cuda.synchronize()
            fh.barrier(channel=0)                      # every replica is zero before anyone's first arrival can land
            torch.cuda.synchronize()
            self._flags = (words, fh)
        return self._flags

    def _forward_fused(self, x: torch.Tensor):
        """FP8 variant: the down projection and the all-reduce are one kernel per rank (tiles are summed in the NVSwitch
        while later tiles are still being multiplied); no barrier kernels, no side stream."""
        m = x.shape[0]
        sym = self._symm_buffer(m)
        tiles = ((m + 255) // 256) * ((self.hidden + 255) // 256)
        if sym is None or self.variant != "fp8" or self.hidden % 8 != 0 or tiles + 1 > 4096 or m <= 128:
            return None
        try:
            words, fh = self._fused_flags()
        except Exception:
            self.fused_reduce = False
            return None
        buf, hdl = sym
        y = buf[:m]
        ops = self.ops
        xq, sx = ops.fp8_quant_dynamic(x)
        h = ops.gemm_fp8_swiglu(xq, self.w_gu_q, sx[1:], self.s_gu)
        if self.keep_h:
            self.last_h = h
        hq, sh = ops.fp8_quant_dynamic(h)
        ops.gemm_fp8_all_reduce(hq, self.w_down_q, sh[1:], self.s_down, y, hdl.multicast_ptr, words, fh.multicast_ptr, self.rank, self.tp)
        self._fused_calls += 1
        return y

    def _forward_multimem(self, x: torch.Tensor):
        """down-projection partial straight into the symmetric buffer, barrier, in-switch reduce + broadcast, barrier."""
        m = x.shape[0]
        sym = self._symm_buffer(m)
        if sym is None or (m * self.hidden) % (8 * self.tp) != 0:
            return None
        buf, hdl = sym
        y = buf[:m]
        self.forward_partial(x, out=y)
        if self.sync_reduce:
            if m % self.tp == 0:
                self._reduce_block(hdl, 0, m, self.hidden, True, True, 0)      # falls back to barriers by itself
                return y
            sub = self.hidden // self.tp
            if self.hidden % self.tp == 0 and sub % 8 == 0:
                # fewer rows than ranks (a decode step): the contiguous [m x hidden] block seen as [m * tp x hidden / tp]
                self._reduce_block(hdl, 0, m * self.tp, sub, True, True, 0, ld=sub)
                return y
        hdl.barrier(channel=0)
        self.ops.multimem_all_reduce_bf16(hdl.multicast_ptr, m * self.hidden, self.rank, self.tp)
        hdl.barrier(channel=1)
        return y

    def _forward_multimem_split(self, x: torch.Tensor):
        """FP8 variant: the down-projection runs as `split_blocks` column blocks and the in-switch reduce of block i (on a
        side stream) overlaps the GEMM of block i + 1.  One cross-rank barrier before each reduce (block i is written on
        every rank; it also tells that reduce i - 1 has finished everywhere) and one after the last."""
        m = x.shape[0]
        sym = self._symm_buffer(m)
        nb = self.split_blocks
        blk = self.hidden // nb
        if sym is None or self.variant != "fp8" or m % self.tp != 0 or self.hidden % nb != 0 or blk % 256 != 0:
            return None
        buf, hdl = sym
        y = buf[:m]
        ops = self.ops
        if self._comm_stream is None:
            self._comm_stream = torch.cuda.Stream()
        main, comm = torch.cuda.current_stream(), self._comm_stream
        xq, sx = ops.fp8_quant_dynamic(x)
        h = ops.gemm_fp8_swiglu(xq, self.w_gu_q, sx[1:], self.s_gu)
        if self.keep_h:
            self.last_h = h
        hq, sh = ops.fp8_quant_dynamic(h)
        for i in range(nb):
            lo = i * blk
            ops.gemm_fp8(hq, self.w_down_q[lo:lo + blk], sh[1:], self.s_down, out=y[:, lo:lo + blk])
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ev)
                self._reduce_block(hdl, lo * 2, m, blk, i == 0, i == nb - 1, i)
        main.wait_stream(comm)
        return y

    # -- local (per-rank) partial: [M x hidden] --------------------------------------------------
    def forward_partial(self, x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        ops = self.ops
        if self.variant == "fp8":
            xq, sx = ops.fp8_quant_dynamic(x)
            h = ops.gemm_fp8_swiglu(xq, self.w_gu_q, sx[1:], self.s_gu)
            if self.keep_h:
                self.last_h = h
            hq, sh = ops.fp8_quant_dynamic(h)
            return ops.gemm_fp8(hq, self.w_down_q, sh[1:], self.s_down, out=out)
        m = x.shape[0]
        ws1 = self._workspace(m, 2 * self.inter_local, self.hidden)
        gu = ops.gemm_w4a16(x, self.gu_codes, self.gu_scales, self.gu_zeros, 128, workspace=ws1)
        h = ops.swiglu_interleaved(gu)
        ws2 = self._workspace(m, self.hidden, self.inter_local)
        return ops.gemm_w4a16(h, self.d_codes, self.d_scales, self.d_zeros, 128, workspace=ws2, out=out)

    def _workspace(self, m, n, k):
        key = (m > 32, m if m <= 32 else 0, n, k)
        if key not in self._ws:
            self._ws[key] = self.ops.gemm_w4a16_workspace(m, n, k, "cuda")
        return self._ws[key]

    # -- full layer: partial + all-reduce ----------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: bf16 [M x hidden], replicated on every rank.  Returns the reduced bf16 [M x hidden] on every rank: a
        tensor of its own in eager use; under CUDA-graph capture, on the in-switch paths, a view of the layer's symmetric
        buffer that the next replay overwrites."""
        import torch.distributed as dist
        if self.tp == 1:
            return self.forward_partial(x)
        m = x.shape[0]
        chunks = min(self.overlap_chunks, max(1, m // 256))
        if chunks <= 1:
            if self.use_multimem:
                y = self._forward_fused(x) if self.fused_reduce else None
                if y is None:
                    y = self._forward_multimem_split(x) if (self.split_reduce and m >= 512) else None
                if y is None:
                    y = self._forward_multimem(x)
                if y is not None:
                    return self._detach_from_symm(y)
            y = self.forward_partial(x)
            return self._all_reduce(y)
        # M-chunk pipelining: the all-reduce of chunk i runs on a side stream while chunk i+1 computes
        bounds = [(i * m) // chunks for i in range(chunks + 1)]
        main = torch.cuda.current_stream()
        sym = self._symm_buffer(m) if self.use_multimem else None
        if sym is not None and all(((bounds[i + 1] - bounds[i]) * self.hidden) % (8 * self.tp) == 0 for i in range(chunks)):
            buf, hdl = sym
            y = buf[:m]
            self._comm_stream.wait_stream(main)
            for i in range(chunks):
                lo, hi = bounds[i], bounds[i + 1]
                self.forward_partial(x[lo:hi], out=y[lo:hi])
                ev = torch.cuda.Event()
                ev.record(main)
                with torch.cuda.stream(self._comm_stream):
                    self._comm_stream.wait_event(ev)
                    hdl.barrier(channel=2 * i)
                    self.ops.multimem_all_reduce_bf16(hdl.multicast_ptr + lo * self.hidden * 2, (hi - lo) * self.hidden, self.rank, self.tp)
                    hdl.barrier(channel=2 * i + 1)
            main.wait_stream(self._comm_stream)
            return self._detach_from_symm(y)
        y = torch.empty((m, self.hidden), dtype=torch.bfloat16, device=x.device)
        for i in range(chunks):
            lo, hi = bounds[i], bounds[i + 1]
            self.forward_partial(x[lo:hi], out=y[lo:hi])
            ev = torch.cuda.Event()
            ev.record(main)
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ev)
                dist.all_reduce(y[lo:hi], op=dist.ReduceOp.SUM, group=self.group)
        main.wait_stream(self._comm_stream)
        return y

    def _detach_from_symm(self, y: torch.Tensor) -> torch.Tensor:
        """The in-switch paths reduce in place in the layer's persistent symmetric buffer, which the next call
        overwrites.  Eager callers get a copy, so a result kept across two calls (a residual) stays what it was, as
        with the NCCL path; inside a CUDA-graph capture the view itself is returned (capture() hands it out as the
        graph's static output, valid until the next replay)."""
        return y if torch.cuda.is_current_stream_capturing() else y.clone()

    def _all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if self.reduce_dtype == torch.float32:
            z = y.float()
            dist.all_reduce(z, op=dist.ReduceOp.SUM, group=self.group)
            return z.to(torch.bfloat16)
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=self.group)
        return y

    # -- CUDA-graph replay of the whole layer ---------------------------------------------------------
    def capture(self, m: int):
        """Captures forward() for a fixed batch of m rows into a CUDA graph.  Returns (x_static, y_static, graph):
        fill x_static, call graph.replay(), read y_static.  A decode step is a dozen launches of a few microseconds
        each, so replaying them from a graph removes the host launch cost from the step."""
        dev = torch.device("cuda", torch.cuda.current_device())
        x_static = torch.zeros((m, self.hidden), dtype=torch.bfloat16, device=dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):                       # warm-up outside capture: workspaces, attributes, symmetric buffers
                self.forward(x_static)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            y_static = self.forward(x_static)
        return x_static, y_static, graph

    # -- bookkeeping for the benchmark -------------------------------------------------------------
    def flops(self, m: int) -> float:
        """Whole-layer flop count over all ranks: 2 * M * 3 * hidden * inter."""
        return 2.0 * m * 3 * self.hidden * self.inter

    def weight_bytes_local(self) -> int:
        if self.variant == "fp8":
            return self.w_gu_q.numel() + self.w_down_q.numel()
        n = self.gu_codes.numel() * 4 + self.d_codes.numel() * 4
        return n + (self.gu_scales.numel() + self.d_scales.numel()) * 2 + (self.gu_zeros.numel() + self.d_zeros.numel()) * 4

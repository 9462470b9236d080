#!/usr/bin/env python
"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras] [--peaks FILE]

N = 1.  Headline workload: FP8 E4M3 GEMM M = N = K = 8192, bf16 operands N(0,1) quantised per tensor
(scale = absmax/448), f32 accumulate, bf16 output = acc * sA * sB.

  value     TFLOP/s of the GEMM kernel with the E4M3 operands already resident in HBM: the median over
            `repeats` timed regions of exactly K launches each (ms_per_step, spread and every region's
            time are in the line).
  e2e       the same metric through the host-buffer path: pinned bf16 host operands -> H2D ->
            absmax + quantize of both operands -> GEMM -> D2H of the bf16 result, every step.
  roofline  the GEMM kernel against the tensor-core peak: 2 x the measured bf16 burst figure (the timed
            regions are milliseconds of isolated launches, not a sustained loop; FP8 issues at twice the
            bf16 rate and no FP8 figure is measured).  `roofline.configs` is the per-kernel table of
            the whole path: name -> [ms per launch, fraction of its roofline] (HBM copy bandwidth for
            the memory-bound kernels, 2x / 4x the bf16 burst figure for 8-bit / 4-bit tensor kernels).
  extras    the same kernels in long form (bytes, GB/s, launches per call).
  cpu_baseline / --impl reference
            the CPU oracle (a C restatement of the reference's scalar loops; the reference itself is
            a Rust workspace that cannot be built here) on a bounded sample of the same workload.

N > 1 (one process per GPU under torchrun).  The workload that shards: the tensor-parallel FP8 SwiGLU
MLP of Llama-3-70B shape at M = 2048, gate/up column-sharded, down row-sharded, partial sums combined
in the NVSwitch (or by one NCCL all-reduce); strong scaling, time = max over ranks.  The line carries
`tp1_ms` (the same layer on one GPU, measured on rank 0 in the same run) and `speedup_vs_tp1`, a
`parity` block (the layer's output on seeded inputs against the same partial sums combined by an NCCL
all-reduce and against the CPU oracle on a row sample; the run exits non-zero above 1e-2), and the
largest of the step's phases.  `--impl reference` at N > 1 times the reference's CPU form of the same
layer (f32 column- and row-parallel loops, ranks one after the other) on a row sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M = N = K = 8192
FLOP = 2.0 * M * N * K
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline GEMM kernel, from an ncu capture of
# `bench.py --case gemm_fp8` (algorithmic operand + output bytes: 268435456)
NCU_DRAM_BYTES_PER_LAUNCH = 344_340_736
L2_BYTES = 126 * 1024 * 1024
PEAKS_FILE = os.path.join(ROOT, "MEASURED_PEAKS.json")
MAX_REL = 1e-2


def load_peaks(path=None):
    """Roofline denominators measured on this pool (a copy bandwidth and a bf16 GEMM rate, burst and sustained)."""
    p = path or PEAKS_FILE
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            time.sleep(0.25)                              # the first sample takes a while to appear
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, pw, reasons = [], [], [], set()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            try:
                pw.append(float(f[3]))
            except ValueError:
                pw.append(0.0)
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # the timed regions alternate with idle gaps: the samples under load are those near the highest power draw seen
        top_w = max(pw)
        load = [c for c, w in zip(sm, pw) if w >= 0.6 * top_w] or sm
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm),
                "samples_under_load": len(load), "power_w_max": top_w}


HIDDEN, INTER = 8192, 28672          # Llama-3-70B MLP shape
TP_M = 2048


def tp_workload(variant="fp8"):
    return f"tp_swiglu_mlp_{variant}_hidden{HIDDEN}_inter{INTER}_m{TP_M}"


def workload_config(world: int, variant="fp8"):
    """The `config` object of the JSON line: what is computed, identical for this library's arm and the reference arm
    (how each arm runs it -- buffers, sampling, overlap -- goes into `details`)."""
    if world > 1:
        return {"workload": tp_workload(variant), "parallelism": f"tp{world}", "hidden": HIDDEN, "intermediate": INTER, "m": TP_M,
                "out": "bf16"}
    return {"workload": "fp8_e4m3_gemm_8192x8192x8192", "m": M, "n": N, "k": K, "accumulate": "f32", "out": "bf16"}


# ------------------------------------------------------------------------------------------------ CPU arm

def cpu_gemm_sample(sample_rows: int, threads: int):
    """Times the oracle's FP8 path on `sample_rows` rows of X against the full 8192 x 8192 weight:
    quantised codes -> dequantise -> f32 GEMM in the reference's accumulation order."""
    from oracle import oracle as orc
    rng = np.random.Generator(np.random.Philox(0))
    xq = rng.integers(0, 0x7E, size=(sample_rows, K), dtype=np.uint8)
    wq = rng.integers(0, 0x7E, size=(N, K), dtype=np.uint8)
    t0 = time.perf_counter()
    x = orc.spec_fp8_dequant(xq, 1.0)
    w = orc.spec_fp8_dequant(wq, 1.0)
    orc.ref_linear_f32(x, w, threads=threads)
    dt = time.perf_counter() - t0
    return 2.0 * sample_rows * N * K / dt / 1e12, dt


class CpuTpMlp:
    """The reference's CPU form of the tensor-parallel layer (ColumnLinear / RowLinear / SwiGluFfn: f32 weights, f32
    left-to-right dot products, ranks simulated one after the other, partial sums added in rank order) on `rows` rows
    of X.  The weights are cut into the ranks' shards once, outside the timed region, as from_full_weight does."""

    def __init__(self, tp: int, rows: int):
        blk = np.random.Generator(np.random.Philox(3)).standard_normal(1 << 20, dtype=np.float32) * np.float32(0.02)
        sh = INTER // tp
        reps = (sh * HIDDEN + blk.size - 1) // blk.size
        self.tp, self.rows = tp, rows
        self.shards = []
        for r in range(tp):
            flat = np.tile(np.roll(blk, 17 * r), reps)[: sh * HIDDEN]
            self.shards.append((flat.reshape(sh, HIDDEN), np.roll(flat, 5).reshape(sh, HIDDEN), np.roll(flat, 11).reshape(HIDDEN, sh)))
        self.x = np.random.Generator(np.random.Philox(1)).standard_normal((rows, HIDDEN), dtype=np.float32)
        self.flop = 2.0 * rows * 3 * HIDDEN * INTER

    def step(self, threads: int):
        from oracle import oracle as orc
        t0 = time.perf_counter()
        parts = []
        for wg, wu, wd in self.shards:
            g = orc.ref_linear_f32(self.x, wg, threads=threads)
            u = orc.ref_linear_f32(self.x, wu, threads=threads)
            parts.append(orc.ref_linear_f32(orc.ref_silu_mul(g, u), wd, threads=threads))
        orc.ref_all_reduce_sum(parts)
        return time.perf_counter() - t0


def run_reference(args):
    from oracle import oracle as orc
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    threads = orc.host_cores()                            # explicit: launchers export OMP_NUM_THREADS=1
    if world > 1:
        rows = 8
        cpu = CpuTpMlp(world, rows)
        for _ in range(min(args.warmup, 2)):
            cpu.step(threads)
        times = [cpu.step(threads) for _ in range(args.steps)]
        val = cpu.flop / statistics.median(times) / 1e12
        sample = (f"{rows} of {TP_M} rows of X through the whole layer per step (f32 weights, reference summation order, "
                  f"{world} ranks simulated one after the other, rank-order sum)")
        scaling = "strong"
    else:
        rows = 64
        for _ in range(args.warmup):
            cpu_gemm_sample(8, threads)
        vals, times = [], []
        for _ in range(args.steps):
            v, dt = cpu_gemm_sample(rows, threads)
            vals.append(v)
            times.append(dt)
        val = float(np.mean(vals))
        sample = f"{rows} of {M} rows of X against the full {N}x{K} weight per step (dequantise + f32 GEMM, reference summation order)"
        scaling = "weak"
    line = {
        "impl": "reference", "metric": "quant_gemm_tflops_prefill", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(np.mean(times)) * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(world),
        "details": {"sample": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ GPU arm

def time_region(torch, fn, steps, dist_on):
    """Times `steps` calls of fn() with CUDA events on the current stream, barrier + sync on both sides."""
    if dist_on:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        torch.distributed.barrier()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def timed_median(torch, fn, steps, dist_on, repeats=7, gap_s=0.05, warm=5):
    """`repeats` timed regions of exactly `steps` calls each; before every region an idle gap and then `warm` untimed
    calls, so that each region is what a single run of this script times: warm-up launches followed at once by the timed
    ones, on a GPU that is neither idling at low clocks nor already at its power cap (back to back, 300 ms of FP8 GEMMs
    settle some 25 % lower, at the sustained clock -- `sustained_rate` measures that).  Returns (median ms per step, stats)."""
    regions = []
    for _ in range(repeats):
        time.sleep(gap_s)
        for _ in range(warm):
            fn()
        regions.append(time_region(torch, fn, steps, dist_on))
    per = sorted(r / steps for r in regions)
    med = statistics.median(per)
    return med, {"repeats": len(per), "median": med, "min": per[0], "max": per[-1], "spread": (per[-1] - per[0]) / med if med > 0 else 0.0,
                 "protocol": f"{len(per)} regions of {steps} launches, each after {int(gap_s * 1e3)} ms idle and {warm} untimed launches"}


def sustained_rate(torch, fn, steps, total_ms=400.0):
    """ms per call over back-to-back regions adding up to about `total_ms` (the GPU at its power cap)."""
    first = time_region(torch, fn, steps, False)
    reps = int(min(200, max(3, total_ms / max(first, 1e-3))))
    regions = [time_region(torch, fn, steps, False) for _ in range(reps)]
    return statistics.median(regions[len(regions) // 2:]) / steps


def ring_time(torch, make_call, ring):
    """Average ms per call over a ring of distinct buffer sets (total > L2).  The calls are captured
    once into a CUDA graph and the graph is replayed, so host launch overhead (several microseconds
    per call through ctypes) does not sit between kernels that themselves last a few microseconds.
    Five timed replays; the median is returned."""
    for r in ring:                                       # warm-up: every variant launched (and its attributes set) before capture
        make_call(r)
    torch.cuda.synchronize()
    reps_in_graph = max(1, 24 // len(ring))
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(reps_in_graph):
            for r in ring:
                make_call(r)
    graph.replay()
    torch.cuda.synchronize()
    per = []
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        per.append(e0.elapsed_time(e1) / (3 * reps_in_graph * len(ring)))
    return statistics.median(per)


class Table:
    """Per-kernel results: the long form (`extras`) and the compact table that goes into `roofline.configs`."""

    def __init__(self, peaks):
        self.peaks = peaks
        self.long = {}
        self.short = {}

    def hbm(self, name, short, nbytes, ms, launches=1):
        gbs = nbytes / (ms * 1e-3) / 1e9
        frac = gbs / self.peaks["hbm_gbs"]
        self.long[name] = {"ms": round(ms, 5), "GB/s": round(gbs, 1), "frac_of_hbm": round(frac, 3), "bytes": int(nbytes),
                           "launches_per_call": launches}
        self.short[short] = [float(f"{ms:.3g}"), round(frac, 2)]

    def tensor(self, name, short, flop, ms, rate_x_bf16):
        tf = flop / (ms * 1e-3) / 1e12
        peak = rate_x_bf16 * self.peaks["bf16_tflops"]
        self.long[name] = {"ms": round(ms, 5), "TFLOP/s": round(tf, 1), "frac_of_tensor_peak": round(tf / peak, 3),
                           "peak": f"{rate_x_bf16} x bf16 burst"}
        self.short[short] = [float(f"{ms:.3g}"), round(tf / peak, 2)]


def extras(torch, ops, tab):
    """Memory-bound kernels of the path: GB/s of algorithmic bytes, fraction of the measured copy bandwidth."""
    g = torch.Generator(device="cuda").manual_seed(0)
    # config 1: INT8 per-row quantize / dequantize of 4096x4096 f32 (ring of 4 -> 256 MiB of inputs)
    ring = [torch.randn((4096, 4096), generator=g, device="cuda") * 0.02 for _ in range(4)]
    q8 = [ops.int8_quant_rows(r) for r in ring]
    tab.hbm("int8_quant_rows_4096x4096", "q_i8rows", 67108864 + 16777216 + 16384, ring_time(torch, lambda r: ops.int8_quant_rows(r), ring))
    tab.hbm("int8_dequant_rows_4096x4096", "dq_i8rows", 16777216 + 16384 + 67108864, ring_time(torch, lambda r: ops.int8_dequant_rows(*r), q8))
    x8 = torch.randn((8, 4096), generator=g, device="cuda")
    tab.hbm("gemm_w8a32_m8_4096x4096", "w8a32_m8_4096x4096", 16777216 + 16384 + 131072 + 131072, ring_time(torch, lambda r: ops.gemm_w8a32(x8, *r), q8))
    del ring, q8
    # config 2: bf16 -> E4M3 of 8192x8192 (ring of 3 -> 384 MiB)
    ring = [torch.randn((8192, 8192), generator=g, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    outq = torch.empty((8192, 8192), dtype=torch.uint8, device="cuda")
    stats = torch.empty(2, device="cuda")
    am = torch.empty(1, device="cuda")
    tab.hbm("absmax_bf16_8192x8192", "absmax", 134217728, ring_time(torch, lambda r: ops.absmax(r, out=am), ring))
    # what a plain streaming kernel reaches at the byte counts of the decode weights (the launch costs microseconds
    # whatever it reads): the practical ceiling next to which the decode GEMM lines below should be read
    for nbytes in (8388608, 29360128):
        per = 134217728 // nbytes                                      # disjoint slices of the three big tensors: > 350 MB in all
        small = [ring[i % 3].view(-1)[(i // 3) * (nbytes // 2):(i // 3 + 1) * (nbytes // 2)] for i in range(3 * per)]
        tab.hbm(f"stream_floor_absmax_{nbytes // 1048576}MiB", f"floor_{nbytes // 1048576}MiB", nbytes, ring_time(torch, lambda r: ops.absmax(r, out=am), small))
    one = torch.ones(1, device="cuda")
    tab.hbm("fp8_quant_bf16_8192x8192", "q_fp8", 201326592, ring_time(torch, lambda r: ops.fp8_quant(r, one, out=outq), ring))
    tab.hbm("fp8_quant_dynamic_bf16_8192x8192", "q_fp8_dyn", 335544320, ring_time(torch, lambda r: ops.fp8_quant_dynamic(r, out=outq, stats=stats), ring))
    outi = outq.view(torch.int8)
    wnorm = torch.ones(8192, device="cuda")
    tab.hbm("rmsnorm_int8_quant_rows_bf16_8192x8192", "rms_i8", 201326592 + 8192 * 8, ring_time(torch, lambda r: ops.rmsnorm_int8_quant_rows(r, wnorm), ring))
    tab.hbm("rmsnorm_fp8_quant_rows_bf16_8192x8192", "rms_fp8", 201326592, ring_time(torch, lambda r: ops.rmsnorm_fp8_quant_rows(r, wnorm, one), ring))
    tab.hbm("silu_gate_fp8_quant_bf16_8192x8192", "silu_fp8", 134217728 * 2 + 67108864,
            ring_time(torch, lambda r: ops.silu_gate_fp8_quant(r[0], r[1], one), [(ring[i], ring[(i + 1) % 3]) for i in range(3)]))
    tab.hbm("int8_quant_tensor_bf16_8192x8192(absmax+encode)", "q_i8tensor", 335544320, ring_time(torch, lambda r: ops.quantize_to_int8(r, out=outi, scale=am), ring), 2)
    # config 4 quantizers on the 4096x4096 activation shape (ring of 8 -> 256 MiB)
    ring4 = [r[:4096, :4096].contiguous() for r in ring] + [r[4096:, 4096:].contiguous() for r in ring] + [ring[0][:4096, 4096:].contiguous(), ring[1][4096:, :4096].contiguous()]
    tab.hbm("mxfp8_quant_bf16_4096x4096", "q_mxfp8_4096", 33554432 + 16777216 + 2 * 524288, ring_time(torch, lambda r: ops.mxfp8_quant(r), ring4))
    tab.hbm("nvfp4_quant_bf16_4096x4096(absmax+encode)", "q_nvfp4_4096", 2 * 33554432 + 8388608 + 2 * 1048576, ring_time(torch, lambda r: ops.nvfp4_quant(r), ring4), 2)
    del ring, ring4, outq
    # the same block-scaled quantizers on the weight shape of config 4 (14336 x 4096 bf16, ring of 4 -> 470 MB)
    ringw4 = [torch.randn((14336, 4096), generator=g, device="cuda", dtype=torch.bfloat16) for _ in range(4)]
    nel = 14336 * 4096
    tab.hbm("mxfp8_quant_bf16_14336x4096", "q_mxfp8_14336", nel * 2 + nel + 2 * nel // 32, ring_time(torch, lambda r: ops.mxfp8_quant(r), ringw4))
    tab.hbm("nvfp4_quant_bf16_14336x4096(absmax+encode)", "q_nvfp4_14336", 2 * nel * 2 + nel // 2 + 2 * nel // 16, ring_time(torch, lambda r: ops.nvfp4_quant(r), ringw4), 2)
    del ringw4
    # config 3: W4A16 decode GEMMs; weights cycled through a ring > 4x L2
    for (n, k) in ((6144, 4096), (4096, 4096), (14336, 4096), (4096, 14336)):
        wbytes = n * k // 2 + n * k // 128 * 2 + n * k // 128 // 2
        copies = max(4, int(4 * L2_BYTES // wbytes) + 1)
        w = torch.randn((n, k), generator=g, device="cuda") * 0.02
        c, s, z = ops.int4g_quant_pack(w, 128)
        ring = [(c.clone(), s.clone(), z.clone()) for _ in range(copies)]
        del w
        for m in (1, 8, 16, 32):
            x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
            ws = ops.gemm_w4a16_workspace(m, n, k, "cuda")
            y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            ms = ring_time(torch, lambda r: ops.gemm_w4a16(x, r[0], r[1], r[2], 128, workspace=ws, out=y), ring)
            tab.hbm(f"gemm_w4a16_m{m}_{n}x{k}", f"w4_m{m}_{n}x{k}", wbytes + m * k * 2 + m * n * 2, ms)
            if m == 16:
                del tab.short[f"w4_m{m}_{n}x{k}"]                      # the compact table keeps M = 1, 8, 32
        del ring
    # config 4 at decode batch sizes: the block-scaled GEMMs as weight streams (weights cycled through a ring > 4x L2)
    for (n, k) in ((14336, 4096), (4096, 14336)):
        w = torch.randn((n, k), generator=g, device="cuda").to(torch.bfloat16)
        b8, b4 = n * k + n * k // 32, n * k // 2 + n * k // 16
        cb, _, fb = ops.mxfp8_quant(w)
        pb, _, fb4, stb = ops.nvfp4_quant(w)
        del w
        ring8 = [(cb.clone(), fb.clone()) for _ in range(int(4 * L2_BYTES // b8) + 1)]
        ring4 = [(pb.clone(), fb4.clone()) for _ in range(int(4 * L2_BYTES // b4) + 1)]
        for m in (1, 8, 32):
            x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
            y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
            ca, _, fa = ops.mxfp8_quant(x)
            pa, _, fa4, sta = ops.nvfp4_quant(x)
            ms = ring_time(torch, lambda r: ops.gemm_mxfp8(ca, fa, r[0], r[1], out=y), ring8)
            tab.hbm(f"gemm_mxfp8_m{m}_{n}x{k}", f"mxfp8_m{m}_{n}x{k}", b8 + m * k * 33 // 32 + m * n * 2, ms)
            ms = ring_time(torch, lambda r: ops.gemm_nvfp4(pa, fa4, sta, r[0], r[1], stb, out=y), ring4)
            tab.hbm(f"gemm_nvfp4_m{m}_{n}x{k}", f"nvfp4_m{m}_{n}x{k}", b4 + m * k * 9 // 16 + m * n * 2, ms)
        del ring8, ring4
    # the offline W4 quantize + pack kernel on the largest weight
    ringw = [torch.randn((14336, 4096), generator=g, device="cuda") * 0.02 for _ in range(3)]
    tab.hbm("int4g_quant_pack_f32_14336x4096", "q_int4g", 14336 * 4096 * 4 + 14336 * 4096 // 2 + 458752 * 2 + 458752 // 2,
            ring_time(torch, lambda r: ops.int4g_quant_pack(r, 128), ringw))
    tab.hbm("nf4_quant_f32_14336x4096_b64", "q_nf4", 14336 * 4096 * 4 + 14336 * 4096 // 2 + 14336 * 4096 // 64 * 4,
            ring_time(torch, lambda r: ops.nf4_quant(r, 64), ringw))
    packs = [ops.nf4_quant(ringw[i % 3].view(-1), 64) for i in range(6)]                      # 6 x 30 MB of packed weights
    for mrows in (1, 8):
        xn = torch.randn((mrows, 4096), generator=g, device="cuda").to(torch.bfloat16)
        tab.hbm(f"gemm_nf4_m{mrows}_14336x4096_b64", f"nf4_m{mrows}_14336x4096", 14336 * 4096 // 2 + 14336 * 4096 // 64 * 4 + mrows * (4096 + 14336) * 2,
                ring_time(torch, lambda r: ops.gemm_nf4(xn, r[0], r[1], 14336, 64), packs))
    del packs
    # decode GEMMs on a weight of the TP1 MLP size (57344 x 8192, 470 MB per copy; two copies in rotation)
    wbig = [torch.randn((57344, 8192), generator=g, device="cuda", dtype=torch.bfloat16) for _ in range(1)]
    fp8w = [ops.fp8_quant_dynamic(wbig[0]) for _ in range(2)]
    i8w = [ops.int8_quant_rows(wbig[0].float()) for _ in range(2)]
    del wbig
    for mrows in (1, 8, 32):
        xd = torch.randn((mrows, 8192), generator=g, device="cuda").to(torch.bfloat16)
        xq8, sx8 = ops.fp8_quant_dynamic(xd)
        tab.hbm(f"gemm_fp8_m{mrows}_57344x8192", f"fp8_m{mrows}_57344x8192", 57344 * 8192 + mrows * 8192 + 2 * mrows * 57344,
                ring_time(torch, lambda r: ops.gemm_fp8(xq8, r[0], sx8[1:], r[1][1:]), fp8w))
        xi8, sxi = ops.int8_quant_rows(xd.float())
        tab.hbm(f"gemm_w8a8_m{mrows}_57344x8192", f"w8a8_m{mrows}_57344x8192", 57344 * 8192 + mrows * 8192 + 2 * mrows * 57344 + 4 * 57344,
                ring_time(torch, lambda r: ops.gemm_w8a8(xi8, r[0], sxi, r[1]), i8w))
    del fp8w, i8w
    # offline weight preparation: one GPTQ layer (4096 x 4096, INT4 symmetric), Hessian from 8192 synthetic samples
    n = 4096
    xs = torch.randn((2 * n, n), generator=g, device="cuda")
    hess = (2.0 * xs.T @ xs / (2 * n)).float()
    hess = torch.maximum(hess, hess.T)
    del xs
    wq = ringw[0][:n].contiguous()
    gq = ops.GptqQuantizer(ops.GptqConfig(bits=4))
    gq.quantize_layer(wq, n, n, hess)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    gq.quantize_layer(wq, n, n, hess)
    e1.record()
    torch.cuda.synchronize()
    blocks = n // 32
    tab.long["gptq_quantize_layer_4096x4096_int4"] = {"ms": round(e0.elapsed_time(e1), 3), "launches_per_call": 2 + 3 * blocks - 2 + 2 * blocks - 1 + 2}


def prefill_extras(torch, ops, tab, steps):
    """The other prefill GEMMs of the path, timed like the headline (operands resident, `steps` launches per region):
    W8A8 8192^3 and the block-scaled GEMMs of the M = 4096, N = 14336, K = 4096 configuration."""
    g = torch.Generator(device="cuda").manual_seed(3)
    a = torch.randn((8192, 8192), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((8192, 8192), generator=g, device="cuda").to(torch.bfloat16)
    y = torch.empty((8192, 8192), dtype=torch.bfloat16, device="cuda")
    qa, sa = ops.int8_quant_rows(a.float())
    qb, sb = ops.int8_quant_rows(b.float())
    fn = lambda: ops.gemm_w8a8(qa, qb, sa, sb, out=y)  # noqa: E731
    for _ in range(3):
        fn()
    ms, _ = timed_median(torch, fn, steps, False, repeats=5)
    tab.tensor("gemm_w8a8_8192x8192x8192", "gemm_w8a8_8192", 2.0 * 8192 ** 3, ms, 2)
    del a, b, y, qa, qb
    m, n, k = 4096, 14336, 4096
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((n, k), generator=g, device="cuda").to(torch.bfloat16)
    y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ca, _, fa = ops.mxfp8_quant(a)
    cb, _, fb = ops.mxfp8_quant(b)
    fn = lambda: ops.gemm_mxfp8(ca, fa, cb, fb, out=y)  # noqa: E731
    for _ in range(3):
        fn()
    ms, _ = timed_median(torch, fn, steps, False, repeats=5)
    tab.tensor("gemm_mxfp8_4096x14336x4096", "gemm_mxfp8_cfg4", 2.0 * m * n * k, ms, 2)
    pa, _, fa4, sta = ops.nvfp4_quant(a)
    pb, _, fb4, stb = ops.nvfp4_quant(b)
    fn = lambda: ops.gemm_nvfp4(pa, fa4, sta, pb, fb4, stb, out=y)  # noqa: E731
    for _ in range(3):
        fn()
    ms, _ = timed_median(torch, fn, steps, False, repeats=5)
    tab.tensor("gemm_nvfp4_4096x14336x4096", "gemm_nvfp4_cfg4", 2.0 * m * n * k, ms, 4)


def make_tp_layer(torch, variant, world, rank, overlap_chunks=1):
    """Random-init weights N(0, 0.02) generated directly as this rank's shards (seeded per rank)."""
    from oxicuda_b200.dist_infer import TpSwiGluMlp
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    sh = INTER // world
    wg = (torch.randn((sh, HIDDEN), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    wu = (torch.randn((sh, HIDDEN), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    wd = (torch.randn((HIDDEN, sh), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    layer = TpSwiGluMlp(wg, wu, wd, variant, tp=world, rank=rank, overlap_chunks=overlap_chunks, already_sharded=True)
    del wg, wu, wd
    torch.cuda.empty_cache()
    return layer


def time_tp1_layer(torch, variant, m, iters):
    """The whole layer on one GPU (TP = 1), replayed from a CUDA graph: ms per step."""
    layer = make_tp_layer(torch, variant, 1, 0)
    x = torch.randn((m, HIDDEN), device="cuda").to(torch.bfloat16)
    for _ in range(3):
        layer.forward(x)
    fn = lambda: layer.forward(x)  # noqa: E731
    try:
        xs_, _, gr_ = layer.capture(m)
        xs_.copy_(x)
        fn = gr_.replay
    except Exception as exc:
        print(f"graph capture unavailable ({exc}); eager launches", file=sys.stderr)
        torch.cuda.synchronize()
    ms, st = timed_median(torch, fn, iters, False, repeats=5)
    out = (ms, st, layer.flops(m), layer.weight_bytes_local())
    del layer
    torch.cuda.empty_cache()
    return out


def mlp_extras(torch, tab):
    """The tensor-parallel MLP at TP = 1 (the denominator of the 1 -> 8 GPU scaling figure)."""
    for variant in ("fp8", "w4a16"):
        for m in (1, 64, 2048):
            ms, _, flops, wbytes = time_tp1_layer(torch, variant, m, 10 if m == 2048 else 30)
            name = f"tp_mlp_{variant}_m{m}_tp1"
            tf = flops / (ms * 1e-3) / 1e12
            gbs = wbytes / (ms * 1e-3) / 1e9
            tab.long[name] = {"ms": round(ms, 4), "TFLOP/s": round(tf, 2), "weight_GB/s": round(gbs, 1),
                              "frac_of_hbm": round(gbs / tab.peaks["hbm_gbs"], 3)}
            if m == 2048:
                peak = (2.0 if variant == "fp8" else 1.0) * tab.peaks["bf16_tflops"]
                tab.short[f"mlp_{variant}_m{m}_tp1"] = [round(ms, 4), round(tf / peak, 3)]
            else:
                tab.short[f"mlp_{variant}_m{m}_tp1"] = [round(ms, 4), round(gbs / tab.peaks["hbm_gbs"], 3)]


def tp_parity(torch, ops, layer, world, rank, rows=16):
    """Outside every timed region: the layer on seeded activations against (i) the same partial sums combined by an NCCL
    all-reduce and (ii) the CPU oracle on `rows` sampled rows -- each of the two GEMMs of every rank against the f64
    product of the dequantised codes it consumed, and the layer output against the sum of those per-rank products."""
    import torch.distributed as dist
    from oracle import oracle as orc
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn((TP_M, HIDDEN), generator=g, device="cuda").to(torch.bfloat16)
    y = layer.forward(x).float()
    # (i) the same partials through NCCL, summed in f32
    part = layer.forward_partial(x)
    z = part.float()
    dist.all_reduce(z, op=dist.ReduceOp.SUM)
    z = z.to(torch.bfloat16).float()
    vs_nccl = float((y - z).abs().max() / z.abs().max())
    # (ii) oracle on sampled rows, from the codes the GPU consumed
    sel = torch.randint(0, TP_M, (rows,), generator=torch.Generator().manual_seed(5)).cuda()
    xq, sx = ops.fp8_quant_dynamic(x)
    h = ops.gemm_fp8_swiglu(xq, layer.w_gu_q, sx[1:], layer.s_gu)
    hq, sh = ops.fp8_quant_dynamic(h)
    torch.cuda.synchronize()
    dx = orc.e4m3_to_f32(xq[sel].cpu().numpy()).astype(np.float64)
    sgu = float(sx[1]) * float(layer.s_gu[0])
    n2 = layer.w_gu_q.shape[0]
    h_ref = np.empty((rows, n2 // 2), np.float64)
    for b0 in range(0, n2, 2048):                             # blocks of 8 gate/up groups keep the f64 weight copy small
        dw = orc.e4m3_to_f32(layer.w_gu_q[b0:b0 + 2048].cpu().numpy()).astype(np.float64).reshape(-1, 2, 128, HIDDEN)
        gate = (dx @ dw[:, 0].reshape(-1, HIDDEN).T) * sgu
        up = (dx @ dw[:, 1].reshape(-1, HIDDEN).T) * sgu
        h_ref[:, b0 // 2:b0 // 2 + gate.shape[1]] = gate / (1.0 + np.exp(-gate)) * up
    h_gpu = h[sel].float().cpu().numpy()
    err_h = float(np.abs(h_gpu - h_ref).max() / np.abs(h_ref).max())
    dh = orc.e4m3_to_f32(hq[sel].cpu().numpy()).astype(np.float64)
    sd = float(sh[1]) * float(layer.s_down[0])
    p_ref = np.empty((rows, HIDDEN), np.float64)
    for b0 in range(0, HIDDEN, 1024):
        p_ref[:, b0:b0 + 1024] = (dh @ orc.e4m3_to_f32(layer.w_down_q[b0:b0 + 1024].cpu().numpy()).astype(np.float64).T) * sd
    err_p = float(np.abs(part[sel].float().cpu().numpy() - p_ref).max() / np.abs(p_ref).max())
    # every rank's partial rounds to bf16 before the reduce; sum the rounded oracle partials in f64
    p_bf = torch.from_numpy(p_ref.astype(np.float32)).to(torch.bfloat16).double().cuda()
    dist.all_reduce(p_bf, op=dist.ReduceOp.SUM)
    y_ref = p_bf.cpu().numpy()
    err_y = float(np.abs(y[sel].double().cpu().numpy() - y_ref).max() / np.abs(y_ref).max())
    worst = torch.tensor([vs_nccl, err_h, err_p, err_y], device="cuda", dtype=torch.float64)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    w = [float(v) for v in worst.cpu()]
    return {"max_rel_vs_nccl": w[0], "max_rel_vs_oracle": max(w[1:]), "gate_up_gemm": w[1], "down_gemm": w[2], "layer_output": w[3],
            "rows": rows, "tolerance": MAX_REL, "ok": max(w) <= MAX_REL}


def tp_phases(torch, ops, layer, x, steps=10):
    """Per-phase CUDA-event times of one rank's step, each phase timed alone (rank 0 reports): the four kernels of the
    rank's shard, and what is left of the whole step (exchange, cross-rank barriers, rank skew)."""
    def t(fn):
        for _ in range(2):
            fn()
        return time_region(torch, fn, steps, False) / steps
    xq, sx = ops.fp8_quant_dynamic(x)
    h = ops.gemm_fp8_swiglu(xq, layer.w_gu_q, sx[1:], layer.s_gu)
    hq, sh = ops.fp8_quant_dynamic(h)
    yb = torch.empty((x.shape[0], HIDDEN), dtype=torch.bfloat16, device="cuda")
    return {
        "quant_x": t(lambda: ops.fp8_quant_dynamic(x)),
        "gate_up_gemm": t(lambda: ops.gemm_fp8_swiglu(xq, layer.w_gu_q, sx[1:], layer.s_gu, out=h)),
        "quant_h": t(lambda: ops.fp8_quant_dynamic(h)),
        "down_gemm": t(lambda: ops.gemm_fp8(hq, layer.w_down_q, sh[1:], layer.s_down, out=yb)),
    }


def tp_attention_projections(torch, world, rank, peaks):
    """Configuration 3's attention projections under tensor parallelism, FP8: QKV (6144 x 4096) column-parallel with the
    all-gather of ColumnLinear::all_gather, O (4096 x 4096) row-parallel with the all-reduce of RowLinear::all_reduce.
    The first 4096 gathered columns stand in for the attention output.  Returns per-batch times and the largest deviation
    from the same two products computed in f32 from the bf16 weights (two FP8 GEMMs deep: a sanity figure, the parity
    tests of the two layers hold the 1e-2 bar per GEMM)."""
    from oxicuda_b200.dist_infer import ColumnLinear, RowLinear
    g = torch.Generator(device="cuda").manual_seed(11)
    wqkv = (torch.randn((6144, 4096), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    wo = (torch.randn((4096, 4096), generator=g, device="cuda") * 0.02).to(torch.bfloat16)
    col = ColumnLinear.from_full_weight(4096, 6144, wqkv, None, world, rank, "fp8")
    row = RowLinear.from_full_weight(4096, 4096, wo, None, world, rank, "fp8")
    out = {}
    for m in (2048, 32):
        x = torch.randn((m, 4096), generator=g, device="cuda").to(torch.bfloat16)

        def step():
            qkv = col.forward(x)                                  # local GEMM, all-gather -> [m x 6144]
            return row.forward(qkv[:, :4096])                     # slice, local GEMM, all-reduce -> [m x 4096]
        for _ in range(3):
            y = step()
        ms = time_region(torch, step, 20, True) / 20
        ref = ((x.float() @ wqkv.float().T)[:, :4096].to(torch.bfloat16).float() @ wo.float().T)
        err = float((y.float() - ref).abs().max() / ref.abs().max())
        flop = 2.0 * m * 4096 * (6144 + 4096)
        out[f"m{m}"] = {"ms": round(ms, 4), "TFLOP/s_all_ranks": round(flop / (ms * 1e-3) / 1e12, 1), "max_rel_vs_f32": round(err, 4)}
    return out


def run_tp_mlp(args, torch, world, rank, local_rank, peaks):
    """N > 1: the tensor-parallel FP8 SwiGLU MLP (hidden 8192, intermediate 28672, M = 2048), weights sharded over
    the ranks, partial sums combined in the NVSwitch (or by one NCCL all-reduce).  Strong scaling: the layer is fixed."""
    from oxicuda_b200 import ops
    import torch.distributed as dist
    m = TP_M
    variant = os.environ.get("OXQ_BENCH_TP_VARIANT", "fp8")
    chunks = int(os.environ.get("OXQ_BENCH_TP_CHUNKS", "1"))
    # the same layer on one GPU, measured on rank 0 in this very run: the denominator of the scaling figure
    tp1 = None
    if rank == 0:
        tp1_ms, tp1_stats, _, _ = time_tp1_layer(torch, variant, m, 10)
        tp1 = {"ms": tp1_ms, "stats": tp1_stats}
    dist.barrier()
    layer = make_tp_layer(torch, variant, world, rank, overlap_chunks=chunks)
    parity = tp_parity(torch, ops, layer, world, rank) if variant == "fp8" else None
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn((m, HIDDEN), generator=g, device="cuda").to(torch.bfloat16)
    for _ in range(max(args.warmup, 3)):
        layer.forward(x)
    # the step is replayed from a CUDA graph when capture works (OXQ_BENCH_TP_GRAPH=0 keeps eager launches)
    step_fn = lambda: layer.forward(x)  # noqa: E731
    graphed = False
    if os.environ.get("OXQ_BENCH_TP_GRAPH", "1") != "0":
        try:
            xs_, ys_, gr_ = layer.capture(m)
            xs_.copy_(x)
            step_fn = gr_.replay
            graphed = True
        except Exception as exc:                      # capture is an optimisation, not a requirement
            if rank == 0:
                print(f"graph capture unavailable: {exc}", file=sys.stderr)
            torch.cuda.synchronize()
    graphed_all = torch.tensor([1 if graphed else 0], device="cuda")
    dist.all_reduce(graphed_all, op=dist.ReduceOp.MIN)
    if int(graphed_all.item()) == 0:
        step_fn, graphed = (lambda: layer.forward(x)), False
    for _ in range(3):
        step_fn()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms, stats = timed_median(torch, step_fn, args.steps, True)
    clocks = sampler.stop() if rank == 0 else None
    value = layer.flops(m) / (ms * 1e-3) / 1e12
    phases = tp_phases(torch, ops, layer, x) if variant == "fp8" else None
    # decode-shaped points of the same layer (latency-bound; reported, not the headline)
    small = {}
    for mm in (1, 64):
        xs = torch.randn((mm, HIDDEN), generator=g, device="cuda").to(torch.bfloat16)
        for _ in range(3):
            layer.forward(xs)
        fn_small, mode = (lambda: layer.forward(xs)), "eager"
        if graphed:                                   # a decode step is a dozen launches of microseconds each: replay them from a graph
            try:
                xs_g, _, gr_small = layer.capture(mm)
                xs_g.copy_(xs)
                fn_small, mode = gr_small.replay, "cuda_graph"
            except Exception:
                torch.cuda.synchronize()
        ok_all = torch.tensor([1 if mode == "cuda_graph" else 0], device="cuda")
        dist.all_reduce(ok_all, op=dist.ReduceOp.MIN)
        if int(ok_all.item()) == 0:
            fn_small, mode = (lambda: layer.forward(xs)), "eager"
        for _ in range(3):
            fn_small()
        t = time_region(torch, fn_small, 20, True) / 20
        small[f"m{mm}"] = {"ms": round(t, 4), "weight_GB/s_all_ranks": round(world * layer.weight_bytes_local() / (t * 1e-3) / 1e9, 1), "launch": mode}
    attn = tp_attention_projections(torch, world, rank, peaks) if variant == "fp8" else None
    # End to end: pinned host activations in, reduced result out, every step, the host traffic sharded over the ranks:
    # every rank copies its 1/N of the rows of X in over its own PCIe link, the ranks all-gather X over NVLink, and every
    # rank copies its own 1/N of the rows of the result out.  Consecutive steps are double-buffered over three streams.
    per = m // world
    lo = rank * per
    x_h = x[lo:lo + per].cpu().pin_memory()
    y_h = [torch.empty((per, HIDDEN), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    x_d = [torch.empty_like(x) for _ in range(2)]
    y_d = [torch.empty((per, HIDDEN), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in, ev_free = [torch.cuda.Event() for _ in range(2)], [torch.cuda.Event() for _ in range(2)]
    ev_done, ev_out = [torch.cuda.Event() for _ in range(2)], [torch.cuda.Event() for _ in range(2)]
    main = torch.cuda.current_stream()
    step_no = [0]

    x_in = [torch.empty((per, HIDDEN), dtype=torch.bfloat16, device="cuda") for _ in range(2)]   # this rank's rows, as they arrive

    def e2e_step():
        i = step_no[0] & 1
        step_no[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[i])
            x_in[i].copy_(x_h, non_blocking=True)
            ev_in[i].record(s_in)
        main.wait_event(ev_in[i])
        main.wait_event(ev_out[i])
        if graphed:
            # the whole layer replayed from its CUDA graph: X is gathered straight into the graph's input buffer
            dist.all_gather_into_tensor(xs_, x_in[i])
            ev_free[i].record(main)
            gr_.replay()
            y = ys_
        else:
            dist.all_gather_into_tensor(x_d[i], x_in[i])
            ev_free[i].record(main)
            y = layer.forward(x_d[i])
        y_d[i].copy_(y[lo:lo + per])
        ev_done[i].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            y_h[i].copy_(y_d[i], non_blocking=True)
            ev_out[i].record(s_out)

    def e2e_region(steps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        s_in.wait_event(e0)
        for _ in range(steps):
            e2e_step()
        main.wait_stream(s_out)
        main.wait_stream(s_in)
        e1.record(main)
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    e2e_region(2)
    e2e_steps = max(4, min(args.steps, 10))
    e2e_ms = statistics.median([e2e_region(e2e_steps) / e2e_steps for _ in range(3)])
    if rank == 0:
        # per-rank GEMM time at the tensor peak vs the bytes every rank must move through NVLink for the all-reduce
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        t_compute = layer.flops(m) / world / (fp8_peak * 1e12)
        t_link = 2.0 * (world - 1) / world * m * HIDDEN * 2 / 770e9
        target = max(t_compute, t_link)
        # this library's kernels per step: absmax + quantize (x), gate/up GEMM, absmax + quantize (h), down GEMM, reduce;
        # with the split reduce the down GEMM and the reduce run twice (the cross-rank barriers are torch's kernels)
        split = world > 1 and variant == "fp8" and chunks <= 1 and bool(layer.use_multimem) and bool(getattr(layer, "split_reduce", False)) and m >= 512
        kernels_per_step = 9 if split else (min(chunks, m // 256) if world > 1 else 1) * 7
        line = {
            "metric": "quant_gemm_tflops_prefill", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp8_e4m3" if variant == "fp8" else "w4a16", "data": "synthetic",
            "config": workload_config(world, variant),
            "details": {"all_reduce": "in-switch (multimem.ld_reduce / multimem.st over the NVLS mapping) when available, else NCCL bf16",
                        "multimem": bool(layer.use_multimem), "split_reduce": split, "cuda_graph": graphed, "m_chunks": chunks,
                        "l2": "weights per rank exceed the 126 MB L2 up to tp8 (88 MB FP8 per rank at tp8 plus activations)"},
            "timing": stats,
            "tp1_ms": tp1["ms"], "tp1_timing": tp1["stats"], "speedup_vs_tp1": tp1["ms"] / ms,
            "roofline": {"bound": "tensor", "achieved": value, "peak": fp8_peak * world, "unit": "TFLOP/s", "frac": value / (fp8_peak * world),
                         "traffic": None, "target_ms": target * 1e3, "frac_of_target": target * 1e3 / ms,
                         "peak_note": f"per rank: max(flop / (2 x bf16 burst, {peaks['source']}), all-reduce bytes / 770 GB/s); regions are milliseconds of isolated steps"},
            "e2e": {"value": layer.flops(m) / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": m * HIDDEN * 2,
                    "d2h_bytes_per_step": m * HIDDEN * 2, "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "overlap": "every rank copies 1/N of the rows of X in and 1/N of the rows of the result out over its own PCIe link; X is all-gathered over NVLink; steps double-buffered over three streams"},
            "gpu_launches": args.steps * kernels_per_step * stats["repeats"], "clocks": clocks, "extras": {"decode_points": small},
        }
        if attn is not None:
            line["extras"]["qkv_o_projections_fp8"] = attn
        if parity is not None:
            line["parity"] = parity
        if phases is not None:
            kern = sum(phases.values())
            ph = {k: round(v, 4) for k, v in phases.items()}
            ph["exchange_barriers_skew"] = round(max(ms - kern, 0.0), 4)
            ph["largest"] = max(ph, key=lambda k: ph[k])
            line["phases_ms"] = ph
        print(json.dumps(line), flush=True)
    if parity is not None and not parity["ok"]:
        raise SystemExit(f"rank {rank}: tensor-parallel layer differs from its references by more than {MAX_REL}: {parity}")


def run_ours(args):
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    from oxicuda_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    torch.cuda.set_device(local_rank)
    if dist_on:
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    peaks = load_peaks(args.peaks)
    if dist_on:
        try:
            run_tp_mlp(args, torch, world, rank, local_rank, peaks)
        finally:
            torch.distributed.barrier()
            torch.distributed.destroy_process_group()
        return

    g = torch.Generator(device="cuda").manual_seed(rank)
    a = torch.randn((M, K), generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn((N, K), generator=g, device="cuda").to(torch.bfloat16)
    qa, sa = ops.fp8_quant_dynamic(a)
    qb, sb = ops.fp8_quant_dynamic(b)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    sa1, sb1 = sa[1:], sb[1:]

    def step():
        ops.gemm_fp8(qa, qb, sa1, sb1, out=y)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    if ops.handle().device_status() != 0:
        raise SystemExit("device-side wait expired during warm-up")
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_per_step, stats = timed_median(torch, step, args.steps, False)
    value = FLOP / (ms_per_step * 1e-3) / 1e12
    sus_ms = sustained_rate(torch, step, args.steps)
    sus_value = FLOP / (sus_ms * 1e-3) / 1e12
    clocks = sampler.stop()                               # samples of the timed regions and of the sustained loop after them

    # ---- end to end through host buffers ------------------------------------------------------
    # Every step copies both bf16 operands from pinned host memory, quantises them, multiplies and copies the bf16
    # result back.  Steps are independent batches, so they are double-buffered over three streams: step i+1's
    # host-to-device copies run while step i computes and returns its result (PCIe is full duplex).
    a_h = a.cpu().pin_memory()
    b_h = b.cpu().pin_memory()
    y_h = [torch.empty((M, N), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    a_d, b_d = [torch.empty_like(a) for _ in range(2)], [torch.empty_like(b) for _ in range(2)]
    y2 = [torch.empty_like(y) for _ in range(2)]
    qa2, qb2 = torch.empty_like(qa), torch.empty_like(qb)
    st_a, st_b = torch.empty(2, device="cuda"), torch.empty(2, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]          # operands of the slot have arrived
    ev_free = [torch.cuda.Event() for _ in range(2)]        # the slot's operands have been consumed
    ev_done = [torch.cuda.Event() for _ in range(2)]        # the slot's result is ready on the device
    ev_out = [torch.cuda.Event() for _ in range(2)]         # the slot's result has left the device
    main = torch.cuda.current_stream()
    step_no = [0]

    def e2e_step():
        i = step_no[0] & 1
        step_no[0] += 1
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_free[i])
            a_d[i].copy_(a_h, non_blocking=True)
            b_d[i].copy_(b_h, non_blocking=True)
            ev_in[i].record(s_in)
        main.wait_event(ev_in[i])
        main.wait_event(ev_out[i])                          # y2[i] of two steps ago has been copied out
        ops.fp8_quant_dynamic(a_d[i], out=qa2, stats=st_a)
        ops.fp8_quant_dynamic(b_d[i], out=qb2, stats=st_b)
        ev_free[i].record(main)
        ops.gemm_fp8(qa2, qb2, st_a[1:], st_b[1:], out=y2[i])
        ev_done[i].record(main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[i])
            y_h[i].copy_(y2[i], non_blocking=True)
            ev_out[i].record(s_out)

    def e2e_region(steps):
        """All copies and kernels of `steps` steps lie between the two timing events on the main stream."""
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(main)
        s_in.wait_event(e0)
        for _ in range(steps):
            e2e_step()
        main.wait_stream(s_out)
        main.wait_stream(s_in)
        e1.record(main)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    e2e_steps = max(4, min(args.steps, 10))
    e2e_region(2)
    e2e_all = sorted(e2e_region(e2e_steps) / e2e_steps for _ in range(5))
    e2e_ms = statistics.median(e2e_all)
    e2e_val = FLOP / (e2e_ms * 1e-3) / 1e12

    tab = Table(peaks)
    cpu = None
    if not args.no_extras:
        del a_h, b_h, y_h, a_d, b_d, y2, qa2, qb2
        torch.cuda.empty_cache()
        prefill_extras(torch, ops, tab, args.steps)
        torch.cuda.empty_cache()
        extras(torch, ops, tab)
        mlp_extras(torch, tab)
    from oracle import oracle as orc
    threads = orc.host_cores()
    rows = 64
    v, dt = cpu_gemm_sample(rows, threads)
    cpu = {"value": v, "unit": "TFLOP/s", "cores": threads, "kind": "port",
           "sample": f"{rows} of {M} rows of X against the full {N}x{K} weight (dequantise + f32 GEMM, reference summation order), {dt:.1f} s"}

    fp8_peak = 2.0 * peaks["bf16_tflops"]
    frac = value / fp8_peak
    line = {
        "metric": "quant_gemm_tflops_prefill", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": workload_config(1),
        "details": {"l2": "operands + output = 256 MiB per step, larger than the 126 MB L2"},
        "timing": stats,
        "roofline": {"bound": "tensor", "achieved": value, "peak": fp8_peak, "unit": "TFLOP/s",
                     "frac": frac, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                     "traffic_note": "DRAM bytes read + written per launch from an ncu capture of this kernel at this size; algorithmic operand + output bytes are 268435456",
                     "peak_note": f"2 x bf16 burst ({peaks['source']}): every timed region is {args.steps} launches after an idle gap; nominal dense FP8 is 4500",
                     "frac_of_nominal": value / 4500.0,
                     "sustained": {"achieved": sus_value, "ms_per_step": sus_ms, "peak": 2.0 * peaks["bf16_tflops_sustained"],
                                   "frac": sus_value / (2.0 * peaks["bf16_tflops_sustained"]),
                                   "note": "the same launches back to back for about 400 ms (power cap reached), against 2 x the sustained bf16 figure"},
                     "configs": tab.short},
        "e2e": {"value": e2e_val, "unit": "TFLOP/s", "h2d_bytes_per_step": 2 * M * K * 2, "d2h_bytes_per_step": M * N * 2,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "repeats": len(e2e_all), "min_ms": e2e_all[0], "max_ms": e2e_all[-1],
                "overlap": "steps double-buffered over three streams: host-to-device copies of step i+1 run during the kernels and the device-to-host copy of step i"},
        "gpu_launches": args.steps * stats["repeats"],
        "clocks": clocks,
        "cpu_baseline": cpu,
    }
    if frac > 1.05:
        line["roofline"]["warning"] = "fraction above 1 against a measured peak: check that the timed launches did the work and that the peak file is from this pool"
    if tab.long:
        line["extras"] = tab.long
    print(json.dumps(line), flush=True)


def run_case(args):
    """Single-kernel mode (what the ncu captures run): `--case gemm_fp8` launches the headline GEMM,
    the other cases one memory-bound kernel each, W warm-up + K timed launches, one JSON line."""
    import torch
    from oxicuda_b200 import ops
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(0)
    sz = args.size
    if args.case in ("gemm_fp8", "gemm_w8a8", "gemm_mxfp8", "gemm_nvfp4"):
        m, n, k = (sz, sz, sz) if args.case in ("gemm_fp8", "gemm_w8a8") else (4096 * sz // 8192, 14336 * sz // 8192, 4096 * sz // 8192)
        a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
        b = torch.randn((n, k), generator=g, device="cuda").to(torch.bfloat16)
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        if args.case == "gemm_fp8":
            qa, sa = ops.fp8_quant_dynamic(a)
            qb, sb = ops.fp8_quant_dynamic(b)
            fn = lambda: ops.gemm_fp8(qa, qb, sa[1:], sb[1:], out=y)  # noqa: E731
        elif args.case == "gemm_w8a8":
            qa, sa = ops.int8_quant_rows(a.float())
            qb, sb = ops.int8_quant_rows(b.float())
            fn = lambda: ops.gemm_w8a8(qa, qb, sa, sb, out=y)  # noqa: E731
        elif args.case == "gemm_mxfp8":
            ca, _, fa = ops.mxfp8_quant(a)
            cb, _, fb = ops.mxfp8_quant(b)
            fn = lambda: ops.gemm_mxfp8(ca, fa, cb, fb, out=y)  # noqa: E731
        else:
            pa, _, fa, sta = ops.nvfp4_quant(a)
            pb, _, fb, stb = ops.nvfp4_quant(b)
            fn = lambda: ops.gemm_nvfp4(pa, fa, sta, pb, fb, stb, out=y)  # noqa: E731
        work, unit = 2.0 * m * n * k, "TFLOP/s"
    elif args.case == "fp8_quant":
        x = torch.randn((sz, sz), generator=g, device="cuda").to(torch.bfloat16)
        q = torch.empty((sz, sz), dtype=torch.uint8, device="cuda")
        one = torch.ones(1, device="cuda")
        fn = lambda: ops.fp8_quant(x, one, out=q)  # noqa: E731
        work, unit = 3.0 * sz * sz, "GB/s"
        m = n = k = sz
    elif args.case in ("mxfp8_quant", "nvfp4_quant"):
        rows_, k = 14336 * sz // 8192, 4096                              # --size 8192: the 14336 x 4096 weight of configuration 4
        x = torch.randn((rows_, k), generator=g, device="cuda").to(torch.bfloat16)
        fn = (lambda: ops.mxfp8_quant(x)) if args.case == "mxfp8_quant" else (lambda: ops.nvfp4_quant(x))  # noqa: E731
        nel = rows_ * k
        work, unit = float(nel * 2 + nel + 2 * nel // 32) if args.case == "mxfp8_quant" else float(2 * nel * 2 + nel // 2 + 2 * nel // 16), "GB/s"
        m, n = rows_, k
    elif args.case == "int4g_quant":
        n, k = 14336 * sz // 8192, 4096
        x = torch.randn((n, k), generator=g, device="cuda") * 0.02
        fn = lambda: ops.int4g_quant_pack(x, 128)  # noqa: E731
        work, unit = float(n * k * 4 + n * k // 2 + n * k // 128 * 2 + n * k // 256), "GB/s"
        m = n
    elif args.case == "int8_quant_rows":
        x = torch.randn((sz, sz), generator=g, device="cuda") * 0.02
        fn = lambda: ops.int8_quant_rows(x)  # noqa: E731
        work, unit = 5.0 * sz * sz + 4 * sz, "GB/s"
        m = n = k = sz
    elif args.case == "gemm_w4a16":
        n, k, m = 14336, 4096, args.m
        w = torch.randn((n, k), generator=g, device="cuda") * 0.02
        c, sc, z = ops.int4g_quant_pack(w, 128)
        ring = [(c.clone(), sc.clone(), z.clone()) for _ in range(20)]
        x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
        ws = ops.gemm_w4a16_workspace(m, n, k, "cuda")
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        it = [0]

        def fn():
            r = ring[it[0] % len(ring)]
            it[0] += 1
            ops.gemm_w4a16(x, r[0], r[1], r[2], 128, workspace=ws, out=y)
        work, unit = float(n * k // 2 + n * k // 128 * 2 + n * k // 256 + m * k * 2 + m * n * 2), "GB/s"
    elif args.case == "gemm_fp8_decode":
        n, k, m = 57344 * sz // 8192, 8192, args.m                        # --size 8192: the TP1 gate/up weight of the MLP, 470 MB
        ws = []
        for _ in range(2):
            wq, st = ops.fp8_quant_dynamic(torch.randn((n, k), generator=g, device="cuda", dtype=torch.bfloat16))
            ws.append((wq, st))
        xq, sx = ops.fp8_quant_dynamic(torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16))
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        it = [0]

        def fn():
            it[0] += 1
            r = ws[it[0] % 2]
            ops.gemm_fp8(xq, r[0], sx[1:], r[1][1:], out=y)
        work, unit = float(n * k + m * k + 2 * m * n), "GB/s"
    elif args.case in ("gemm_mxfp8_decode", "gemm_nvfp4_decode"):
        n, k, m = 57344 * sz // 8192, 8192, args.m                        # two weights of n x 8192 in rotation
        mx = args.case == "gemm_mxfp8_decode"
        ws = []
        for _ in range(2):
            wb = torch.randn((n, k), generator=g, device="cuda", dtype=torch.bfloat16)
            ws.append(ops.mxfp8_quant(wb) if mx else ops.nvfp4_quant(wb))
            del wb
        xb = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
        xq = ops.mxfp8_quant(xb) if mx else ops.nvfp4_quant(xb)
        y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        it = [0]

        def fn():
            it[0] += 1
            r = ws[it[0] % 2]
            if mx:
                ops.gemm_mxfp8(xq[0], xq[2], r[0], r[2], out=y)
            else:
                ops.gemm_nvfp4(xq[0], xq[2], xq[3], r[0], r[2], r[3], out=y)
        work, unit = float((n * k * 33 // 32 if mx else n * k * 9 // 16) + m * k + 2 * m * n), "GB/s"
    elif args.case in ("rmsnorm_int8", "rmsnorm_fp8", "silu_gate_fp8"):
        ring = [torch.randn((sz, sz), generator=g, device="cuda").to(torch.bfloat16) for _ in range(3)]
        wn = torch.ones(sz, device="cuda")
        one = torch.ones(1, device="cuda")
        it = [0]

        def fn():
            it[0] += 1
            r = ring[it[0] % 3]
            if args.case == "rmsnorm_int8":
                ops.rmsnorm_int8_quant_rows(r, wn)
            elif args.case == "rmsnorm_fp8":
                ops.rmsnorm_fp8_quant_rows(r, wn, one)
            else:
                ops.silu_gate_fp8_quant(r, ring[(it[0] + 1) % 3], one)
        work, unit = (5.0 if args.case == "silu_gate_fp8" else 3.0) * sz * sz, "GB/s"
        m = n = k = sz
    elif args.case in ("nf4_quant", "gemm_nf4"):
        n, k, m = 14336 * sz // 8192, 4096, args.m                        # --size 8192 is the full 14336 x 4096 weight
        ring = [torch.randn((n, k), generator=g, device="cuda") * 0.02 for _ in range(3)]
        it = [0]
        if args.case == "nf4_quant":
            def fn():
                it[0] += 1
                ops.nf4_quant(ring[it[0] % 3].view(-1), 64)
            work, unit = float(n * k * 4 + n * k // 2 + n * k // 64 * 4), "GB/s"
        else:
            packs = [ops.nf4_quant(ring[i % 3].view(-1), 64) for i in range(6)]
            x = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
            y = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")

            def fn():
                it[0] += 1
                r = packs[it[0] % 6]
                ops.gemm_nf4(x, r[0], r[1], n, 64, out=y)
            work, unit = float(n * k // 2 + n * k // 64 * 4 + m * (k + n) * 2), "GB/s"
    else:
        raise SystemExit(f"unknown case {args.case}")
    for _ in range(args.warmup):
        fn()
    ms = time_region(torch, fn, args.steps, False) / args.steps
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"case": args.case, "m": m, "n": n, "k": k, "ms_per_launch": ms, "rate": rate, "unit": unit,
                      "steps": args.steps, "warmup": args.warmup}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--peaks", default=None, help="JSON file with hbm_gbs / bf16_tflops / bf16_tflops_sustained (default: the pool's measured peaks beside this script)")
    ap.add_argument("--case", default=None, help="single-kernel mode, e.g. gemm_fp8, gemm_mxfp8, gemm_nvfp4, fp8_quant, mxfp8_quant, nvfp4_quant, int4g_quant, int8_quant_rows, gemm_w4a16, gemm_fp8_decode, gemm_mxfp8_decode, gemm_nvfp4_decode, nf4_quant, gemm_nf4")
    ap.add_argument("--size", type=int, default=8192)
    ap.add_argument("--m", type=int, default=8)
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()

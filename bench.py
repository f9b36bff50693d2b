#!/usr/bin/env python
"""Benchmark of the block-scaled FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--passes R] [--impl ours|reference] [--detail]

One *pass* runs the six DeepSeek-V3-shaped dense FP8 GEMMs with M = 4096 that the benchmark specification's metric is
quoted on (its config 2): D[M,N] = A[M,K] @ B[N,K]^T, A quantised per token per 128 of K, B per 128 x 128 block, UE8M0
scales pre-packed, BF16 output, synthetic N(0,1) data.  A *step* is R passes (default 128, ~0.1 s of GEMMs), so that
the timed region lasts seconds: the SM clock and the board power settle where a long-running job holds them, the clock
sampler collects hundreds of samples, and the roofline denominator is the sustained one.  `value` is the aggregate
TFLOP/s (2 M N K over the six shapes x R x steps / device time) with operands resident in HBM; `e2e` is the same step
through the public Python API with host buffers (pinned host -> device copies of A, SFA, B, SFB and a device -> host
read of D for every GEMM inside the timed region).

With N > 1 (torchrun) the SAME six GEMMs are split column-parallel along N (`dist.shard_columns`: rank r holds all of
A, rows [lo, hi) of B / SFB and writes D[:, lo:hi]); no collective runs in the timed region; value = total FLOP / the
slowest rank's time: strong scaling.  The line also carries `grouped_ep`: the contiguous grouped GEMM of config 3 (32
experts, both shapes) with 32 / N experts per rank and the masked decode GEMM of config 4 (16 groups, CUDA graph) with
16 / N groups per rank, aggregate TFLOP/s over the ranks.  After the timing the shards are gathered with NCCL
(`dist.uneven_all_gather`, the pattern of the reference's deep_gemm/utils/dist.py:38-66) and compared with a
single-GPU run on rank 0: `shard_check`.

`--impl reference` times the reference path's CPU implementation (the numpy port of its torch dequantise-then-matmul,
oracle/) on the host cores on the same six shapes.
"""
from __future__ import annotations

import argparse
import json
import os
import random
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_DENSE = 4096
DENSE_NK = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]
GROUPED_NK = [(4096, 7168), (7168, 2048)]
NOMINAL_FP8_TFLOPS = 4500.0
FP8_FLOP_PER_CLK_PER_SM = 16384          # dense FP8 tensor rate of one SM: 8192 multiply-adds per clock
DEFAULT_PASSES = 128
# dram__bytes_read.sum + dram__bytes_write.sum per launch of dg_gemm_fp8_fp4 at M = 4096 on one GPU, from one ncu
# capture of this script (profiles/dg_gemm_fp8_fp4_dense_m4096.md), with the tile the capture ran (rows per CTA, tile
# columns, raster group, CTAs per tile): the figure is reported only while the heuristics still choose that tile (D
# written late in a launch may still sit in L2 when it ends).
NCU_DRAM_BYTES = {(2112, 7168): (46705920, (256, 240, 4, 2)), (24576, 1536): (229373696, (128, 240, 8, 2)),
                  (32768, 512): (247539968, (256, 240, 4, 2)), (7168, 16384): (535451904, (128, 224, 8, 2)),
                  (4096, 7168): (72103424, (256, 240, 4, 2)), (7168, 2048): (31843328, (128, 224, 8, 2))}


def flops_of(m, n, k):
    return 2.0 * m * n * k


def dense_bytes(m, n, k):
    """A + B + D + packed scales: the bytes one launch has to move (tests/test_fp8_fp4.py:110 of the reference)."""
    return m * k + n * k + m * n * 2 + (m + n) * (-(-k // 512)) * 4


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------------
# Clock and power sampling during a timed region (NVML reads only)
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period, self.samples, self.power, self.reasons = index, period_s, [], [], set()
        self.max_mhz, self._stop, self._thread, self._nvml = None, threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None

    def _run(self):
        nv = self._nvml
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                self.power.append(nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0)
                get = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
                mask = get(self._h)
                for name, bit in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        # the first quarter of the samples still shows the ramp from idle
        s = sorted(self.samples[len(self.samples) // 4:])
        w = sorted(self.power[len(self.power) // 4:])
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_mhz_min": s[0] if s else None, "sm_max_mhz": self.max_mhz,
                "power_w": round(w[len(w) // 2], 1) if w else None, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ----------------------------------------------------------------------------------------------------
# CPU arm: the reference path's dequantise-then-matmul on the host cores (numpy port in oracle/)
# ----------------------------------------------------------------------------------------------------
def cpu_inputs(nk_list):
    """The same recipe as the GPU arm, prepared on the host by the oracle's quantisers (row chunks in parallel)."""
    import oracle
    cases = []
    for i, (n, k) in enumerate(nk_list):
        a, b = oracle.seeded_bf16_rows((M_DENSE, k), 100 + i), oracle.seeded_bf16_rows((n, k), 200 + i)
        cases.append(oracle.quantise_dense_parallel(a, b))
    return cases


def cpu_step(cases):
    import oracle
    out = None
    for qa, sfa, qb, sfb in cases:
        out = oracle.bf16_round(oracle.dequant_gemm_nt(qa, sfa, qb, sfb))
    return out


def time_cpu(steps, warmup, nk_list=None):
    """Seconds per step of the CPU port over `nk_list` (default: all six shapes) with every host core this process may
    use (torchrun exports OMP_NUM_THREADS=1 for its workers, so the BLAS pool is widened explicitly)."""
    import numpy  # noqa: F401  (BLAS must be loaded before its pool can be resized)
    import oracle
    nk_list = nk_list or DENSE_NK
    cases = cpu_inputs(nk_list)
    ncpu = oracle.host_threads()
    threads = ncpu
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        limiter = threadpool_limits(limits=ncpu)
    except Exception:
        limiter = None
    for _ in range(warmup):
        cpu_step(cases)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(cases)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    try:
        blas = [p["num_threads"] for p in threadpool_info() if p.get("user_api") == "blas"]
        threads = max(blas) if blas else ncpu
    except Exception:
        pass
    if limiter is not None:
        limiter.restore_original_limits()
    flops = sum(flops_of(M_DENSE, n, k) for n, k in nk_list)
    return flops / dt / 1e12, dt, threads


def run_reference_arm(args, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))           # bounded: a CPU step over the six shapes is ~15 s
    warm = max(0, min(args.warmup, 1))
    tflops, dt, threads = time_cpu(steps, warm)
    sample = f"all six M={M_DENSE} shapes of config 2 (one pass), dequantise + FP32 matmul, {steps} steps of {dt:.1f} s"
    line = {
        "impl": "reference", "metric": "dense_fp8_gemm_tflops", "value": round(tflops, 4), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "dense_fp8_gemm_nt_m4096 (BASELINE config 2, the six (N,K) at M=4096)",
                   "shapes_mnk": [[M_DENSE, n, k] for n, k in DENSE_NK], "passes_per_step": 1,
                   "sample": sample},
        "cpu_baseline": {"value": round(tflops, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": round(tflops, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------
def make_dense_case(m, n, k, seed, torch, dg, columns=None, fp4=False):
    """One dense case; with `columns = (lo, hi)` only that column shard of the problem: rows [lo, hi) of B and of its
    scales (cut on multiples of 128, so the 128 x 128 scale blocks are those of the whole matrix) and D[:, lo:hi].
    `fp4`: both operands packed E2M1 with 1 x 32 scales (the kind::mxf4 kernel; profiling runs on one GPU)."""
    from deepgemm_amd_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp4, per_token_cast_to_fp8
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16, generator=g)
    b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=g)
    if fp4:
        assert columns is None
        qa, sfa = per_token_cast_to_fp4(a, True, 32)
        qb, sfb = per_token_cast_to_fp4(b, True, 32)
        raw = (sfa, sfb)
        sfa = dg.transform_sf_into_required_layout(sfa, m, k, (1, 32))
        sfb = dg.transform_sf_into_required_layout(sfb, n, k, (1, 32))
        d = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
        return {"m": m, "n": n, "k": k, "full_n": n, "columns": (0, n), "a": (qa, sfa), "b": (qb, sfb), "d": d, "seed": seed,
                "scales_fp32": raw, "recipe": {"recipe_a": (1, 32), "recipe_b": (1, 32)}}
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    qb, sfb = per_block_cast_to_fp8(b, True)
    lo, hi = columns if columns is not None else (0, n)
    assert lo % 128 == 0
    qb, sfb = qb[lo:hi].contiguous(), sfb[lo // 128:-(-hi // 128)].contiguous()
    raw = (sfa, sfb)
    sfa = dg.transform_sf_into_required_layout(sfa, m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(sfb, hi - lo, k, (128, 128))
    d = torch.empty((m, hi - lo), device="cuda", dtype=torch.bfloat16)
    return {"m": m, "n": hi - lo, "k": k, "full_n": n, "columns": (lo, hi), "a": (qa, sfa), "b": (qb, sfb), "d": d, "seed": seed,
            "scales_fp32": raw, "recipe": {"recipe": (1, 1, 128)}}


def flat_storage(t, torch):
    """The whole allocation behind a (possibly strided) tensor as a flat view, for host <-> device copies."""
    span = 1 + sum((s - 1) * st for s, st in zip(t.shape, t.stride()))
    return torch.as_strided(t, (span,), (1,))


def time_events(fn, steps, torch, dist_barrier):
    dist_barrier()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    end.record()
    torch.cuda.synchronize()
    dist_barrier()
    return start.elapsed_time(end) / 1e3


def max_over_ranks(value, torch, dist, world):
    t = torch.tensor([value], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def dequant_reference(case, torch):
    """Dequantise-then-matmul value of a dense case on the GPU: a BF16 tensor-core matmul of the dequantised operands
    (an FP8 value times a power of two is exact in BF16), the yardstick of shard_check."""
    from deepgemm_amd_b200.utils import cast_back_from_fp8
    qa, qb = case["a"][0], case["b"][0]
    sfa, sfb = case["scales_fp32"]                       # per token x 128 of K; per 128 x 128 block
    n, k = qb.shape
    a_deq = cast_back_from_fp8(qa, sfa).bfloat16()
    rows = torch.arange(n, device=qb.device) // 128
    cols = torch.arange(k, device=qb.device) // 128
    b_deq = (qb.float() * sfb[rows][:, cols]).bfloat16()
    return (a_deq @ b_deq.t()).float()


def grouped_layout(seed=0, groups=32, expected=8192, alignment=128):
    """Token counts per expert int(8192 U(0.7, 1.3)), padded to the alignment (tests/generators.py:383-404)."""
    rng = random.Random(seed)
    actual = [int(expected * rng.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [-(-x // alignment) * alignment for x in actual]
    return actual, aligned


def make_contiguous_shard(n, k, experts, actual, aligned, torch, dg):
    """Experts [g0, g1) of the config-3 problem: their row segments of A (padding rows zero), their weights, expert ids
    re-based to the shard.  Every expert's data comes from its own seed, so any rank can rebuild any shard."""
    from deepgemm_amd_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp8
    g0, g1 = experts
    rows = sum(aligned[g0:g1])
    qa = torch.empty((rows, k), device="cuda", dtype=torch.float8_e4m3fn)
    sfa = torch.empty((rows, k // 128), device="cuda", dtype=torch.float32)
    layout = torch.full((rows,), -1, dtype=torch.int, device="cuda")
    qbs, sfbs, start = [], [], 0
    for g in range(g0, g1):
        gen = torch.Generator(device="cuda").manual_seed(7000 + 31 * g + n)
        a = torch.randn((aligned[g], k), device="cuda", dtype=torch.bfloat16, generator=gen)
        a[actual[g]:] = 0
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=gen)
        qa[start:start + aligned[g]], sfa[start:start + aligned[g]] = per_token_cast_to_fp8(a, True, 128)
        q, s = per_block_cast_to_fp8(w, True)
        qbs.append(q)
        sfbs.append(s)
        layout[start:start + actual[g]] = g - g0
        start += aligned[g]
        del a, w
    sfa_p = dg.transform_sf_into_required_layout(sfa, rows, k, (1, 128))
    sfb_p = dg.transform_sf_into_required_layout(torch.stack(sfbs), n, k, (128, 128), g1 - g0)
    d = torch.empty((rows, n), device="cuda", dtype=torch.bfloat16)
    return {"a": (qa, sfa_p), "b": (torch.stack(qbs), sfb_p), "d": d, "layout": layout, "rows": rows,
            "valid": sum(actual[g0:g1]), "n": n, "k": k}


def make_masked_shard(groups, max_m, n, k, counts, torch, dg):
    """Groups [g0, g1) of the config-4 decode problem, each from its own seed."""
    from deepgemm_amd_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp8
    g0, g1 = groups
    qa = torch.empty((g1 - g0, max_m, k), device="cuda", dtype=torch.float8_e4m3fn)
    sfa = torch.empty((g1 - g0, max_m, k // 128), device="cuda")
    qb = torch.empty((g1 - g0, n, k), device="cuda", dtype=torch.float8_e4m3fn)
    sfb = torch.empty((g1 - g0, n // 128, k // 128), device="cuda")
    for g in range(g0, g1):
        gen = torch.Generator(device="cuda").manual_seed(9000 + g)
        a = torch.randn((max_m, k), device="cuda", dtype=torch.bfloat16, generator=gen)
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=gen)
        qa[g - g0], sfa[g - g0] = per_token_cast_to_fp8(a, True, 128)
        qb[g - g0], sfb[g - g0] = per_block_cast_to_fp8(w, True)
    sfa_p = dg.transform_sf_into_required_layout(sfa, max_m, k, (1, 128), g1 - g0)
    sfb_p = dg.transform_sf_into_required_layout(sfb, n, k, (128, 128), g1 - g0)
    masked = torch.tensor(counts[g0:g1], dtype=torch.int, device="cuda")
    d = torch.zeros((g1 - g0, max_m, n), device="cuda", dtype=torch.bfloat16)
    return {"a": (qa, sfa_p), "b": (qb, sfb_p), "d": d, "masked": masked, "valid": sum(counts[g0:g1])}


def run_grouped_ep(torch, dist, dg, rank, world, barrier, check):
    """Configs 3 and 4 expert-parallel over the ranks: every rank holds 32 / N experts (16 / N groups) and runs the
    grouped GEMM on its shard; time = slowest rank (device events, 256 MB L2 flush before every call), TFLOP/s counts
    valid rows over all ranks.  With `check`, the shards' outputs are gathered afterwards and compared on rank 0 with a
    single-GPU run over all experts."""
    from deepgemm_amd_b200.dist import shard_experts, uneven_all_gather
    from deepgemm_amd_b200.testing import bench as bench_events
    out, checks = {}, {}
    actual, aligned = grouped_layout()
    g0, g1 = shard_experts(32, world, rank)
    for n, k in GROUPED_NK:
        name = f"contiguous_g32_n{n}_k{k}"
        if g1 > g0:
            sh = make_contiguous_shard(n, k, (g0, g1), actual, aligned, torch, dg)
            call = lambda: dg.m_grouped_fp8_gemm_nt_contiguous(sh["a"], sh["b"], sh["d"], sh["layout"], recipe=(1, 1, 128))
            barrier()
            t = bench_events(call, 3, 10)
        else:
            sh, t = None, 0.0
        t_max = max_over_ranks(t, torch, dist, world)
        out[name] = {"tflops": round(flops_of(sum(actual), n, k) / t_max / 1e12, 1), "ms": round(t_max * 1e3, 3),
                     "experts_per_gpu": g1 - g0, "rows_total": sum(aligned), "rows_valid": sum(actual)}
        if check and world > 1:
            local = sh["d"] if sh is not None else torch.empty((0, n), device="cuda", dtype=torch.bfloat16)
            gathered = uneven_all_gather(local, dim=0)
            if rank == 0:
                del sh
                full = make_contiguous_shard(n, k, (0, 32), actual, aligned, torch, dg)
                dg.m_grouped_fp8_gemm_nt_contiguous(full["a"], full["b"], full["d"], full["layout"], recipe=(1, 1, 128))
                valid = full["layout"] >= 0
                checks[name] = {"bitwise_equal_to_single_gpu": bool(torch.equal(gathered[valid].view(torch.int16), full["d"][valid].view(torch.int16))),
                                "rows_compared": int(valid.sum())}
                del full
            del gathered
        sh = None
        torch.cuda.empty_cache()
    # config 4: masked decode GEMM, replayed from a CUDA graph
    groups, max_m, n, k = 16, 256, 4096, 7168
    rng = random.Random(4)
    counts = [rng.randint(45, 83) for _ in range(groups)]
    g0, g1 = shard_experts(groups, world, rank)
    name = f"masked_g{groups}_maxm{max_m}_n{n}_k{k}_cuda_graph"
    t, sh = 0.0, None
    if g1 > g0:
        sh = make_masked_shard((g0, g1), max_m, n, k, counts, torch, dg)
        call = lambda: dg.m_grouped_fp8_gemm_nt_masked(sh["a"], sh["b"], sh["d"], sh["masked"], 64, recipe=(1, 1, 128))
        call()
        torch.cuda.synchronize()
        graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                call()
        barrier()
        t = bench_events(graph.replay, 3, 20)
    t_max = max_over_ranks(t, torch, dist, world)
    out[name] = {"tflops": round(flops_of(sum(counts), n, k) / t_max / 1e12, 1), "us": round(t_max * 1e6, 1),
                 "gbs": round((sum(counts) * k + groups * n * k + sum(counts) * n * 2) / t_max / 1e9, 0),
                 "groups_per_gpu": g1 - g0, "rows_valid": sum(counts)}
    if check and world > 1:
        local = sh["d"] if sh is not None else torch.empty((0, max_m, n), device="cuda", dtype=torch.bfloat16)
        gathered = uneven_all_gather(local, dim=0)
        if rank == 0:
            full = make_masked_shard((0, groups), max_m, n, k, counts, torch, dg)
            dg.m_grouped_fp8_gemm_nt_masked(full["a"], full["b"], full["d"], full["masked"], 64, recipe=(1, 1, 128))
            checks[name] = {"bitwise_equal_to_single_gpu": bool(torch.equal(gathered.view(torch.int16), full["d"].view(torch.int16)))}
    out["scaling"] = "strong (the whole problem is split over the ranks)"
    out["timing"] = "mean of 10 calls (C4: 20 graph replays), a 256 MB L2 flush before each, device events, max over ranks"
    return out, checks


def run_reference_gpu(timeout_s=420):
    """The UNMODIFIED reference's own sm_100 kernel on this GPU, for the same six shapes: baseline/reference_arm.py in a
    child process (the reference installed by baseline/build_ref.py into the git-ignored baseline/_ref; its JIT runtime,
    an un-vendored submodule, is replaced by the stand-in under baseline/deep_jit_standin).  Burst = its own bench_kineto
    (profiler kernel time, L2 flushed before every call); sustained = the same back-to-back loop as `sustained_rows`."""
    import subprocess
    import tempfile
    script = os.path.join(ROOT, "baseline", "reference_arm.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "deep_gemm")):
        return {"unavailable": "baseline/_ref holds no reference installation on this machine (built by baseline/build_ref.py where the reference tree exists)"}
    with tempfile.NamedTemporaryFile(suffix=".json", delete=False) as f:
        out_path = f.name
    try:
        res = subprocess.run([sys.executable, script, "--stage", "dense", "--m", str(M_DENSE), "--sustained", "--out", out_path],
                             capture_output=True, text=True, timeout=timeout_s)
        if res.returncode != 0 or not os.path.getsize(out_path):
            tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or ["no output"]
            return {"unavailable": f"reference_arm.py exited {res.returncode}: {tail[0][:160]}"}
        data = json.load(open(out_path))
    except subprocess.TimeoutExpired:
        return {"unavailable": f"reference_arm.py did not finish within {timeout_s} s"}
    finally:
        try:
            os.unlink(out_path)
        except OSError:
            pass
    rows = data.get("dense", [])
    if len(rows) != len(DENSE_NK):
        return {"unavailable": "reference_arm.py returned no dense rows", "detail": {k: v for k, v in data.items() if k != "dense"}}
    flops = sum(flops_of(M_DENSE, n, k) for n, k in DENSE_NK)
    burst = sum(r["us"] for r in rows) * 1e-6
    sustained = sum(r.get("sustained_us", 0.0) for r in rows) * 1e-6
    return {"what": "the reference's sm100_fp8_fp4_gemm_1d1d_impl through its own Python API, heuristics and launcher (DeepGEMM "
                    + str(data.get("reference_version")) + ", DeepJIT replaced by a stand-in)",
            "burst_tflops": round(flops / burst / 1e12, 1), "sustained_tflops": round(flops / sustained / 1e12, 1) if sustained else None,
            "bitwise_equal_to_this_repository": all(r.get("bitwise_equal_to_this_repository") for r in rows),
            "rows": [{k: r.get(k) for k in ("case", "us", "tflops", "sustained_us", "sustained_tflops", "sm_mhz", "power_w")} for r in rows]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--passes", type=int, default=DEFAULT_PASSES, help="passes over the six shapes per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--detail", action="store_true", help="also time each shape of configs 2-5 on its own (rank 0)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-grouped", action="store_true", help="skip the grouped_ep record (profiling runs)")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the run of the reference's own GPU kernel (N = 1 only)")
    ap.add_argument("--no-graph", action="store_true", help="launch every GEMM from Python instead of replaying one CUDA graph per step")
    ap.add_argument("--pdl", action="store_true", help="launch the GEMMs with programmatic dependent launch (set_pdl)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--shapes", default="", help="comma-separated NxK subset of the six dense shapes (profiling runs)")
    ap.add_argument("--fp4", action="store_true", help="both operands FP4 with 1 x 32 scales: the kind::mxf4 kernel (profiling runs, one GPU)")
    ap.add_argument("--m", type=int, default=M_DENSE, help="rows of A (profiling runs of the M = 64 / 128 shapes; the metric is quoted at 4096)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    args.passes = max(1, args.passes)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    import deepgemm_amd_b200 as dg
    from deepgemm_amd_b200.dist import init_dist, shard_columns, uneven_all_gather

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GEMM path has no CPU fallback (use --impl reference for the CPU arm)")
    rank, world, local_rank = init_dist()
    torch.cuda.set_device(local_rank)
    num_sms = torch.cuda.get_device_properties(local_rank).multi_processor_count

    def barrier():
        if world > 1:
            dist.barrier()

    nk_list = DENSE_NK
    if args.shapes:
        nk_list = [tuple(int(v) for v in s.split("x")) for s in args.shapes.split(",")]
    # The same problem on every rank (same seeds); with N > 1 each rank keeps its column shard of B and D
    cases = []
    for i, (n, k) in enumerate(nk_list):
        cols = shard_columns(n, world, rank) if world > 1 else None
        if cols is not None and cols[1] <= cols[0]:
            continue                                   # fewer 128-column blocks than ranks: this rank idles on this shape
        cases.append(make_dense_case(args.m, n, k, 1000 + i, torch, dg, cols, fp4=args.fp4))
    pass_flops = sum(flops_of(args.m, n, k) for n, k in nk_list)            # of the WHOLE problem, whatever the split

    def one_pass():
        for c in cases:
            dg.fp8_fp4_gemm_nt(c["a"], c["b"], c["d"], **c["recipe"])

    # The library's launch option (the reference's set_pdl): a GEMM's set-up overlaps the tail of the one before.
    # Off by default, as in the library: on this step it measured 2 % slower.
    dg.set_pdl(args.pdl)
    one_pass()
    torch.cuda.synchronize()
    # One step = R passes.  Replaying them from a CUDA graph keeps the host out of the timed region (the launches of a
    # pass cost ~70 us of Python, comparable with a pass on 8 GPUs); --no-graph launches every GEMM from Python.
    graph = None
    if not args.no_graph and cases:
        graph, gstream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(gstream):
            with torch.cuda.graph(graph, stream=gstream):
                for _ in range(args.passes):
                    one_pass()

    def step():
        if graph is not None:
            graph.replay()
        else:
            for _ in range(args.passes):
                one_pass()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if dg.kernel_status() != 0:
        raise SystemExit(f"kernel reported status {dg.kernel_status():#x}")

    barrier()                      # first collective initialises NCCL: keep that out of the sampled region
    with ClockSampler(local_rank) as clocks:
        dt = time_events(step, args.steps, torch, barrier)
    dt_max = max_over_ranks(dt, torch, dist, world)
    value = pass_flops * args.passes * args.steps / dt_max / 1e12

    # ---- end to end through the public API with host buffers ---------------------------------------
    host, dev_flat = [], []
    for c in ([] if args.no_e2e else cases):
        tensors = [c["a"][0], c["a"][1], c["b"][0], c["b"][1]]
        flats = [flat_storage(x, torch) for x in tensors]
        flats = [f.view(torch.uint8) if f.dtype == torch.float8_e4m3fn else f for f in flats]
        host.append([f.cpu().pin_memory() for f in flats] + [torch.empty(c["d"].shape, dtype=c["d"].dtype).pin_memory()])
        dev_flat.append(flats)
    h2d = sum(h.numel() * h.element_size() for hs in host for h in hs[:-1])
    d2h = sum(hs[-1].numel() * hs[-1].element_size() for hs in host)

    # Copies in, GEMMs and copies out run on three streams chained by events, so that the two PCIe directions and the
    # tensor cores work at the same time; every stream is joined back into the current one at the end of a pass.
    # A case's inputs are not overwritten before its previous GEMM has read them, nor its D before the previous
    # read-back has finished.
    s_in, s_mm, s_out = (torch.cuda.Stream() for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in cases]
    ev_mm = [torch.cuda.Event() for _ in cases]
    ev_out = [torch.cuda.Event() for _ in cases]

    def e2e_pass():
        cur = torch.cuda.current_stream()
        for s_ in (s_in, s_mm, s_out):
            s_.wait_stream(cur)
        for i, (c, hs, fs) in enumerate(zip(cases, host, dev_flat)):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_mm[i])                 # the previous pass's GEMM of this case has consumed the inputs
                for h, f in zip(hs[:-1], fs):
                    f.copy_(h, non_blocking=True)
                ev_in[i].record(s_in)
            with torch.cuda.stream(s_mm):
                s_mm.wait_event(ev_in[i])
                s_mm.wait_event(ev_out[i])                # the previous pass's read-back of this D is complete
                dg.fp8_fp4_gemm_nt(c["a"], c["b"], c["d"], **c["recipe"])
                ev_mm[i].record(s_mm)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_mm[i])
                hs[-1].copy_(c["d"], non_blocking=True)
                ev_out[i].record(s_out)
        for s_ in (s_in, s_mm, s_out):
            cur.wait_stream(s_)

    def e2e_step():
        for _ in range(args.passes):
            e2e_pass()

    e2e_steps = max(1, min(args.steps, 3))
    e2e_value = None
    if not args.no_e2e:
        e2e_pass()
        e2e_dt = max_over_ranks(time_events(e2e_step, e2e_steps, torch, barrier), torch, dist, world)
        e2e_value = pass_flops * args.passes * e2e_steps / e2e_dt / 1e12

    # ---- the partitions of configs 3 and 4, and the shards checked against one GPU ------------------
    grouped, checks = (None, {})
    if not args.no_grouped and not args.shapes and args.m == M_DENSE:
        grouped, checks = run_grouped_ep(torch, dist, dg, rank, world, barrier, check=True)
    dense_check = None
    if world > 1 and not args.shapes:
        worst, bitwise = 0.0, True
        for i, (n, k) in enumerate(nk_list):
            mine = [c for c in cases if c["full_n"] == n and c["k"] == k]
            local = mine[0]["d"] if mine else torch.empty((args.m, 0), device="cuda", dtype=torch.bfloat16)
            gathered = uneven_all_gather(local, dim=1)
            if rank == 0:
                full = make_dense_case(args.m, n, k, 1000 + i, torch, dg)
                dg.fp8_gemm_nt(full["a"], full["b"], full["d"], recipe=(1, 1, 128))
                bitwise = bitwise and bool(torch.equal(gathered.view(torch.int16), full["d"].view(torch.int16)))
                from deepgemm_amd_b200.testing import calc_diff
                worst = max(worst, float(calc_diff(gathered, dequant_reference(full, torch))))
                del full
            del gathered
        dense_check = {"calc_diff_max_vs_dequantised_matmul": worst, "bitwise_equal_to_single_gpu": bitwise, "shapes": len(nk_list)}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    clk = clocks.summary()
    per_gpu = value / world
    # The dominant (only) kernel of the step is the tcgen05 GEMM; FP8 runs at twice the BF16 tensor rate, so the measured
    # denominator is 2 x the cuBLAS BF16 figure: the sustained one when the timed region is long enough for clocks and
    # power to settle (>= 1 s), else the burst one.
    sustained = dt_max >= 1.0
    peak_fp8 = 2.0 * (peaks["bf16_sustained"] if sustained else peaks["bf16_burst"])
    peak_at_clock = None if not clk["sm_mhz"] else FP8_FLOP_PER_CLK_PER_SM * num_sms * clk["sm_mhz"] * 1e6 / 1e12
    traffic = None
    if world == 1 and args.m == M_DENSE:
        known = []
        for c in cases:
            cfg = dg.get_gemm_config(0, c["m"], c["n"], c["k"])
            ent = NCU_DRAM_BYTES.get((c["n"], c["k"]))
            known.append(ent[0] if ent is not None and ent[1] == (cfg["block_m"], cfg["block_n"], cfg["raster_group"], cfg["cluster_size"]) else None)
        traffic = None if any(v is None for v in known) else round(sum(known) / len(known))
    launches_per_step = args.passes * len(cases)
    algorithmic = sum(dense_bytes(c["m"], c["n"], c["k"]) for c in cases) / max(len(cases), 1)
    line = {
        "metric": "dense_fp8_gemm_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt_max / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)",
        "data": "synthetic",
        "config": {"workload": "dense_fp8_gemm_nt_m4096 (BASELINE config 2, the six (N,K) at M=4096)" if args.m == M_DENSE and not args.shapes and not args.fp4
                               else f"profiling subset: M={args.m}, {len(nk_list)} of the dense shapes" + (", FP4 x FP4 (kind::mxf4)" if args.fp4 else ""),
                   "shapes_mnk": [[args.m, n, k] for n, k in nk_list],
                   "passes_per_step": args.passes,
                   "scales": "UE8M0 packed int32, A 1x128, B 128x128 pre-broadcast",
                   "pdl": args.pdl, "cuda_graph_per_step": graph is not None,
                   "l2": "no flush: every pass streams its operands (1.0 GB on one GPU, >= 0.25 GB per rank on eight) through "
                         "six different shapes, more than the 126 MB L2",
                   "parallelism": "1 GPU" if world == 1 else f"column-parallel along N over {world} ranks (shards on multiples of 128 columns), "
                                                             "A replicated, no collective in the timed region"},
        "pct_of_nominal_fp8_peak": round(100.0 * per_gpu / NOMINAL_FP8_TFLOPS, 2),
        "roofline": {"bound": "tensor", "achieved": round(per_gpu, 2), "peak": round(peak_fp8, 1), "unit": "TFLOP/s",
                     "frac": round(per_gpu / peak_fp8, 4), "traffic": traffic, "traffic_unit": "bytes per launch (mean of the step's launches)",
                     "algorithmic_bytes_per_launch": round(algorithmic),
                     "regime": "sustained" if sustained else "burst",
                     "timed_region_s": round(dt_max, 3),
                     "peak_source": f"2 x bf16_tflops{'_sustained' if sustained else ''} of MEASURED_PEAKS.json ({peaks['source']}); nominal FP8 dense 4500",
                     "frac_of_nominal": round(per_gpu / NOMINAL_FP8_TFLOPS, 4),
                     "peak_at_sampled_clock": None if peak_at_clock is None else round(peak_at_clock, 1),
                     "frac_clock_adjusted": None if peak_at_clock is None else round(per_gpu / peak_at_clock, 4),
                     "clock_adjusted_note": f"{FP8_FLOP_PER_CLK_PER_SM} FLOP/clk/SM x {num_sms} SMs x the median SM clock sampled during the timed region"},
        "clocks": clk,
        "e2e": {"value": None if e2e_value is None else round(e2e_value, 3), "unit": "TFLOP/s",
                "h2d_bytes_per_step": h2d * args.passes, "d2h_bytes_per_step": d2h * args.passes,
                "steps": e2e_steps, "per_rank_bytes": world > 1,
                "overlap": "copies in, GEMMs and copies out on three streams chained by events"},
        "gpu_launches": args.steps * launches_per_step,
    }
    if grouped is not None:
        line["grouped_ep"] = grouped
    if dense_check is not None or checks:
        line["shard_check"] = {"dense_column_parallel": dense_check, "grouped_expert_parallel": checks}
    if world == 1 and not args.no_cpu_baseline:
        tflops, cdt, threads = time_cpu(1, 0)
        line["cpu_baseline"] = {"value": round(tflops, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                                "sample": f"one pass over all six M={M_DENSE} shapes, {cdt:.1f} s of dequantise + FP32 matmul on the host"}
    if world == 1 and not args.no_reference_gpu and not args.shapes and args.m == M_DENSE:
        # our own six shapes in the same two regimes, then the reference's kernel: both after the timed regions above
        ours = sustained_rows(torch, dg, local_rank, num_sms, dense_only=True, with_library=False)
        line["per_shape_sustained"] = ours
        line["reference_gpu"] = run_reference_gpu()
    if args.detail:
        line["detail"] = detail_rows(torch, dg)
        line["sustained"] = sustained_rows(torch, dg, local_rank, num_sms)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def make_grouped_b(groups, n, k, fp4, torch, dg):
    from deepgemm_amd_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp4
    b = torch.randn((groups, n, k), device="cuda", dtype=torch.bfloat16)
    if fp4:
        qs = [per_token_cast_to_fp4(b[g], True, 32) for g in range(groups)]
        recipe = (1, 32)
    else:
        qs = [per_block_cast_to_fp8(b[g], True) for g in range(groups)]
        recipe = (128, 128)
    qb = torch.stack([q for q, _ in qs])
    sfb = dg.transform_sf_into_required_layout(torch.stack([s for _, s in qs]), n, k, recipe, groups)
    return qb, sfb


def detail_rows(torch, dg):
    """Per-case kernel times (torch profiler records, 256 MB L2 flush before every call) for benchmark configurations 2-5.  TFLOP/s counts valid
    rows only and GB/s the bytes of A, B, D and scales, as the reference's tests print them
    (tests/test_fp8_fp4.py:108-111,170-174,229-237)."""
    import random
    from deepgemm_amd_b200.testing import bench_kineto
    from deepgemm_amd_b200.utils import per_token_cast_to_fp4, per_token_cast_to_fp8
    rows = []
    kernels = ("dg_gemm_fp8_fp4", "splitk_reduce_kernel")      # the split-K second pass counts as part of the GEMM

    def bench(fn, warmups, tests):
        for _ in range(warmups):
            fn()
        return bench_kineto(fn, kernels, tests, span=True)      # GEMM start to reduce end: the two overlap under PDL

    def add(case, t, flops, byts):
        rows.append({"case": case, "us": round(t * 1e6, 1), "tflops": round(flops / t / 1e12, 1), "gbs": round(byts / t / 1e9, 0)})

    # config 2: dense sweep
    for m in (16, 64, 128, 4096):                      # (16: a decode batch, beside the three row counts of config 2)
        for i, (n, k) in enumerate(DENSE_NK):
            c = make_dense_case(m, n, k, 77 + i, torch, dg)
            t = bench(lambda: dg.fp8_gemm_nt(c["a"], c["b"], c["d"], recipe=(1, 1, 128)), 3, 10)
            add(f"dense m{m} n{n} k{k}", t, flops_of(m, n, k), m * k + n * k + m * n * 2 + (m + n) * (k // 128))
    # the library yardstick the reference's tests print beside their kernel (tests/test_fp8_fp4.py:102-107): cuBLASLt FP8
    # with one scale per tensor (a different, cheaper operation: no block scales), same method, same flush
    for n, k in DENSE_NK:
        try:
            x8 = torch.randn((M_DENSE, k), device="cuda").to(torch.float8_e4m3fn)
            w8 = torch.randn((n, k), device="cuda").to(torch.float8_e4m3fn)
            one = torch.ones((), device="cuda")
            lib_call = lambda: torch._scaled_mm(x8, w8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            for _ in range(3):
                lib_call()
            t = bench_kineto(lib_call, ("nvjet", "gemm", "cutlass", "sm100", "sm90"), 10)
            add(f"torch._scaled_mm (cuBLASLt, per-tensor scales) fp8 m{M_DENSE} n{n} k{k}", t, flops_of(M_DENSE, n, k), M_DENSE * k + n * k + M_DENSE * n * 2)
            del x8, w8
        except Exception as exc:                        # the yardstick is optional: a torch build without it must not stop the run
            rows.append({"case": f"torch._scaled_mm fp8 m{M_DENSE} n{n} k{k}", "error": repr(exc)[:120]})
    # the step before the GEMM: per-token cast of BF16 activations straight to the packed scale layout (HBM-bound)
    for m, k in ((4096, 7168), (32768, 7168)):
        x = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
        t = bench_kineto(lambda: dg.per_token_cast(x, "e4m3", 128), "per_token_cast_kernel", 10)
        rows.append({"case": f"per-token cast bf16->e4m3 + packed UE8M0 m{m} k{k}", "us": round(t * 1e6, 1), "tflops": 0.0,
                     "gbs": round((m * k * 3 + m * k // 128) / t / 1e9, 0)})
        del x
    # config 5 (dense): FP8 x FP4
    for n, k in ((7168, 2048), (4096, 7168)):
        a = torch.randn((M_DENSE, k), device="cuda", dtype=torch.bfloat16)
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
        qa, sfa = per_token_cast_to_fp8(a, True, 128)
        qb, sfb = per_token_cast_to_fp4(w, True, 32)
        sfa = dg.transform_sf_into_required_layout(sfa, M_DENSE, k, (1, 128))
        sfb = dg.transform_sf_into_required_layout(sfb, n, k, (1, 32))
        d = torch.empty((M_DENSE, n), device="cuda", dtype=torch.bfloat16)
        t = bench(lambda: dg.fp8_fp4_gemm_nt((qa, sfa), (qb, sfb), d, recipe_a=(1, 128), recipe_b=(1, 32)), 3, 10)
        add(f"fp8xfp4 dense m{M_DENSE} n{n} k{k}", t, flops_of(M_DENSE, n, k), M_DENSE * k + n * k // 2 + M_DENSE * n * 2)
        del a, w, qa, qb, d
    # FP4 x FP4 through kind::mxf4 (packed operands in shared memory, twice the FP8 tensor rate; nominal dense FP4 peak 9000 TFLOP/s)
    for n, k in ((7168, 2048), (4096, 7168), (7168, 16384)):
        a = torch.randn((M_DENSE, k), device="cuda", dtype=torch.bfloat16)
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
        qa, sfa = per_token_cast_to_fp4(a, True, 32)
        qb, sfb = per_token_cast_to_fp4(w, True, 32)
        sfa = dg.transform_sf_into_required_layout(sfa, M_DENSE, k, (1, 32))
        sfb = dg.transform_sf_into_required_layout(sfb, n, k, (1, 32))
        d = torch.empty((M_DENSE, n), device="cuda", dtype=torch.bfloat16)
        t = bench(lambda: dg.fp4_gemm_nt((qa, sfa), (qb, sfb), d, recipe_a=(1, 32), recipe_b=(1, 32)), 3, 10)
        add(f"fp4xfp4 (kind::mxf4) dense m{M_DENSE} n{n} k{k}", t, flops_of(M_DENSE, n, k), (M_DENSE + n) * k // 2 + M_DENSE * n * 2)
        del a, w, qa, qb, d
    # configs 3 and 5 (grouped): 32 experts, tokens per expert int(8192 U(0.7, 1.3)) aligned to 128
    rng = random.Random(0)
    groups = 32
    actual = [int(8192 * rng.uniform(0.7, 1.3)) for _ in range(groups)]
    valid = sum(actual)
    # (alignment 128: the configuration as written; 256: what get_theoretical_mk_alignment_for_contiguous_layout() recommends
    #  on sm_100 and what lets CTA pairs run: a pair multiplies 256 consecutive rows with one expert's weights)
    for alignment in (128, 256):
        aligned = [-(-x // alignment) * alignment for x in actual]
        m_total = sum(aligned)
        layout = torch.full((m_total,), -1, dtype=torch.int, device="cuda")
        start = 0
        for g, (am, al) in enumerate(zip(actual, aligned)):
            layout[start:start + am] = g
            start += al
        dg.set_mk_alignment_for_contiguous_layout(alignment)
        for n, k in ((4096, 7168), (7168, 2048)):
            a = torch.randn((m_total, k), device="cuda", dtype=torch.bfloat16)
            a[layout < 0] = 0
            qa, sfa = per_token_cast_to_fp8(a, True, 128)
            del a
            sfa = dg.transform_sf_into_required_layout(sfa, m_total, k, (1, 128))
            d = torch.empty((m_total, n), device="cuda", dtype=torch.bfloat16)
            for fp4 in ((False, True) if alignment == 128 else (False,)):
                qb, sfb = make_grouped_b(groups, n, k, fp4, torch, dg)
                rb = (1, 32) if fp4 else (1, 128)
                t = bench(lambda: dg.m_grouped_fp8_fp4_gemm_nt_contiguous((qa, sfa), (qb, sfb), d, layout, recipe_a=(1, 128), recipe_b=rb), 2, 5)
                add(f"{'fp8xfp4 ' if fp4 else ''}m-grouped contiguous G{groups}{'' if alignment == 128 else ' alignment 256'} M{m_total} (valid {valid}) n{n} k{k}", t,
                    flops_of(valid, n, k), m_total * k + groups * n * k // (2 if fp4 else 1) + m_total * n * 2)
                del qb, sfb
            del qa, sfa, d
    dg.set_mk_alignment_for_contiguous_layout(128)
    # config 4: masked decode GEMM replayed from a CUDA graph
    groups, max_m, n, k = 16, 256, 4096, 7168
    masked = torch.tensor([rng.randint(45, 83) for _ in range(groups)], dtype=torch.int, device="cuda")
    a = torch.randn((groups * max_m, k), device="cuda", dtype=torch.bfloat16)
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    qa, sfa = qa.view(groups, max_m, k), dg.transform_sf_into_required_layout(sfa.view(groups, max_m, -1), max_m, k, (1, 128), groups)
    qb, sfb = make_grouped_b(groups, n, k, False, torch, dg)
    d = torch.empty((groups, max_m, n), device="cuda", dtype=torch.bfloat16)
    call = lambda: dg.m_grouped_fp8_gemm_nt_masked((qa, sfa), (qb, sfb), d, masked, 64, recipe=(1, 1, 128))
    call()
    torch.cuda.synchronize()
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            call()
    t = bench(graph.replay, 3, 20)
    vm = int(masked.sum().item())
    add(f"m-grouped masked (CUDA graph) G{groups} max_m{max_m} valid {vm} n{n} k{k}", t, flops_of(vm, n, k),
        vm * k + groups * n * k + vm * n * 2)
    del qa, sfa, qb, sfb, d, a, graph
    # k-grouped contiguous (MoE weight gradients, tests/generators.py:251-254): FP32 D accumulated in place
    for g, m, n, k_per in ((4, 4096, 7168, 8192), (8, 7168, 2048, 4096)):
        ks = [k_per] * g
        ak = torch.randn((g * k_per, m), device="cuda").to(torch.float8_e4m3fn)
        bk = torch.randn((g * k_per, n), device="cuda").to(torch.float8_e4m3fn)
        lay = torch.tensor(ks, dtype=torch.int, device="cuda")
        sfak = torch.ones((g * k_per // 128, m), device="cuda")
        sfbk = torch.ones((g * k_per // 128, n), device="cuda")
        dk = torch.zeros((g, m, n), device="cuda")
        t = bench(lambda: dg.k_grouped_fp8_gemm_tn_contiguous((ak, sfak), (bk, sfbk), dk, ks, lay, c=dk, recipe=(1, 1, 128)), 2, 5)
        add(f"k-grouped contiguous G{g} m{m} n{n} k{k_per}/group fp32 accumulate", t, flops_of(m, n, g * k_per),
            g * k_per * (m + n) + 2 * g * m * n * 4)
        del ak, bk, sfak, sfbk, dk
    # batched GEMM behind fp8_einsum (tests/test_einsum.py:128-186): BF16 output and the quantised (e4m3, scales) pair
    b_, h, r, dd = 4096, 8, 4096, 1024
    x = torch.randn((b_ * h, r), device="cuda", dtype=torch.bfloat16)
    qx, sfx = per_token_cast_to_fp8(x, True, 128)
    qx, sfx = qx.view(b_, h, r), sfx.view(b_, h, r // 128)
    qy, sfy = make_grouped_b(h, dd, r, False, torch, dg)
    z = torch.empty((b_, h, dd), device="cuda", dtype=torch.bfloat16)
    t = bench(lambda: dg.fp8_einsum("bhr,hdr->bhd", (qx, sfx), (qy, sfy), z, recipe=(1, 1, 128)), 2, 8)
    add(f"fp8_einsum bhr,hdr->bhd b{b_} h{h} r{r} d{dd} bf16 out", t, flops_of(b_ * h, dd, r), b_ * h * r + h * dd * r + b_ * h * dd * 2)
    zq = torch.empty((b_, h, dd), device="cuda", dtype=torch.float8_e4m3fn)
    sfd = torch.empty((h * dd // 128, b_), device="cuda", dtype=torch.int).t()
    t = bench(lambda: dg.fp8_einsum("bhr,hdr->bhd", (qx, sfx), (qy, sfy), (zq, sfd), recipe=(1, 1, 128)), 2, 8)
    add(f"fp8_einsum bhr,hdr->bhd b{b_} h{h} r{r} d{dd} quantised (e4m3 + 1x32 scales) out", t, flops_of(b_ * h, dd, r),
        b_ * h * r + h * dd * r + b_ * h * dd)
    del x, qx, sfx, qy, sfy, z, zq, sfd
    # BF16 operands (the same kernel, kind::f16), with torch.matmul (cuBLAS) timed beside it
    for n, k in ((4096, 7168), (7168, 2048)):
        a16 = torch.randn((M_DENSE, k), device="cuda", dtype=torch.bfloat16)
        b16 = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
        d16 = torch.empty((M_DENSE, n), device="cuda", dtype=torch.bfloat16)
        t = bench(lambda: dg.bf16_gemm_nt(a16, b16, d16), 3, 10)
        add(f"bf16 dense m{M_DENSE} n{n} k{k}", t, flops_of(M_DENSE, n, k), 2 * (M_DENSE * k + n * k + M_DENSE * n))
        for _ in range(3):
            torch.matmul(a16, b16.t(), out=d16)
        t = bench_kineto(lambda: torch.matmul(a16, b16.t(), out=d16), ("nvjet", "gemm", "cutlass", "sm100", "sm90"), 10)
        add(f"torch.matmul (cuBLAS) bf16 m{M_DENSE} n{n} k{k}", t, flops_of(M_DENSE, n, k), 2 * (M_DENSE * k + n * k + M_DENSE * n))
        del a16, b16, d16
    # einsum 'bmk,bnk->mn' (tests/test_einsum.py:21-41): a BF16 GEMM reduced over the batch as well
    for s_, m_, n_, k_ in ((4096, 256, 256, 256), (8192, 384, 128, 384)):
        ab, bb = torch.randn((s_, m_, k_), device="cuda", dtype=torch.bfloat16), torch.randn((s_, n_, k_), device="cuda", dtype=torch.bfloat16)
        acc = torch.zeros((m_, n_), device="cuda", dtype=torch.float)
        t = bench(lambda: dg.einsum("bmk,bnk->mn", ab, bb, acc, c=acc), 2, 8)
        add(f"bf16 einsum bmk,bnk->mn b{s_} m{m_} n{n_} k{k_} fp32 accumulate", t, flops_of(m_, n_, s_ * k_), 2 * s_ * (m_ + n_) * k_ + m_ * n_ * 4)
        del ab, bb, acc
    return rows


def sustained_rows(torch, dg, device_index, num_sms, seconds=1.5, dense_only=False, with_library=True):
    """The M = 4096 dense shapes and the two config-3 grouped shapes, each run back to back for ~`seconds` (CUDA graph of
    20 launches replayed), with the SM clock and board power sampled meanwhile: time, TFLOP/s, median MHz, median W,
    thousands of SM cycles per launch (time x clock) and the fraction of the FP8 tensor rate at that clock.  The library
    yardstick (torch._scaled_mm, cuBLASLt FP8 with per-tensor scales) runs in the same loop.  This is the regime a
    long-running job sees: clocks settle under the board's power limit within the first tenths of a second."""
    rows = []

    def run(label, fn, flops):
        try:
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(5):
                fn()
            e1.record()
            torch.cuda.synchronize()
            per = e0.elapsed_time(e1) / 5 / 1e3
            graph, stream, per_graph = torch.cuda.CUDAGraph(), torch.cuda.Stream(), 20
            with torch.cuda.stream(stream):
                with torch.cuda.graph(graph, stream=stream):
                    for _ in range(per_graph):
                        fn()
            reps = max(1, int(seconds / (per * per_graph)))
            torch.cuda.synchronize()
            with ClockSampler(device_index, 0.005) as smp:
                e0.record()
                for _ in range(reps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / 1e3 / (reps * per_graph)
            c = smp.summary()
            mhz = c["sm_mhz"] or 0
            peak = FP8_FLOP_PER_CLK_PER_SM * num_sms * mhz * 1e6 / 1e12
            rows.append({"case": label, "us": round(t * 1e6, 1), "tflops": round(flops / t / 1e12, 1), "sm_mhz": mhz,
                         "power_w": c["power_w"], "kcycles": round(t * mhz * 1e3, 1), "reasons": c["reasons"],
                         "frac_clock_adjusted": round(flops / t / 1e12 / peak, 3) if peak else None,
                         "frac_of_nominal": round(flops / t / 1e12 / NOMINAL_FP8_TFLOPS, 3)})
            del graph
        except Exception as exc:
            rows.append({"case": label, "error": repr(exc)[:160]})

    for i, (n, k) in enumerate(DENSE_NK):
        c = make_dense_case(M_DENSE, n, k, 300 + i, torch, dg)
        cfg = dg.get_gemm_config(0, M_DENSE, n, k)
        tile = f"{cfg['block_m'] * cfg['cluster_size']}x{cfg['block_n']} per {'CTA pair' if cfg['cluster_size'] == 2 else 'CTA'}"
        run(f"dense m{M_DENSE} n{n} k{k} [{tile}, {cfg['num_stages']} stages]",
            lambda: dg.fp8_gemm_nt(c["a"], c["b"], c["d"], recipe=(1, 1, 128)), flops_of(M_DENSE, n, k))
        x8, w8, one = c["a"][0], c["b"][0], torch.ones((), device="cuda")
        if with_library:
            run(f"torch._scaled_mm (cuBLASLt, per-tensor scales) m{M_DENSE} n{n} k{k}",
                lambda: torch._scaled_mm(x8, w8.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16), flops_of(M_DENSE, n, k))
        del c, x8, w8
    if dense_only:
        return rows
    actual, aligned = grouped_layout()
    for n, k in GROUPED_NK:
        sh = make_contiguous_shard(n, k, (0, 32), actual, aligned, torch, dg)
        run(f"m-grouped contiguous G32 rows {sum(aligned)} (valid {sum(actual)}) n{n} k{k}",
            lambda: dg.m_grouped_fp8_gemm_nt_contiguous(sh["a"], sh["b"], sh["d"], sh["layout"], recipe=(1, 1, 128)),
            flops_of(sum(actual), n, k))
        del sh
        torch.cuda.empty_cache()
    return rows


if __name__ == "__main__":
    main()

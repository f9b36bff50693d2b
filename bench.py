#!/usr/bin/env python
"""Benchmark of the block-scaled FP8 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--detail]

A *step* is one pass over the six DeepSeek-V3-shaped dense FP8 GEMMs with M = 4096 that the benchmark specification's
metric is quoted on (its config 2): D[M,N] = A[M,K] @ B[N,K]^T, A quantised per token per 128 of K, B per
128 x 128 block, UE8M0 scales pre-packed, BF16 output, synthetic N(0,1) data.  `value` is the aggregate
TFLOP/s (2 M N K over the six shapes / device time) with operands resident in HBM; `e2e` is the same pass
through the public Python API with host buffers (pinned host -> device copies of A, SFA, B, SFB and a
device -> host read of D inside the timed region).  With N > 1 (torchrun) every rank runs the same
per-GPU workload on its own shard-shaped data (column-parallel shards of an N-times wider problem) and no
collective runs in the timed region: weak scaling, value = sum over ranks.

`--impl reference` times the reference path's CPU implementation (the numpy port of its torch
dequantise-then-matmul, oracle/) on the host cores on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

M_DENSE = 4096
DENSE_NK = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]
NOMINAL_FP8_TFLOPS = 4500.0
CPU_SAMPLE_NK = (2112, 7168)          # the bounded sample the CPU arm times (1 of the 6 shapes)
# dram__bytes_read.sum + dram__bytes_write.sum per launch of dg_gemm_fp8_fp4 at M = 4096, from one ncu capture of this
# script (profiles/dg_gemm_fp8_fp4_dense_m4096.md); D written late in a launch may still sit in L2 when it ends.
NCU_DRAM_BYTES = {(2112, 7168): 46332928, (24576, 1536): 231155456, (32768, 512): 247204352,
                  (7168, 16384): 461400576, (4096, 7168): 62027264, (7168, 2048): 31307264}


def flops_of(m, n, k):
    return 2.0 * m * n * k


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_burst": p["bf16_tflops"], "bf16_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------------
# Clock sampling during the timed region (NVML reads only)
# ----------------------------------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index: int, period_s: float = 0.002):
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
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
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# ----------------------------------------------------------------------------------------------------
# CPU arm: the reference path's dequantise-then-matmul on the host cores (numpy port in oracle/)
# ----------------------------------------------------------------------------------------------------
def cpu_sample_inputs(seed=0):
    import numpy as np
    import oracle
    n, k = CPU_SAMPLE_NK
    rng = np.random.default_rng(seed)
    a = oracle.bf16_round(rng.standard_normal((M_DENSE, k)).astype(np.float32))
    b = oracle.bf16_round(rng.standard_normal((n, k)).astype(np.float32))
    qa, sfa = oracle.per_token_cast_to_fp8(a, True, 128)
    qb, sfb = oracle.per_block_cast_to_fp8(b, True)
    return qa, sfa, qb, oracle.broadcast_sf_along_mn(sfb, n, 128)


def cpu_step(inputs):
    import oracle
    qa, sfa, qb, sfb = inputs
    return oracle.bf16_round(oracle.dequant_gemm_nt(qa, sfa, qb, sfb))


_CPU_THREADS_USED = None


def cpu_threads():
    if _CPU_THREADS_USED is not None:
        return _CPU_THREADS_USED
    try:
        from threadpoolctl import threadpool_info
        blas = [p["num_threads"] for p in threadpool_info() if p.get("user_api") == "blas"]
        if blas:
            return max(blas)
    except Exception:
        pass
    return os.cpu_count() or 1


def time_cpu(steps, warmup):
    import numpy  # noqa: F401  (make sure BLAS is loaded before counting threads)
    inputs = cpu_sample_inputs()
    # Use every host core this process may run on (torchrun exports OMP_NUM_THREADS=1 for its workers)
    try:
        ncpu = len(os.sched_getaffinity(0))
    except AttributeError:
        ncpu = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits
        limiter = threadpool_limits(limits=ncpu)
    except Exception:
        limiter = None
    for _ in range(warmup):
        cpu_step(inputs)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(inputs)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    global _CPU_THREADS_USED
    _CPU_THREADS_USED = cpu_threads()
    if limiter is not None:
        limiter.restore_original_limits()
    n, k = CPU_SAMPLE_NK
    return flops_of(M_DENSE, n, k) / dt / 1e12, dt


def run_reference_arm(args, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 8))           # bounded: each CPU step is ~0.5-3 s
    warm = max(1, min(args.warmup, 2))
    tflops, dt = time_cpu(steps, warm)
    n, k = CPU_SAMPLE_NK
    sample = f"M={M_DENSE},N={n},K={k} (1 of the 6 dense shapes), dequantise + FP32 matmul, {steps} steps"
    line = {
        "impl": "reference", "metric": "dense_fp8_gemm_tflops", "value": round(tflops, 4), "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warm, "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "dense_fp8_gemm_nt_m4096 (config 2), bounded sample", "sample": sample},
        "cpu_baseline": {"value": round(tflops, 4), "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": round(tflops, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------
def make_dense_case(m, n, k, seed, torch, dg):
    from deepgemm_amd_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp8
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16, generator=g)
    b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=g)
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    qb, sfb = per_block_cast_to_fp8(b, True)
    sfa = dg.transform_sf_into_required_layout(sfa, m, k, (1, 128))
    sfb = dg.transform_sf_into_required_layout(sfb, n, k, (128, 128))
    d = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    return {"m": m, "n": n, "k": k, "a": (qa, sfa), "b": (qb, sfb), "d": d}


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--detail", action="store_true", help="also time each shape of configs 2-5 on its own (rank 0)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--pdl", action="store_true", help="launch the GEMMs with programmatic dependent launch (set_pdl)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    ap.add_argument("--shapes", default="", help="comma-separated NxK subset of the six dense shapes (profiling runs)")
    ap.add_argument("--m", type=int, default=M_DENSE, help="rows of A (profiling runs of the M = 64 / 128 shapes; the metric is quoted at 4096)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist
    import deepgemm_amd_b200 as dg
    from deepgemm_amd_b200.dist import init_dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the GEMM path has no CPU fallback (use --impl reference for the CPU arm)")
    rank, world, local_rank = init_dist()
    torch.cuda.set_device(local_rank)

    def barrier():
        if world > 1:
            dist.barrier()

    nk_list = DENSE_NK
    if args.shapes:
        nk_list = [tuple(int(v) for v in s.split("x")) for s in args.shapes.split(",")]
    cases = [make_dense_case(args.m, n, k, 1000 * rank + i, torch, dg) for i, (n, k) in enumerate(nk_list)]
    step_flops = sum(flops_of(c["m"], c["n"], c["k"]) for c in cases)

    def step():
        for c in cases:
            dg.fp8_gemm_nt(c["a"], c["b"], c["d"], recipe=(1, 1, 128))

    # The library's launch option (the reference's set_pdl): a GEMM's set-up overlaps the tail of the one before.
    # Off by default, as in the library: on this step it measured 2 % slower.
    dg.set_pdl(args.pdl)
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if dg.kernel_status() != 0:
        raise SystemExit(f"kernel reported status {dg.kernel_status():#x}")

    barrier()                      # first collective initialises NCCL: keep that out of the sampled region
    with ClockSampler(local_rank) as clocks:
        dt = time_events(step, args.steps, torch, barrier)
    t = torch.tensor([dt], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dt_max = float(t.item())
    value = world * step_flops * args.steps / dt_max / 1e12

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
    # tensor cores work at the same time; every stream is joined back into the current one at the end of a step, where
    # the timing events are recorded.  A case's inputs are not overwritten before its previous GEMM has read them, nor
    # its D before the previous read-back has finished.
    s_in, s_mm, s_out = (torch.cuda.Stream() for _ in range(3))
    ev_in = [torch.cuda.Event() for _ in cases]
    ev_mm = [torch.cuda.Event() for _ in cases]
    ev_out = [torch.cuda.Event() for _ in cases]

    def e2e_step():
        cur = torch.cuda.current_stream()
        for s_ in (s_in, s_mm, s_out):
            s_.wait_stream(cur)
        for i, (c, hs, fs) in enumerate(zip(cases, host, dev_flat)):
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_mm[i])                 # the previous step's GEMM of this case has consumed the inputs
                for h, f in zip(hs[:-1], fs):
                    f.copy_(h, non_blocking=True)
                ev_in[i].record(s_in)
            with torch.cuda.stream(s_mm):
                s_mm.wait_event(ev_in[i])
                s_mm.wait_event(ev_out[i])                # the previous step's read-back of this D is complete
                dg.fp8_gemm_nt(c["a"], c["b"], c["d"], recipe=(1, 1, 128))
                ev_mm[i].record(s_mm)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_mm[i])
                hs[-1].copy_(c["d"], non_blocking=True)
                ev_out[i].record(s_out)
        for s_ in (s_in, s_mm, s_out):
            cur.wait_stream(s_)

    e2e_steps = max(1, min(args.steps, 10))
    e2e_value = None
    if not args.no_e2e:
        e2e_step()
        e2e_dt = time_events(e2e_step, e2e_steps, torch, barrier)
        te = torch.tensor([e2e_dt], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_value = world * step_flops * e2e_steps / float(te.item()) / 1e12

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peaks = load_peaks()
    clk = clocks.summary()
    per_gpu = value / world
    # The dominant (only) kernel of the step is the tcgen05 GEMM; FP8 runs at twice the BF16 tensor rate, so the
    # measured denominator is 2 x the cuBLAS BF16 figure (sustained: the kernel is timed inside a long loop).
    peak_fp8 = 2.0 * peaks["bf16_sustained"]
    known = [NCU_DRAM_BYTES.get((c["n"], c["k"])) for c in cases]
    traffic = None if any(v is None for v in known) else round(sum(known) / len(known))
    algorithmic = sum(c["m"] * c["k"] + c["n"] * c["k"] + c["m"] * c["n"] * 2 + (c["m"] + c["n"]) * (c["k"] // 128) for c in cases) / len(cases)
    line = {
        "metric": "dense_fp8_gemm_tflops", "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt_max / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 (fp32 accumulate, bf16 out)",
        "data": "synthetic",
        "config": {"workload": "dense_fp8_gemm_nt_m4096 (BASELINE config 2, the six (N,K) at M=4096)" if args.m == M_DENSE and not args.shapes
                               else f"profiling subset: M={args.m}, {len(nk_list)} of the dense shapes",
                   "shapes_mnk": [[c["m"], c["n"], c["k"]] for c in cases],
                   "scales": "UE8M0 packed int32, A 1x128, B 128x128 pre-broadcast",
                   "pdl": args.pdl,
                   "l2": "no flush: one step streams 1.0 GB through six different shapes, 8x the 126 MB L2",
                   "parallelism": f"replicated shards x{world}, no collective in the timed region"},
        "pct_of_nominal_fp8_peak": round(100.0 * per_gpu / NOMINAL_FP8_TFLOPS, 2),
        "roofline": {"bound": "tensor", "achieved": round(per_gpu, 2), "peak": round(peak_fp8, 1), "unit": "TFLOP/s",
                     "frac": round(per_gpu / peak_fp8, 4), "traffic": traffic, "traffic_unit": "bytes per launch (mean of the step's launches)",
                     "algorithmic_bytes_per_launch": round(algorithmic),
                     "peak_source": f"2 x bf16_tflops_sustained of MEASURED_PEAKS.json ({peaks['source']}); nominal FP8 dense 4500",
                     "frac_of_nominal": round(per_gpu / NOMINAL_FP8_TFLOPS, 4)},
        "clocks": clk,
        "e2e": {"value": None if e2e_value is None else round(e2e_value, 3), "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_steps, "overlap": "copies in, GEMMs and copies out on three streams chained by events"},
        "gpu_launches": args.steps * len(cases),
    }
    if world == 1 and not args.no_cpu_baseline:
        tflops, cdt = time_cpu(2, 1)
        n, k = CPU_SAMPLE_NK
        line["cpu_baseline"] = {"value": round(tflops, 4), "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
                                "sample": f"M={M_DENSE},N={n},K={k} (1 of the 6 shapes), 2 steps of {cdt:.2f} s"}
    if args.detail:
        line["detail"] = detail_rows(torch, dg)
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
    # configs 3 and 5 (grouped): 32 experts, tokens per expert int(8192 U(0.7, 1.3)) aligned to 128
    rng = random.Random(0)
    groups = 32
    actual = [int(8192 * rng.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [-(-x // 128) * 128 for x in actual]
    m_total, valid = sum(aligned), sum(actual)
    layout = torch.full((m_total,), -1, dtype=torch.int, device="cuda")
    start = 0
    for g, (am, al) in enumerate(zip(actual, aligned)):
        layout[start:start + am] = g
        start += al
    for n, k in ((4096, 7168), (7168, 2048)):
        a = torch.randn((m_total, k), device="cuda", dtype=torch.bfloat16)
        a[layout < 0] = 0
        qa, sfa = per_token_cast_to_fp8(a, True, 128)
        del a
        sfa = dg.transform_sf_into_required_layout(sfa, m_total, k, (1, 128))
        d = torch.empty((m_total, n), device="cuda", dtype=torch.bfloat16)
        for fp4 in (False, True):
            qb, sfb = make_grouped_b(groups, n, k, fp4, torch, dg)
            rb = (1, 32) if fp4 else (1, 128)
            t = bench(lambda: dg.m_grouped_fp8_fp4_gemm_nt_contiguous((qa, sfa), (qb, sfb), d, layout, recipe_a=(1, 128), recipe_b=rb), 2, 5)
            add(f"{'fp8xfp4 ' if fp4 else ''}m-grouped contiguous G{groups} M{m_total} (valid {valid}) n{n} k{k}", t,
                flops_of(valid, n, k), m_total * k + groups * n * k // (2 if fp4 else 1) + m_total * n * 2)
            del qb, sfb
        del qa, sfa, d
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


if __name__ == "__main__":
    main()

#!/usr/bin/env python
"""Runs the UNMODIFIED reference (DeepGEMM 2.8.1, installed by baseline/build_ref.py into baseline/_ref) on one GPU:
its own sm_100 kernel `sm100_fp8_fp4_gemm_1d1d_impl` through its own Python API, heuristics, tensor maps and launcher,
for the shapes of the benchmark configurations, timed the way this repository's kernels are timed.

    python baseline/reference_arm.py --stage layout|small|dense|grouped|all [--out rows.json] [--sustained]
    python baseline/reference_arm.py --stage probe [--m 4096]     # three plain calls per dense shape, for a profiler

Stages go from harmless to heavy so that a first run on a new machine can stop early:
  layout   only the reference's scale-packing kernel (plain CUDA, no TMA, no barriers), compared bit for bit with this
           repository's packer: proves the stand-in JIT compiles, loads, passes arguments and launches correctly;
  small    one 128 x 256 x 512 GEMM compared with the dequantise-then-matmul value;
  dense    the six M = 4096 shapes of config 2 (+ M = 64 / 128), burst timing (the reference's own bench_kineto: torch
           profiler kernel time, L2 flushed before every call) and, with --sustained, a back-to-back loop with clocks;
  grouped  config 3 (32 experts, both shapes, alignment 128 and the reference's recommended 256) and config 4.

The reference package is imported under the name `deep_gemm_reference` (this repository already provides a module
called `deep_gemm`).  Its JIT cache goes to baseline/_ref/jit_cache.  Prints one JSON object; nothing here is product
code and nothing in the product imports it.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import random
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF_PKG = os.path.join(HERE, "_ref", "deep_gemm")
DENSE_NK = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]


def load_reference():
    if not os.path.isfile(os.path.join(REF_PKG, "__init__.py")):
        raise SystemExit(json.dumps({"unavailable": "baseline/_ref holds no reference installation (run baseline/build_ref.py where the reference's source tree is mounted)"}))
    os.environ.setdefault("DG_JIT_CACHE_DIR", os.path.join(HERE, "_ref", "jit_cache"))
    spec = importlib.util.spec_from_file_location("deep_gemm_reference", os.path.join(REF_PKG, "__init__.py"),
                                                  submodule_search_locations=[REF_PKG])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["deep_gemm_reference"] = mod
    spec.loader.exec_module(mod)
    return mod


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def calc_diff(x, y):
    x, y = x.double(), y.double()
    return float(1 - 2 * (x * y).sum() / (x * x + y * y).sum())


def dequant_ref(ref, qa, sfa, qb, sfb_block, torch):
    n, k = qb.shape
    a_deq = ref.utils.cast_back_from_fp8(qa, sfa).bfloat16()
    rows = torch.arange(n, device="cuda") // 128
    cols = torch.arange(k, device="cuda") // 128
    b_deq = (qb.float() * sfb_block[rows][:, cols]).bfloat16()
    return (a_deq @ b_deq.t()).float()


def make_dense(ref, m, n, k, seed, torch):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16, generator=g)
    b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=g)
    qa, sfa = ref.utils.per_token_cast_to_fp8(a, use_ue8m0=True, gran_k=128)
    qb, sfb = ref.utils.per_block_cast_to_fp8(b, use_ue8m0=True)
    psfa = ref.transform_sf_into_required_layout(sfa, m, k, (1, 128))
    psfb = ref.transform_sf_into_required_layout(sfb, n, k, (128, 128))
    d = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    return {"qa": qa, "sfa": sfa, "qb": qb, "sfb": sfb, "psfa": psfa, "psfb": psfb, "d": d}


def stage_layout(ref, torch, out):
    """The scale-packing kernel of the reference against this repository's, bit for bit (values and strides)."""
    sys.path.insert(0, ROOT)
    import deepgemm_amd_b200 as ours
    ok = True
    for mn, k, groups in ((4096, 7168, 1), (4097, 7296, 2), (128, 512, 1)):
        shape = (groups, mn, -(-k // 128)) if groups > 1 else (mn, -(-k // 128))
        exps = torch.randint(100, 140, shape, device="cuda", dtype=torch.int32)
        sf = (exps << 23).view(torch.float32)
        theirs = ref.transform_sf_into_required_layout(sf, mn, k, (1, 128), groups if groups > 1 else None)
        mine = ours.transform_sf_into_required_layout(sf, mn, k, (1, 128), groups if groups > 1 else None)
        torch.cuda.synchronize()
        same = theirs.shape == mine.shape and theirs.stride() == mine.stride() and bool(torch.equal(theirs, mine))
        log(f"layout mn={mn} k={k} groups={groups}: shape {tuple(theirs.shape)} stride {theirs.stride()} equal={same}")
        ok = ok and same
    out["layout_kernel_bitwise_equal_to_ours"] = ok
    return ok


def stage_small(ref, torch, out):
    m, n, k = 128, 256, 512
    c = make_dense(ref, m, n, k, 1, torch)
    log("launching the reference GEMM 128 x 256 x 512 ...")
    ref.fp8_gemm_nt((c["qa"], c["psfa"]), (c["qb"], c["psfb"]), c["d"], recipe=(1, 1, 128))
    torch.cuda.synchronize()
    diff = calc_diff(c["d"], dequant_ref(ref, c["qa"], c["sfa"], c["qb"], c["sfb"], torch))
    log(f"small GEMM calc_diff vs dequantised matmul: {diff:.3e}")
    out["small_gemm_calc_diff"] = diff
    return diff < 1e-3


def sustained(fn, flops, torch, seconds=1.5):
    from bench import ClockSampler, FP8_FLOP_PER_CLK_PER_SM
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
    with ClockSampler(torch.cuda.current_device(), 0.005) as smp:
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
    t = e0.elapsed_time(e1) / 1e3 / (reps * per_graph)
    c = smp.summary()
    mhz = c["sm_mhz"] or 0
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    peak = FP8_FLOP_PER_CLK_PER_SM * sms * mhz * 1e6 / 1e12
    return {"sustained_us": round(t * 1e6, 1), "sustained_tflops": round(flops / t / 1e12, 1), "sm_mhz": mhz, "power_w": c["power_w"],
            "kcycles": round(t * mhz * 1e3, 1), "frac_clock_adjusted": round(flops / t / 1e12 / peak, 3) if peak else None}


def stage_dense(ref, torch, out, with_sustained, ms):
    sys.path.insert(0, ROOT)
    import deepgemm_amd_b200 as ours
    rows = []
    for m in ms:
        for i, (n, k) in enumerate(DENSE_NK):
            c = make_dense(ref, m, n, k, 77 + i, torch)
            call = lambda: ref.fp8_gemm_nt((c["qa"], c["psfa"]), (c["qb"], c["psfb"]), c["d"], recipe=(1, 1, 128))
            t0 = time.time()
            call()
            torch.cuda.synchronize()
            first = time.time() - t0
            mine = torch.empty_like(c["d"])
            ours.fp8_gemm_nt((c["qa"], c["psfa"]), (c["qb"], c["psfb"]), mine, recipe=(1, 1, 128))
            torch.cuda.synchronize()
            row = {"case": f"dense m{m} n{n} k{k}", "first_call_s": round(first, 1),
                   "calc_diff_vs_dequantised_matmul": calc_diff(c["d"], dequant_ref(ref, c["qa"], c["sfa"], c["qb"], c["sfb"], torch)),
                   "bitwise_equal_to_this_repository": bool(torch.equal(c["d"].view(torch.int16), mine.view(torch.int16)))}
            t = ref.testing.bench_kineto(call, "gemm_", suppress_kineto_output=True)
            flops = 2.0 * m * n * k
            row.update({"us": round(t * 1e6, 1), "tflops": round(flops / t / 1e12, 1)})
            if with_sustained and m == 4096:
                row.update(sustained(call, flops, torch))
            log(row)
            rows.append(row)
            del c
    out["dense"] = rows


def stage_probe(ref, torch, out, ms):
    """Three plain calls of the reference's GEMM per dense shape and nothing else on the GPU in between: what a
    counter capture of its kernel (one launch per shape) runs."""
    for m in ms:
        for i, (n, k) in enumerate(DENSE_NK):
            c = make_dense(ref, m, n, k, 77 + i, torch)
            for _ in range(3):
                ref.fp8_gemm_nt((c["qa"], c["psfa"]), (c["qb"], c["psfb"]), c["d"], recipe=(1, 1, 128))
            torch.cuda.synchronize()
            del c
    out["probe"] = {"calls_per_shape": 3, "m": ms, "shapes_nk": [list(x) for x in DENSE_NK]}


def stage_grouped(ref, torch, out, with_sustained):
    rows = []
    rng = random.Random(0)
    groups = 32
    actual = [int(8192 * rng.uniform(0.7, 1.3)) for _ in range(groups)]
    for alignment in (128, 256):
        aligned = [-(-x // alignment) * alignment for x in actual]
        m_total = sum(aligned)
        layout = torch.full((m_total,), -1, dtype=torch.int, device="cuda")
        start = 0
        for g, (am, al) in enumerate(zip(actual, aligned)):
            layout[start:start + am] = g
            start += al
        ref._C.set_mk_alignment_for_contiguous_layout(alignment)
        for n, k in ((4096, 7168), (7168, 2048)):
            a = torch.randn((m_total, k), device="cuda", dtype=torch.bfloat16)
            a[layout < 0] = 0
            qa, sfa = ref.utils.per_token_cast_to_fp8(a, use_ue8m0=True, gran_k=128)
            del a
            psfa = ref.transform_sf_into_required_layout(sfa, m_total, k, (1, 128))
            qbs, sfbs = [], []
            for g in range(groups):
                w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
                q, s = ref.utils.per_block_cast_to_fp8(w, use_ue8m0=True)
                qbs.append(q)
                sfbs.append(s)
            qb, sfb = torch.stack(qbs), torch.stack(sfbs)
            psfb = ref.transform_sf_into_required_layout(sfb, n, k, (128, 128), groups)
            d = torch.empty((m_total, n), device="cuda", dtype=torch.bfloat16)
            call = lambda: ref.m_grouped_fp8_gemm_nt_contiguous((qa, psfa), (qb, psfb), d, layout, recipe=(1, 1, 128))
            call()
            torch.cuda.synchronize()
            g0 = groups - 1
            r0 = sum(aligned[:g0])
            diff = calc_diff(d[r0:r0 + actual[g0]], dequant_ref(ref, qa[r0:r0 + actual[g0]], sfa[r0:r0 + actual[g0]], qb[g0], sfb[g0], torch))
            t = ref.testing.bench_kineto(call, "gemm_", suppress_kineto_output=True, num_tests=5)
            flops = 2.0 * sum(actual) * n * k
            row = {"case": f"m-grouped contiguous G32 alignment {alignment} rows {m_total} (valid {sum(actual)}) n{n} k{k}",
                   "us": round(t * 1e6, 1), "tflops": round(flops / t / 1e12, 1), "calc_diff_last_expert": diff}
            if with_sustained:
                row.update(sustained(call, flops, torch))
            log(row)
            rows.append(row)
            del qa, sfa, psfa, qb, sfb, psfb, d
            torch.cuda.empty_cache()
    ref._C.set_mk_alignment_for_contiguous_layout(128)
    # config 4: masked decode GEMM in a CUDA graph
    groups, max_m, n, k = 16, 256, 4096, 7168
    masked = torch.tensor([rng.randint(45, 83) for _ in range(groups)], dtype=torch.int, device="cuda")
    a = torch.randn((groups * max_m, k), device="cuda", dtype=torch.bfloat16)
    qa, sfa = ref.utils.per_token_cast_to_fp8(a, use_ue8m0=True, gran_k=128)
    qa = qa.view(groups, max_m, k)
    psfa = ref.transform_sf_into_required_layout(sfa.view(groups, max_m, -1), max_m, k, (1, 128), groups)
    qbs, sfbs = [], []
    for g in range(groups):
        q, s = ref.utils.per_block_cast_to_fp8(torch.randn((n, k), device="cuda", dtype=torch.bfloat16), use_ue8m0=True)
        qbs.append(q)
        sfbs.append(s)
    qb = torch.stack(qbs)
    psfb = ref.transform_sf_into_required_layout(torch.stack(sfbs), n, k, (128, 128), groups)
    d = torch.empty((groups, max_m, n), device="cuda", dtype=torch.bfloat16)
    call = lambda: ref.m_grouped_fp8_gemm_nt_masked((qa, psfa), (qb, psfb), d, masked, 64, recipe=(1, 1, 128))
    call()
    torch.cuda.synchronize()
    graph, stream = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            call()
    t = ref.testing.bench_kineto(graph.replay, "gemm_", suppress_kineto_output=True)
    vm = int(masked.sum().item())
    rows.append({"case": f"m-grouped masked (CUDA graph) G{groups} max_m{max_m} valid {vm} n{n} k{k}", "us": round(t * 1e6, 1),
                 "tflops": round(2.0 * vm * n * k / t / 1e12, 1), "gbs": round((vm * k + groups * n * k + vm * n * 2) / t / 1e9)})
    log(rows[-1])
    out["grouped"] = rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--stage", default="all", choices=["layout", "small", "dense", "grouped", "all", "probe"])
    ap.add_argument("--sustained", action="store_true")
    ap.add_argument("--m", default="4096", help="comma-separated row counts of the dense stage")
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    import torch
    if not torch.cuda.is_available():
        raise SystemExit(json.dumps({"unavailable": "no CUDA device"}))
    ref = load_reference()
    out = {"reference_version": ref.__version__, "jit": "stand-in for the un-vendored DeepJIT (baseline/deep_jit_standin)",
           "device": torch.cuda.get_device_name(0)}
    log("reference", ref.__version__, "loaded; num_sms", ref.get_num_sms())
    order = ["layout", "small", "dense", "grouped"]
    if args.stage == "probe":
        stage_probe(ref, torch, out, [int(v) for v in args.m.split(",")])
        out["ok"] = True
        print(json.dumps(out), flush=True)
        return
    upto = order if args.stage == "all" else order[:order.index(args.stage) + 1]
    ok = True
    if "layout" in upto:
        ok = stage_layout(ref, torch, out)
    if ok and "small" in upto:
        ok = stage_small(ref, torch, out)
    if ok and "dense" in upto:
        stage_dense(ref, torch, out, args.sustained, [int(v) for v in args.m.split(",")])
    if ok and "grouped" in upto:
        stage_grouped(ref, torch, out, args.sustained)
    out["ok"] = ok
    text = json.dumps(out)
    if args.out:
        with open(args.out, "w") as f:
            f.write(text + "\n")
    print(text, flush=True)


if __name__ == "__main__":
    main()

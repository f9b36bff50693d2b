"""The allocation-free dense GEMM entry point (dg_fp8_fp4_gemm_noalloc), called through the C ABI.

Who needs it: code that is not allowed to allocate device memory when it calls the GEMM -- a latency-critical serving
thread that must never wait on the allocator, a process that hands out its whole memory budget at start-up and forbids
cudaMalloc afterwards, or a host application that owns all device memory itself.  The K-sliced GEMM path keeps its
FP32 partial panels in a fixed 16 MiB array inside the library image for these callers.  This file is collected last
on purpose, so that a run stopping at the first failure has already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from gpu_helpers import fp8_cuda, packed_sf_cuda, quantise_dense, seeded_bf16

pytestmark = pytest.mark.gpu

dg = pytest.importorskip("deepgemm_amd_b200")
from deepgemm_amd_b200 import _lib, api  # noqa: E402

FIXED_SCRATCH_BYTES = 16 << 20


def _args(qa, sfa, qb, sfb, d):
    a = (fp8_cuda(qa), packed_sf_cuda(sfa))
    b = (fp8_cuda(qb), packed_sf_cuda(sfb))
    m, k = qa.shape
    n = qb.shape[0]
    args = api._fill_args(a[0], a[1], b[0], b[1], d, m, n, k, 1, _lib.DG_MAJOR_K, _lib.DG_MAJOR_K, 128, 128)
    return args, (a, b)                     # keep the operand tensors alive while the kernels run


@pytest.mark.parametrize("m,n,k", [(128, 2112, 7168), (64, 4096, 7168), (256, 512, 512)])
def test_noalloc_entry_point_matches_the_allocating_one_on_two_calls_in_a_row(m, n, k):
    qa, sfa, qb, sfb, _ = quantise_dense(seeded_bf16((m, k), 60), seeded_bf16((n, k), 61))
    ref = oracle.dequant_gemm_nt(qa, sfa, qb, sfb)

    want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    args, keep = _args(qa, sfa, qb, sfb, want)
    _lib.check(_lib.lib.dg_fp8_fp4_gemm(C.byref(args)))              # the existing, allocating entry point
    torch.cuda.synchronize()
    assert oracle.calc_diff(want.float().cpu().numpy(), ref) < 1e-3

    for call in range(2):                                             # the array keeps the previous call's panels
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        args2, keep2 = _args(qa, sfa, qb, sfb, got)
        _lib.check(_lib.lib.dg_fp8_fp4_gemm_noalloc(C.byref(args2)))
        torch.cuda.synchronize()
        out = got.float().cpu().numpy()
        assert not np.isnan(out).any(), call
        assert oracle.calc_diff(out, want.float().cpu().numpy()) < 1e-5, call
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), call      # same kernels, same summation order


def test_noalloc_entry_point_rejects_a_problem_beyond_its_fixed_scratch(monkeypatch):
    # two K-slices of a 512 x 4224 output need 2 * 512 * 4224 * 4 bytes = 16.5 MiB of panels
    # (slices reduced through the workspace: slices reduced inside a thread-block cluster need no scratch at all)
    monkeypatch.setenv("DG_FORCE_SPLIT_K", "2")
    monkeypatch.setenv("DG_FORCE_SPLIT_CLUSTER", "-1")
    monkeypatch.setenv("DG_FORCE_BLOCK_N", "240")
    m, n, k = 512, 4224, 16384
    cfg = dg.get_gemm_config(0, m, n, k)
    needed = cfg["num_splits"] * (-(-m // 128) * 128) * (-(-n // 4) * 4) * 4
    if cfg["num_splits"] < 2 or needed <= FIXED_SCRATCH_BYTES:
        pytest.skip(f"the heuristics do not slice this shape beyond the fixed buffer ({cfg})")
    qa, sfa, qb, sfb, _ = quantise_dense(seeded_bf16((m, k), 62), seeded_bf16((n, k), 63))
    d = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    args, keep = _args(qa, sfa, qb, sfb, d)
    rc = _lib.lib.dg_fp8_fp4_gemm_noalloc(C.byref(args))
    assert rc == 1 and "bytes of scratch" in _lib.last_error() and "dg_fp8_fp4_gemm" in _lib.last_error()
    torch.cuda.synchronize()
    assert not d.any()                                                # nothing was launched
    _lib.check(_lib.lib.dg_fp8_fp4_gemm(C.byref(args)))              # the allocating entry point takes it
    torch.cuda.synchronize()
    assert oracle.calc_diff(d.float().cpu().numpy(), oracle.dequant_gemm_nt(qa, sfa, qb, sfb)) < 1e-3
    # the same slicing reduced inside clusters fits the entry point that allocates nothing, and gives the same bits
    monkeypatch.setenv("DG_FORCE_SPLIT_CLUSTER", "1")
    cfg = dg.get_gemm_config(0, m, n, k)
    assert cfg["num_splits"] == 2 and cfg["split_in_cluster"] == 1
    d2 = torch.zeros_like(d)
    args2, keep2 = _args(qa, sfa, qb, sfb, d2)
    _lib.check(_lib.lib.dg_fp8_fp4_gemm_noalloc(C.byref(args2)))
    torch.cuda.synchronize()
    assert torch.equal(d2.view(torch.int16), d.view(torch.int16))


def test_noalloc_entry_point_really_keeps_its_panels_in_the_fixed_array(monkeypatch):
    """The default slicings above are reduced inside a thread-block cluster and never touch the array.  Here the slices
    are forced through the workspace form, so the FP32 panels of the GEMM land in the library's fixed array and the
    second kernel reads them from there.  Two calls in a row with a different shape in between (whose panels overwrite
    the first shape's) must both give the bits of the allocating entry point, and the second call must leave the
    device's free memory as it found it."""
    monkeypatch.setenv("DG_FORCE_SPLIT_CLUSTER", "-1")
    monkeypatch.setenv("DG_FORCE_SPLIT_K", "4")
    shapes = [(128, 2112, 7168), (96, 1000, 4096), (128, 2112, 7168)]
    cases = {}
    for m, n, k in set(shapes):
        cfg = dg.get_gemm_config(0, m, n, k)
        assert cfg["num_splits"] > 1 and cfg["split_in_cluster"] == 0, cfg
        assert cfg["num_splits"] * (-(-m // 128) * 128) * (-(-n // 4) * 4) * 4 <= FIXED_SCRATCH_BYTES
        qa, sfa, qb, sfb, _ = quantise_dense(seeded_bf16((m, k), 64 + m), seeded_bf16((n, k), 65 + n))
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        args, keep = _args(qa, sfa, qb, sfb, want)
        _lib.check(_lib.lib.dg_fp8_fp4_gemm(C.byref(args)))          # the allocating entry point, same slicing
        torch.cuda.synchronize()
        assert oracle.calc_diff(want.float().cpu().numpy(), oracle.dequant_gemm_nt(qa, sfa, qb, sfb)) < 1e-3
        cases[(m, n, k)] = (qa, sfa, qb, sfb, want)
    for call, shape in enumerate(shapes):
        qa, sfa, qb, sfb, want = cases[shape]
        got = torch.full(want.shape, float("nan"), dtype=torch.bfloat16, device="cuda")
        args, keep = _args(qa, sfa, qb, sfb, got)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        _lib.check(_lib.lib.dg_fp8_fp4_gemm_noalloc(C.byref(args)))
        torch.cuda.synchronize()
        if call > 0:                                                  # (the first call may load the kernel image)
            assert torch.cuda.mem_get_info()[0] == free_before, call
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (call, shape)

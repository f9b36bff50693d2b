"""Size-independent properties of the kernels at the full sizes of the benchmark configurations, over every row of
every expert (the comparison with the CPU oracle itself, on oracle-quantised operands, is test_full_size_oracle_gpu.py).
The yardstick here is a BF16 tensor-core matmul of the dequantised operands (an FP8 or FP4 value times a power of two is
exact in BF16, so that product differs from ours only in the order of the FP32 sums):

  * calc_diff < 1e-3 against the dequantise-then-matmul value (the criterion of tests/test_fp8_fp4.py:54-57);
  * scaling every scale of A by 2^3 (adding 3 to the UE8M0 exponents) multiplies D by 8 exactly: bit-for-bit in BF16;
  * permuting the rows of A (with their scales) permutes the rows of D bit for bit;
  * rows the contract leaves alone (padding, rows beyond masked_m) keep a sentinel."""
import random

import pytest
import torch

import deepgemm_amd_b200 as dg
from deepgemm_amd_b200.testing import calc_diff
from deepgemm_amd_b200.utils import (align, cast_back_from_fp4, cast_back_from_fp8, per_block_cast_to_fp8, per_token_cast_to_fp4,
                                     per_token_cast_to_fp8)

pytestmark = pytest.mark.gpu

DENSE_NK = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]
SENTINEL = -7.0


def _dequant_block(q, sf):
    """e4m3 [n, k] with one scale per 128 x 128 block -> BF16 (exact)."""
    n, k = q.shape
    rows = torch.arange(n, device=q.device) // 128
    cols = torch.arange(k, device=q.device) // 128
    return (q.float() * sf[rows][:, cols]).bfloat16()


def _ref(a_deq, b_deq):
    return (a_deq @ b_deq.t()).float()


@pytest.mark.parametrize("m", [64, 128, 4096])
@pytest.mark.parametrize("n,k", DENSE_NK)
def test_dense_config_2_at_full_size(m, n, k):
    torch.manual_seed(m + n + k)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    qb, sfb = per_block_cast_to_fp8(b, True)
    d = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    dg.reset_kernel_status()
    dg.fp8_gemm_nt((qa, sfa), (qb, sfb), d)
    assert dg.kernel_status() == 0
    ref = _ref(cast_back_from_fp8(qa, sfa).bfloat16(), _dequant_block(qb, sfb))
    assert calc_diff(d, ref) < 1e-3
    assert calc_diff(d, ref.bfloat16()) < 1e-5                       # what remains is BF16 rounding of differently ordered sums
    # exponent shift: exact
    d8 = torch.empty_like(d)
    dg.fp8_gemm_nt((qa, sfa * 8.0), (qb, sfb), d8)
    assert torch.equal((d.float() * 8.0).bfloat16().view(torch.int16), d8.view(torch.int16))
    # row permutation: exact
    perm = torch.randperm(m, device="cuda")
    dp = torch.empty_like(d)
    dg.fp8_gemm_nt((qa[perm].contiguous(), sfa[perm].contiguous()), (qb, sfb), dp)
    assert torch.equal(dp.view(torch.int16), d[perm].view(torch.int16))


@pytest.mark.parametrize("b_fp4", [False, True])
@pytest.mark.parametrize("n,k", [(4096, 7168), (7168, 2048)])
def test_contiguous_grouped_configs_3_and_5_at_full_size(n, k, b_fp4):
    groups, expected = 32, 8192
    random.seed(n + k)
    torch.manual_seed(n)
    actual = [int(expected * random.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [align(x, 128) for x in actual]
    m = sum(aligned)
    layout = torch.full((m,), -1, device="cuda", dtype=torch.int32)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    start = 0
    for g, (rows, padded) in enumerate(zip(actual, aligned)):
        layout[start:start + rows] = g
        a[start + rows:start + padded] = 0
        start += padded
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    del a
    b = torch.randn((groups, n, k), device="cuda", dtype=torch.bfloat16)
    pieces = [per_token_cast_to_fp4(b[g], True, 32) if b_fp4 else per_block_cast_to_fp8(b[g], True) for g in range(groups)]
    del b
    qb, sfb = torch.stack([p[0] for p in pieces]), torch.stack([p[1] for p in pieces])
    del pieces
    d = torch.full((m, n), SENTINEL, device="cuda", dtype=torch.bfloat16)
    dg.reset_kernel_status()
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous((qa, sfa), (qb, sfb), d, layout, recipe_a=(1, 128), recipe_b=(1, 32) if b_fp4 else (128, 128))
    assert dg.kernel_status() == 0
    start, worst = 0, 0.0
    for g, (rows, padded) in enumerate(zip(actual, aligned)):
        a_deq = cast_back_from_fp8(qa[start:start + rows], sfa[start:start + rows]).bfloat16()
        b_deq = cast_back_from_fp4(qb[g], sfb[g], 32).bfloat16() if b_fp4 else _dequant_block(qb[g], sfb[g])
        worst = max(worst, float(calc_diff(d[start:start + rows], _ref(a_deq, b_deq))))
        start += padded
    assert worst < 1e-3, worst
    # the exponent shift, over the whole grouped output: exact
    d8 = torch.empty_like(d)
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous((qa, sfa * 8.0), (qb, sfb), d8, layout, recipe_a=(1, 128), recipe_b=(1, 32) if b_fp4 else (128, 128))
    valid = layout >= 0
    assert torch.equal((d[valid].float() * 8.0).bfloat16().view(torch.int16), d8[valid].view(torch.int16))


def test_masked_decode_config_4_at_full_size_in_a_cuda_graph():
    groups, max_m, n, k = 16, 256, 4096, 7168
    torch.manual_seed(4)
    a = torch.randn((groups, max_m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((groups, n, k), device="cuda", dtype=torch.bfloat16)
    qa = torch.empty_like(a, dtype=torch.float8_e4m3fn); sfa = torch.empty((groups, max_m, k // 128), device="cuda")
    qb = torch.empty_like(b, dtype=torch.float8_e4m3fn); sfb = torch.empty((groups, n // 128, k // 128), device="cuda")
    for g in range(groups):
        qa[g], sfa[g] = per_token_cast_to_fp8(a[g], True, 128)
        qb[g], sfb[g] = per_block_cast_to_fp8(b[g], True)
    psfa = dg.transform_sf_into_required_layout(sfa, max_m, k, (1, 128), groups)
    psfb = dg.transform_sf_into_required_layout(sfb, n, k, (128, 128), groups)
    masked = torch.randint(45, 84, (groups,), device="cuda", dtype=torch.int)
    d = torch.full((groups, max_m, n), SENTINEL, device="cuda", dtype=torch.bfloat16)
    dg.m_grouped_fp8_gemm_nt_masked((qa, psfa), (qb, psfb), d, masked, 64, recipe=(1, 1, 128))        # warm-up outside the capture
    torch.cuda.synchronize()
    stream, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            dg.m_grouped_fp8_gemm_nt_masked((qa, psfa), (qb, psfb), d, masked, 64, recipe=(1, 1, 128))
    for trial in range(2):                                            # the graph follows new counts without a new capture
        masked.copy_(torch.randint(45, 84, (groups,), device="cuda", dtype=torch.int))
        d.fill_(SENTINEL)
        dg.reset_kernel_status()
        graph.replay()
        assert dg.kernel_status() == 0
        for g in range(groups):
            rows = int(masked[g])
            ref = _ref(cast_back_from_fp8(qa[g, :rows], sfa[g, :rows]).bfloat16(), _dequant_block(qb[g], sfb[g]))
            assert calc_diff(d[g, :rows], ref) < 1e-3
            assert (d[g, rows:] == SENTINEL).all()                    # rows beyond masked_m are left untouched


@pytest.mark.parametrize("n,k", [(7168, 2048), (4096, 7168)])
def test_fp8_x_fp4_dense_config_5_at_full_size(n, k):
    m = 4096
    torch.manual_seed(n + 5)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    qb, sfb = per_token_cast_to_fp4(b, True, 32)
    d = torch.empty((m, n), device="cuda", dtype=torch.bfloat16)
    dg.reset_kernel_status()
    dg.fp8_fp4_gemm_nt((qa, sfa), (qb, sfb), d, recipe_a=(1, 128), recipe_b=(1, 32))
    assert dg.kernel_status() == 0
    ref = _ref(cast_back_from_fp8(qa, sfa).bfloat16(), cast_back_from_fp4(qb, sfb, 32).bfloat16())
    assert calc_diff(d, ref) < 1e-3
    assert calc_diff(d, (a.float() @ b.float().t())) < 1e-2           # the reference's own bound against the unquantised product
    d8 = torch.empty_like(d)
    dg.fp8_fp4_gemm_nt((qa, sfa), (qb, sfb * 8.0), d8, recipe_a=(1, 128), recipe_b=(1, 32))
    assert torch.equal((d.float() * 8.0).bfloat16().view(torch.int16), d8.view(torch.int16))

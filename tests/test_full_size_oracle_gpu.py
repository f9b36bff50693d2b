"""The benchmark configurations at their full sizes against the CPU oracle itself.

Every case draws N(0, 1) BF16 operands, quantises them on the host with the oracle's restatement of the reference's
casts (deep_gemm/utils/math.py:26-72,99-125; row chunks in parallel, the same bytes as one call), runs the GPU kernel
on those bytes and compares D with `oracle.dequant_gemm_nt` of the same bytes: calc_diff < 1e-3, the reference's
criterion (tests/test_fp8_fp4.py:54-57, tests/generators.py:69-74).  What separates the two is the order of the FP32
sums and the final BF16 rounding, so the measured difference is ~1e-6; the test holds it to 1e-5 as well.

  * config 2: M in {64, 128, 4096} x the six (N, K);
  * config 4: 16 groups x 256 rows masked to 45..83, N = 4096, K = 7168, all groups, rows beyond masked_m untouched;
  * config 5: FP8 x FP4 at M = 4096, both shapes;
  * configs 3 and 5 (grouped): 32 experts x ~8192 rows on the GPU, of which four experts (first, last, fewest rows,
    most rows) carry oracle-quantised operands and are compared row for row; the product's torch quantisers must give
    the same bytes for them.

The properties that do not depend on the size (exponent shift, row permutation, sentinels over every expert) stay in
test_full_size_properties_gpu.py.
"""
import random

import numpy as np
import pytest
import torch

import oracle
from gpu_helpers import fp4_cuda, fp8_cuda, in_row_chunks, packed_sf_cuda, quantise_dense_parallel

pytestmark = pytest.mark.gpu

dg = pytest.importorskip("deepgemm_amd_b200")

DENSE_NK = [(2112, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048)]
SENTINEL = -7.0


def _randn_bf16(shape, seed):
    """N(0, 1) BF16 drawn on the GPU (fast at these sizes), returned as the float32 numpy array the oracle takes."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, device="cuda", dtype=torch.bfloat16, generator=g).float().cpu().numpy()


def _check(d, ref, what):
    got = d.float().cpu().numpy()
    diff = oracle.calc_diff(got, ref)
    assert diff < 1e-3, (what, diff)
    # beyond the criterion: only summation order and the BF16 rounding of D separate the two
    assert oracle.calc_diff(got, oracle.bf16_round(ref)) < 1e-5, what


@pytest.mark.parametrize("n,k", DENSE_NK)
@pytest.mark.parametrize("m", [64, 128, 4096])
def test_dense_config_2_against_the_oracle(m, n, k):
    a, b = _randn_bf16((m, k), 11 * m + n), _randn_bf16((n, k), 13 * n + k)
    qa, sfa, qb, sfb = quantise_dense_parallel(a, b)
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.reset_kernel_status()
    dg.fp8_gemm_nt((fp8_cuda(qa), packed_sf_cuda(sfa)), (fp8_cuda(qb), packed_sf_cuda(sfb)), d, recipe=(1, 1, 128))
    assert dg.kernel_status() == 0
    _check(d, oracle.dequant_gemm_nt(qa, sfa, qb, sfb), (m, n, k))


@pytest.mark.parametrize("n,k", [(7168, 2048), (4096, 7168)])
def test_fp8_x_fp4_dense_config_5_against_the_oracle(n, k):
    m = 4096
    a, b = _randn_bf16((m, k), 17 + n), _randn_bf16((n, k), 19 + k)
    qa, sfa, qb, sfb = quantise_dense_parallel(a, b, b_fp4=True)
    d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.reset_kernel_status()
    dg.fp8_fp4_gemm_nt((fp8_cuda(qa), packed_sf_cuda(sfa)), (fp4_cuda(qb), packed_sf_cuda(sfb)), d, recipe_a=(1, 128), recipe_b=(1, 32))
    assert dg.kernel_status() == 0
    _check(d, oracle.dequant_gemm_nt(qa, sfa, qb, sfb, 128, 32, False, True), (m, n, k))
    # the reference's own bound for this pair of formats, against the unquantised product (tests/generators.py:69-74)
    assert oracle.calc_diff(d.float().cpu().numpy(), a @ b.T) < 1e-2


def test_masked_decode_config_4_against_the_oracle():
    groups, max_m, n, k = 16, 256, 4096, 7168
    rng = random.Random(4)
    counts = [rng.randint(45, 83) for _ in range(groups)]
    a, b = _randn_bf16((groups * max_m, k), 23), _randn_bf16((groups * n, k), 29)
    qa, sfa, qb, sfb = quantise_dense_parallel(a, b)              # n is a multiple of 128: blocks never straddle groups
    qa, sfa = qa.reshape(groups, max_m, k), sfa.reshape(groups, max_m, -1)
    qb, sfb = qb.reshape(groups, n, k), sfb.reshape(groups, n, -1)
    d = torch.full((groups, max_m, n), SENTINEL, dtype=torch.bfloat16, device="cuda")
    masked = torch.tensor(counts, dtype=torch.int, device="cuda")
    dg.reset_kernel_status()
    dg.m_grouped_fp8_gemm_nt_masked((fp8_cuda(qa), packed_sf_cuda(sfa)), (fp8_cuda(qb), packed_sf_cuda(sfb)), d, masked, 64,
                                    recipe=(1, 1, 128))
    assert dg.kernel_status() == 0
    ref = oracle.m_grouped_masked_ref(qa, sfa, qb, sfb, counts)
    out = d.float().cpu().numpy()
    valid = ~np.isnan(ref)
    assert valid.sum() == sum(counts) * n
    assert oracle.calc_diff(out[valid], ref[valid]) < 1e-3
    assert oracle.calc_diff(out[valid], oracle.bf16_round(ref[valid])) < 1e-5
    assert (out[~valid] == SENTINEL).all()                        # bit-exact masked-row handling


@pytest.mark.parametrize("b_fp4", [False, True])
@pytest.mark.parametrize("n,k", [(4096, 7168), (7168, 2048)])
def test_contiguous_grouped_configs_3_and_5_sampled_experts_against_the_oracle(n, k, b_fp4):
    from deepgemm_amd_b200.utils import per_block_cast_to_fp8, per_token_cast_to_fp4, per_token_cast_to_fp8
    groups, expected = 32, 8192
    rng = random.Random(0)
    actual = [int(expected * rng.uniform(0.7, 1.3)) for _ in range(groups)]         # tests/generators.py:383-404
    aligned = [oracle.align(x, 128) for x in actual]
    starts = [sum(aligned[:g]) for g in range(groups)]
    m = sum(aligned)
    sampled = sorted({0, groups - 1, int(np.argmin(actual)), int(np.argmax(actual))})
    assert len(sampled) == 4

    gen = torch.Generator(device="cuda").manual_seed(n + k)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16, generator=gen)
    layout = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    for g in range(groups):
        layout[starts[g]:starts[g] + actual[g]] = g
    a[layout < 0] = 0                                                                 # tests/generators.py:406
    qa, sfa = per_token_cast_to_fp8(a, True, 128)
    sfa = dg.transform_sf_into_required_layout(sfa, m, k, (1, 128))
    recipe_b = (1, 32) if b_fp4 else (128, 128)
    qb_all, sfb_all, host = [], [], {}
    for g in range(groups):
        w = torch.randn((n, k), device="cuda", dtype=torch.bfloat16, generator=gen)
        q, s = per_token_cast_to_fp4(w, True, 32) if b_fp4 else per_block_cast_to_fp8(w, True)
        if g in sampled:
            # the oracle's bytes for this expert: the product's torch quantisers must agree, and the oracle's are used
            rows = slice(starts[g], starts[g] + actual[g])
            a_host, w_host = a[rows].float().cpu().numpy(), w.float().cpu().numpy()
            oqa, osfa, oqb, osfb = quantise_dense_parallel(a_host, w_host, b_fp4=b_fp4)
            assert np.array_equal(qa[rows].view(torch.uint8).cpu().numpy(), oqa), g
            assert np.array_equal(q.view(torch.uint8).cpu().numpy(), oqb.view(np.uint8)), g
            host[g] = (oqa, osfa, oqb, osfb)
        qb_all.append(q)
        sfb_all.append(s)
        del w
    del a
    qb = torch.stack(qb_all)
    sfb = dg.transform_sf_into_required_layout(torch.stack(sfb_all), n, k, recipe_b, groups)
    del qb_all, sfb_all
    d = torch.full((m, n), SENTINEL, dtype=torch.bfloat16, device="cuda")
    dg.reset_kernel_status()
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous((qa, sfa), (qb, sfb), d, layout, recipe_a=(1, 128), recipe_b=(1, 32) if b_fp4 else (1, 128))
    assert dg.kernel_status() == 0
    for g in sampled:
        oqa, osfa, oqb, osfb = host[g]
        ref = oracle.dequant_gemm_nt(oqa, osfa, oqb, osfb, 128, 32 if b_fp4 else 128, False, b_fp4)
        _check(d[starts[g]:starts[g] + actual[g]], ref, ("expert", g, n, k, b_fp4))

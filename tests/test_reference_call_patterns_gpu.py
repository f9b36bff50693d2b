"""The call patterns of the reference's own test scripts (tests/test_fp8_fp4.py, tests/test_bf16.py, tests/test_einsum.py
and the generators they use), driven end to end through this package's torch-side helpers, the way a caller that
switches libraries would: quantise with deep_gemm.utils, hand (data, scales) pairs of either majorness to the GEMM, compare
with the BF16 matmul at the reference's tolerances (tests/generators.py:69-74)."""
import random

import pytest
import torch

import deepgemm_amd_b200 as dg
from deepgemm_amd_b200.testing import calc_diff
from deepgemm_amd_b200.utils import (align, ceil_div, per_block_cast_to_fp8, per_token_cast_to_fp4, per_token_cast_to_fp8,
                                     transpose_packed_fp4)

pytestmark = pytest.mark.gpu

# (gran_k_a, gran_k_b, A is FP4, B is FP4): tests/generators.py:76-86
QUANT_CONFIGS = [(128, 128, False, False), (128, 32, False, True), (32, 32, True, True)]


def _tolerance(fa, fb):
    return 0.02 if fa and fb else 0.01 if fa or fb else 0.001


def _cast(x, mn_major, gran, fp4, block):
    if fp4:
        q, sf = per_token_cast_to_fp4(x, True, gran)
        return (q, sf) if not mn_major else (transpose_packed_fp4(q).T, sf)
    q, sf = per_block_cast_to_fp8(x, True, gran) if block else per_token_cast_to_fp8(x, True, gran)
    return (q, sf) if not mn_major else (q.T.contiguous().T, sf)


def _grouped_cast(x, mn_major, gran, fp4, block):
    pieces = [_cast(x[i], False, gran, fp4, block) for i in range(x.size(0))]
    data, sf = torch.stack([p[0] for p in pieces]), torch.stack([p[1] for p in pieces])
    if not mn_major:
        return data, sf
    if fp4:
        return torch.stack([transpose_packed_fp4(p[0]) for p in pieces]).mT, sf
    return data.mT.contiguous().mT, sf


@pytest.mark.parametrize("config", QUANT_CONFIGS)
@pytest.mark.parametrize("m,n,k,ta,tb,accumulate,out_dtype", [
    (1, 2112, 7168, False, False, False, torch.bfloat16), (128, 576, 7168, False, False, True, torch.bfloat16),
    (512, 1536, 768, False, True, False, torch.bfloat16),                     # dgrad: B stored [K, N]
    (768, 512, 1536, True, True, True, torch.float), (768, 512, 1536, True, True, False, torch.bfloat16)])   # wgrad: both transposed
def test_dense_forward_and_backward_forms(config, m, n, k, ta, tb, accumulate, out_dtype):
    ga, gb, fa, fb = config
    if fa and (ta or tb):
        pytest.skip("FP4 x FP4 has no backward forms (tests/generators.py:157)")
    random.seed(m + n + k)
    torch.manual_seed(m * n)
    for alias in (False, True):
        for alpha in (None, random.uniform(-1.0, 1.0)):
            a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
            b = torch.randn((n, k), device="cuda", dtype=torch.bfloat16)
            d = torch.randn((m, n), device="cuda", dtype=out_dtype) * 32 if accumulate else torch.empty((m, n), device="cuda", dtype=out_dtype)
            c = d if accumulate else None
            ref = ((1.0 if alpha is None else alpha) * (a.float() @ b.float().t()) + (c if accumulate else 0)).to(out_dtype)
            # with accumulation (the weight-gradient GEMM) B is quantised per token as well
            qa, qb = _cast(a, ta, ga, fa, False), _cast(b, tb, gb, fb, not accumulate)
            recipe_a, recipe_b = (1, ga), ((1, gb) if fb or accumulate else (gb, gb))
            name = "fp8_fp4_gemm_" + ((("t" if ta else "n") + ("n" if tb else "t")) if alias else "nt")
            if alias:                       # the aliases take the contiguous storage; "nt" reads the majorness off the strides
                qa = qa if not ta else (qa[0].T, qa[1].T)
                qb = qb if not tb else (qb[0].T, qb[1].T)
                assert qa[0].is_contiguous() and qb[0].is_contiguous()
            getattr(dg, name)(qa, qb, d, c=c, disable_ue8m0_cast=False, recipe=None, recipe_a=recipe_a, recipe_b=recipe_b, alpha=alpha)
            assert calc_diff(d, ref) < _tolerance(fa, fb), (name, alpha)


@pytest.mark.parametrize("config", QUANT_CONFIGS)
@pytest.mark.parametrize("use_psum_layout,ensure_zero_padding", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("tb", [False, True])
def test_m_grouped_contiguous_from_torch_side_quantisers(config, use_psum_layout, ensure_zero_padding, tb):
    ga, gb, fa, fb = config
    if fa and tb:
        pytest.skip("FP4 x FP4 takes K-major weights (tests/generators.py:207)")
    groups, expected_m, n, k = 4, 300, 1024, 768
    random.seed(7)
    torch.manual_seed(7)
    alignment = dg.get_mk_alignment_for_contiguous_layout()
    actual = [int(expected_m * random.uniform(0.7, 1.3)) for _ in range(groups)]
    aligned = [align(x, alignment) for x in actual]
    m = sum(aligned)
    a = torch.randn((m, k), device="cuda", dtype=torch.bfloat16)
    b = torch.randn((groups, n, k), device="cuda", dtype=torch.bfloat16)
    layout = torch.empty(groups if use_psum_layout else m, device="cuda", dtype=torch.int32)
    ref = torch.zeros((m, n), device="cuda", dtype=torch.bfloat16)
    valid = torch.zeros(m, device="cuda", dtype=torch.bool)
    start = 0
    for i, (rows, padded) in enumerate(zip(actual, aligned)):
        if use_psum_layout:
            layout[i] = start + rows
        else:
            layout[start:start + rows] = i
            layout[start + rows:start + padded] = -1
        valid[start:start + rows] = True
        a[start + rows:start + padded] = 0
        ref[start:start + padded] = a[start:start + padded] @ b[i].t()
        start += padded
    qa, qb = _cast(a, False, ga, fa, False), _grouped_cast(b, tb, gb, fb, True)
    d = torch.full((m, n), 7.0, device="cuda", dtype=torch.bfloat16)
    dg.m_grouped_fp8_fp4_gemm_nt_contiguous(qa, qb, d, layout, disable_ue8m0_cast=False, recipe=None, recipe_a=(1, ga),
                                            recipe_b=(1, gb) if fb else (gb, gb), use_psum_layout=use_psum_layout,
                                            ensure_zero_padding=ensure_zero_padding)
    assert calc_diff(d[valid], ref[valid]) < _tolerance(fa, fb)
    if ensure_zero_padding:
        assert not d[~valid].any()                                   # tests/utils.py:9-17


@pytest.mark.parametrize("config", QUANT_CONFIGS)
@pytest.mark.parametrize("use_psum_layout", [False, True])
def test_m_grouped_masked_and_its_prefix_sum_form(config, use_psum_layout):
    """tests/test_fp8_fp4.py:178-222: the masked GEMM, and the same problem moved into the prefix-sum layout, whose gap rows
    (data and FP32 scales) stay uninitialised."""
    ga, gb, fa, fb = config
    groups, max_m, expected_m_per_group, n, k = 6, 512, 150, 1024, 768
    random.seed(9)
    torch.manual_seed(9)
    expected_m = int(expected_m_per_group * 1.2)
    dg.set_mk_alignment_for_contiguous_layout(dg.get_theoretical_mk_alignment_for_contiguous_layout(expected_m))
    try:
        alignment = dg.get_mk_alignment_for_contiguous_layout()
        a = torch.randn((groups, max_m, k), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((groups, n, k), device="cuda", dtype=torch.bfloat16)
        d = torch.empty((groups, max_m, n), device="cuda", dtype=torch.bfloat16)
        ref = torch.einsum("gmk,gnk->gmn", a, b)
        masked = [int(expected_m_per_group * random.uniform(0.7, 1.3)) for _ in range(groups)]
        ends, last = [], 0
        for rows in masked:
            ends.append(last + rows)
            last = align(ends[-1], alignment)
        masked_m = torch.tensor(masked, device="cuda", dtype=torch.int)
        psum_m = torch.tensor(ends, device="cuda", dtype=torch.int)
        qa, qb = _grouped_cast(a, False, ga, fa, False), _grouped_cast(b, False, gb, fb, True)
        recipes = dict(disable_ue8m0_cast=False, recipe=None, recipe_a=(1, ga), recipe_b=(1, gb) if fb else (gb, gb))
        if not use_psum_layout:
            for g in range(groups):
                qa[1][g, masked[g]:] = 0
            dg.m_grouped_fp8_fp4_gemm_nt_masked(qa, qb, d, masked_m, expected_m, **recipes)
            valid = torch.arange(max_m, device="cuda")[None, :] < masked_m[:, None]
            assert calc_diff(d[valid], ref[valid]) < _tolerance(fa, fb)
            return

        def to_psum(x):
            out = torch.empty((align(ends[-1], alignment), x.size(-1)), dtype=x.dtype, device=x.device)
            begin = 0
            for g in range(groups):
                out[begin:ends[g]] = x[g, :ends[g] - begin]
                begin = align(ends[g], alignment)
            return out

        qa = (to_psum(qa[0]), to_psum(qa[1]))
        d_psum, ref_psum = to_psum(d), to_psum(ref)
        valid = torch.zeros(d_psum.size(0), device="cuda", dtype=torch.bool)
        begin = 0
        for g in range(groups):
            valid[begin:ends[g]] = True
            begin = align(ends[g], alignment)
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(qa, qb, d_psum, psum_m, use_psum_layout=True, expected_m_for_psum_layout=expected_m, **recipes)
        assert calc_diff(d_psum[valid], ref_psum[valid]) < _tolerance(fa, fb)
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)


def test_fp8_einsum_with_the_quantised_output_pair_and_a_permuted_accumulator():
    """tests/test_einsum.py:128-183."""
    from deepgemm_amd_b200.utils import cast_back_from_fp8
    b, h, r, d = 132, 4, 1024, 512
    torch.manual_seed(11)
    x = torch.randn((b, h, r), device="cuda", dtype=torch.bfloat16)
    y = torch.randn((h, d, r), device="cuda", dtype=torch.bfloat16)
    ref = torch.einsum("bhr,hdr->bhd", x, y)
    xq = per_token_cast_to_fp8(x.view(-1, r), True)
    xq = xq[0].view(b, h, r), xq[1].view(b, h, ceil_div(r, 128))
    pieces = [per_block_cast_to_fp8(y[i], True) for i in range(h)]
    yq = torch.stack([p[0] for p in pieces]), torch.stack([p[1] for p in pieces])
    z = torch.empty((b, h, d), device="cuda", dtype=torch.bfloat16)
    dg.fp8_einsum("bhr,hdr->bhd", xq, yq, z)
    assert calc_diff(z, ref) < 1e-3
    out = torch.empty_like(z, dtype=torch.float8_e4m3fn)
    sfd = torch.empty_strided((b, ceil_div(h * d, 128)), (1, align(b, 4)), dtype=torch.int32, device="cuda")
    dg.fp8_einsum("bhr,hdr->bhd", xq, yq, (out, sfd))
    back = cast_back_from_fp8(out.view(b, h * d), sfd.contiguous(), gran_k=32, use_packed_ue8m0=True)
    assert calc_diff(back, ref.reshape(b, h * d)) < 2e-3
    want_q, want_sf = per_token_cast_to_fp8(z.view(b, h * d), True, 32, use_packed_ue8m0=True)
    assert torch.equal(out.view(b, h * d).view(torch.uint8), want_q.view(torch.uint8)) and torch.equal(sfd.contiguous(), want_sf)
    acc = torch.zeros((h, b, d), device="cuda", dtype=torch.float).permute(1, 0, 2)
    dg.fp8_einsum("bhr,hdr->bhd", xq, yq, acc, c=acc)
    assert torch.equal(acc.bfloat16(), z)                            # the direct output is the rounded FP32 accumulation


def test_bf16_einsum_with_a_strided_operand():
    """tests/test_einsum.py:44-105: the weights are a slice of a wider tensor."""
    b, h, r, d = 96, 8, 512, 256
    torch.manual_seed(12)
    x = torch.randn((b, h, r), device="cuda", dtype=torch.bfloat16)
    y = torch.randn((h, d, r + 128), device="cuda", dtype=torch.bfloat16)[:, :, :r]
    z = torch.empty((b, h, d), device="cuda", dtype=torch.bfloat16)
    dg.einsum("bhr,hdr->bhd", x, y, z)
    assert calc_diff(z, torch.einsum("bhr,hdr->bhd", x, y)) < 1e-10
    acc = torch.zeros((b, h, d), device="cuda", dtype=torch.float)
    dg.einsum("bhr,hdr->bhd", x, y, acc, c=acc)
    assert torch.equal(acc.bfloat16(), z)
    x2 = torch.randn((b, h, d), device="cuda", dtype=torch.bfloat16)
    z2 = torch.empty((b, h, r), device="cuda", dtype=torch.bfloat16)
    dg.einsum("bhd,hdr->bhr", x2, y, z2)
    assert calc_diff(z2, torch.einsum("bhd,hdr->bhr", x2, y)) < 1e-10

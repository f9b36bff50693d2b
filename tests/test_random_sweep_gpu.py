"""A bounded, seeded slice of the randomised sweeps: 60 dense and 40 grouped cases drawn from fixed seeds.

Dense: M from 1 to 513, ragged N and K, FP8 x FP8 / FP8 x FP4 / FP4 x FP4, BF16 and FP32 output, alpha, accumulation.
Grouped: the contiguous, prefix-sum and masked forms with empty groups, alignments 128 and 256, FP4 weights and
MN-major weights.  Every case is held to calc_diff < 1e-3 against the dequantise-then-matmul value (a BF16 tensor-core
matmul of the dequantised operands: an FP8 or FP4 value times a power of two is exact in BF16), to a clean status word,
to no NaN left in D, and to sentinel / zero rows where the contract leaves rows alone.  The torch quantisers used here
are pinned to the oracle bit for bit in test_gemm_gpu.py; the shapes follow the spirit of the reference's
enumerations (tests/generators.py:122-227, 378-485) with the awkward sizes those leave out.
"""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu

dg = pytest.importorskip("deepgemm_amd_b200")
from deepgemm_amd_b200.testing import calc_diff  # noqa: E402
from deepgemm_amd_b200.utils import (align, cast_back_from_fp4, cast_back_from_fp8, per_block_cast_to_fp8,  # noqa: E402
                                     per_token_cast_to_fp4, per_token_cast_to_fp8, transpose_packed_fp4)

SENTINEL = -7.0


def _deq_block(q, sf):
    n, k = q.shape
    return (q.float() * sf[torch.arange(n, device="cuda") // 128][:, torch.arange(k, device="cuda") // 128]).bfloat16()


def _dense_cases(seed, count):
    rng = random.Random(seed)
    cases = []
    for _ in range(count):
        m = rng.choice([1, 2, 7, 16, 17, 31, 32, 33, 48, 63, 64, 65, 100, 128, 129, 200, 256, 300, 513])
        n = rng.choice([128, 136, 264, 576, 1000, 2112, 2048, 4096, 5000, 7168])
        k = rng.choice([128, 256, 384, 512, 640, 1024, 1152, 2048, 2176, 2304, 4096, 7168, 16384])
        fmt = rng.choice(["fp8", "fp8", "fp4b", "fp4ab"])
        out = rng.choice(["bf16", "fp32"])
        acc = rng.random() < 0.2 and out == "fp32"
        alpha = rng.choice([None, None, 0.5, -1.25])
        if fmt != "fp8" and k % 128:
            k = align(k, 128)
        cases.append((m, n, k, fmt, out, acc, alpha))
    return cases


@pytest.mark.parametrize("chunk", range(6))
def test_random_dense_cases(chunk):
    torch.manual_seed(100 + chunk)
    for m, n, k, fmt, out, acc, alpha in _dense_cases(1000 + chunk, 10):
        odt = torch.bfloat16 if out == "bf16" else torch.float
        a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(n, k, device="cuda", dtype=torch.bfloat16)
        if fmt == "fp4ab":
            qa, sfa = per_token_cast_to_fp4(a, True, 32)
            a_deq, ra = cast_back_from_fp4(qa, sfa, 32).bfloat16(), (1, 32)
        else:
            qa, sfa = per_token_cast_to_fp8(a, True, 128)
            a_deq, ra = cast_back_from_fp8(qa, sfa).bfloat16(), (1, 128)
        if fmt == "fp8":
            qb, sfb = per_block_cast_to_fp8(b, True)
            b_deq, rb = _deq_block(qb, sfb), (128, 128)
        else:
            qb, sfb = per_token_cast_to_fp4(b, True, 32)
            b_deq, rb = cast_back_from_fp4(qb, sfb, 32).bfloat16(), (1, 32)
        d0 = torch.randn(m, n, device="cuda", dtype=odt) if acc else None
        d = d0.clone() if acc else torch.full((m, n), float("nan"), device="cuda", dtype=odt)
        ref = (a_deq @ b_deq.t()).float() * (alpha if alpha is not None else 1.0) + (d0 if acc else 0)
        label = f"m{m} n{n} k{k} {fmt} {out} acc{acc} alpha{alpha}"
        dg.reset_kernel_status()
        dg.fp8_fp4_gemm_nt((qa, sfa), (qb, sfb), d, c=d if acc else None, recipe_a=ra, recipe_b=rb, alpha=alpha)
        assert dg.kernel_status() == 0, label
        assert not torch.isnan(d.float()).any(), label
        assert float(calc_diff(d, ref)) < 1e-3, label


def _grouped_cases(seed, count):
    rng = random.Random(seed)
    cases = []
    for _ in range(count):
        kind = rng.choice(["contig", "psum", "masked"])
        g = rng.choice([1, 2, 5, 8])
        n = rng.choice([128, 256, 640, 1024, 2048, 2176])
        k = rng.choice([128, 384, 1024, 2048, 7168])
        fp4 = rng.random() < 0.35
        mn_major_b = rng.random() < 0.3 and kind != "masked"
        alignment = rng.choice([128, 256])
        if kind == "masked":
            max_m = rng.choice([64, 256, 520])
            rows = [rng.randint(0, max_m) for _ in range(g)]
        else:
            max_m = 0
            rows = [rng.choice([0, 1, 77, 128, 130, 256, 300]) for _ in range(g)]
        zero_padding = kind == "psum" and rng.random() < 0.5
        cases.append((kind, g, n, k, fp4, mn_major_b, alignment, max_m, rows, zero_padding))
    return cases


@pytest.mark.parametrize("chunk", range(4))
def test_random_grouped_cases(chunk):
    torch.manual_seed(200 + chunk)
    try:
        for kind, g, n, k, fp4, mn_major_b, alignment, max_m, rows, zero_padding in _grouped_cases(2000 + chunk, 10):
            label = f"{kind} g{g} n{n} k{k} fp4{fp4} mn_major_b{mn_major_b} alignment{alignment} rows{rows}"
            dg.set_mk_alignment_for_contiguous_layout(alignment)
            b = torch.randn(g, n, k, device="cuda", dtype=torch.bfloat16)
            pieces = [per_token_cast_to_fp4(b[i], True, 32) if fp4 else per_block_cast_to_fp8(b[i], True) for i in range(g)]
            qb, sfb = torch.stack([p[0] for p in pieces]), torch.stack([p[1] for p in pieces])
            b_deq = [cast_back_from_fp4(qb[i], sfb[i], 32).bfloat16() if fp4 else _deq_block(qb[i], sfb[i]) for i in range(g)]
            if mn_major_b:      # the same weights stored [K, N]: read off the strides, as csrc/utils/layout.hpp:29-33 does
                qb_in = torch.stack([transpose_packed_fp4(qb[i]) for i in range(g)]).mT if fp4 else qb.mT.contiguous().mT
            else:
                qb_in = qb
            rb = (1, 32) if fp4 else (128, 128)
            dg.reset_kernel_status()
            if kind == "masked":
                a = torch.randn(g, max_m, k, device="cuda", dtype=torch.bfloat16)
                qa = torch.empty_like(a, dtype=torch.float8_e4m3fn)
                sfa = torch.empty(g, max_m, (k + 127) // 128, device="cuda")
                for i in range(g):
                    qa[i], sfa[i] = per_token_cast_to_fp8(a[i], True, 128)
                masked = torch.tensor(rows, device="cuda", dtype=torch.int)
                d = torch.full((g, max_m, n), SENTINEL, device="cuda", dtype=torch.bfloat16)
                dg.m_grouped_fp8_fp4_gemm_nt_masked((qa, sfa), (qb_in, sfb), d, masked, max(1, sum(rows) // g),
                                                    recipe_a=(1, 128), recipe_b=rb)
                assert dg.kernel_status() == 0, label
                for i, r in enumerate(rows):
                    if r:
                        ref = (cast_back_from_fp8(qa[i, :r], sfa[i, :r]).bfloat16() @ b_deq[i].t()).float()
                        assert float(calc_diff(d[i, :r], ref)) < 1e-3, label
                    assert (d[i, r:] == SENTINEL).all(), label
                continue
            aligned = [align(x, alignment) for x in rows]
            m = sum(aligned)
            if m == 0:
                continue
            a = torch.randn(m, k, device="cuda", dtype=torch.bfloat16)
            layout = torch.full((m,), -1, device="cuda", dtype=torch.int32) if kind == "contig" else torch.empty(g, device="cuda", dtype=torch.int32)
            valid = torch.zeros(m, device="cuda", dtype=torch.bool)
            start, segments = 0, []
            for i, (r, p) in enumerate(zip(rows, aligned)):
                if kind == "contig":
                    layout[start:start + r] = i
                else:
                    layout[i] = start + r
                valid[start:start + r] = True
                a[start + r:start + p] = 0
                segments.append((start, r))
                start += p
            qa, sfa = per_token_cast_to_fp8(a, True, 128)
            d = torch.full((m, n), SENTINEL, device="cuda", dtype=torch.bfloat16)
            dg.m_grouped_fp8_fp4_gemm_nt_contiguous((qa, sfa), (qb_in, sfb), d, layout, recipe_a=(1, 128), recipe_b=rb,
                                                    use_psum_layout=kind == "psum", ensure_zero_padding=zero_padding)
            assert dg.kernel_status() == 0, label
            for i, (s0, r) in enumerate(segments):
                if r:
                    ref = (cast_back_from_fp8(qa[s0:s0 + r], sfa[s0:s0 + r]).bfloat16() @ b_deq[i].t()).float()
                    assert float(calc_diff(d[s0:s0 + r], ref)) < 1e-3, label
            if kind == "psum":      # rows between groups: zeros on request, otherwise untouched
                assert (d[~valid] == (0 if zero_padding else SENTINEL)).all(), label
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)

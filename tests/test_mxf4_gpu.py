"""FP4 x FP4 through tcgen05.mma.kind::mxf4: packed operands in shared memory, 256 elements of K per pipeline stage, two
packed scale words per row and stage, twice the FP8 tensor rate.

The reference runs FP4 x FP4 the same way (kIsMXF4, deep_gemm/include/deep_gemm/impls/sm100_fp8_fp4_gemm_1d1d.cuh:51-54,
UMMA_K 64 and BLOCK_K 256 at csrc/jit_kernels/heuristics/sm100.hpp:32) and holds it to the result of the same data
re-encoded as E4M3 (tests/test_fp8_fp4.py:95-100).  Here every case is compared with the CPU oracle and with this
library's own kind::mxf8f6f4 path (DG_DISABLE_MXF4=1), which unpacks the same operands to one byte per element.
"""
import numpy as np
import pytest
import torch

import oracle
from gpu_helpers import diff_report, fp4_cuda, packed_sf_cuda, seeded_bf16

pytestmark = pytest.mark.gpu

dg = pytest.importorskip("deepgemm_amd_b200")
from deepgemm_amd_b200 import _lib  # noqa: E402


def _quantise(m, n, k, seed):
    a, b = seeded_bf16((m, k), seed), seeded_bf16((n, k), seed + 1)
    qa, sfa = oracle.per_token_cast_to_fp4(a, True, 32)
    qb, sfb = oracle.per_token_cast_to_fp4(b, True, 32)
    return qa, sfa, qb, sfb


def _run(qa, sfa, qb, sfb, out_dtype=torch.bfloat16, **kw):
    m, n = qa.shape[0], qb.shape[0]
    d = torch.full((m, n), float("nan"), dtype=out_dtype, device="cuda")
    dg.reset_kernel_status()
    dg.fp4_gemm_nt((fp4_cuda(qa), packed_sf_cuda(sfa)), (fp4_cuda(qb), packed_sf_cuda(sfb)), d, recipe_a=(1, 32), recipe_b=(1, 32), **kw)
    assert dg.kernel_status() == 0
    return d


@pytest.mark.parametrize("m,n,k", [
    (128, 128, 256),            # one tile, one K-block: both packed words, all four MMAs
    (128, 128, 128),            # half a K-block: the second word and the second half of the stage are out of range
    (128, 256, 384),            # an odd number of packed words: the last K-block is half filled
    (1, 128, 512), (129, 304, 640), (200, 2112, 1792),
    (1000, 576, 7168), (4096, 512, 2048),
])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float])
def test_mxf4_matches_the_oracle_and_the_unpacked_path(m, n, k, out_dtype, monkeypatch):
    qa, sfa, qb, sfb = _quantise(m, n, k, 300 + m + k)
    ref = oracle.dequant_gemm_nt(qa, sfa, qb, sfb, 32, 32, True, True)
    d = _run(qa, sfa, qb, sfb, out_dtype)
    out = d.float().cpu().numpy()
    assert not np.isnan(out).any()
    assert oracle.calc_diff(out, ref) < 1e-3, diff_report(out, ref)                       # the benchmark's criterion
    want = ref if out_dtype == torch.float else oracle.bf16_round(ref)
    assert oracle.calc_diff(out, want) < 1e-5, diff_report(out, ref)                     # only the order of the sums differs
    monkeypatch.setenv("DG_DISABLE_MXF4", "1")                                            # the kind::mxf8f6f4 path on the same bytes
    d_unpacked = _run(qa, sfa, qb, sfb, out_dtype)
    assert float(oracle.calc_diff(out, d_unpacked.float().cpu().numpy())) < 1e-9


@pytest.mark.parametrize("cluster,block_m,bn", [(1, 128, 240), (1, 256, 240), (2, 128, 224), (2, 256, 208), (1, 128, 16), (1, 256, 96)])
def test_mxf4_tile_variants_give_the_same_bits(cluster, block_m, bn, monkeypatch):
    """128- and 256-row tiles, single CTAs and CTA pairs, narrow and wide tiles: the K order per output element is the same."""
    m, n, k = 1024, 1200, 1536
    qa, sfa, qb, sfb = _quantise(m, n, k, 77)
    base = _run(qa, sfa, qb, sfb)
    monkeypatch.setenv("DG_FORCE_CLUSTER", str(cluster))
    monkeypatch.setenv("DG_FORCE_BLOCK_M", str(block_m))
    monkeypatch.setenv("DG_FORCE_BLOCK_N", str(bn))
    d = _run(qa, sfa, qb, sfb)
    assert torch.equal(d.view(torch.int16), base.view(torch.int16))
    ref = oracle.dequant_gemm_nt(qa, sfa, qb, sfb, 32, 32, True, True)
    assert oracle.calc_diff(d.float().cpu().numpy(), oracle.bf16_round(ref)) < 1e-5


@pytest.mark.parametrize("m", [1, 16, 64, 128])
def test_mxf4_few_rows_sliced_and_swapped_forms(m):
    """Decode-sized FP4 x FP4 GEMMs go through the K-sliced and operand-swapped forms like the FP8 ones."""
    n, k = 2112, 7168
    qa, sfa, qb, sfb = _quantise(m, n, k, 91)
    d = _run(qa, sfa, qb, sfb)
    ref = oracle.dequant_gemm_nt(qa, sfa, qb, sfb, 32, 32, True, True)
    out = d.float().cpu().numpy()
    assert oracle.calc_diff(out, oracle.bf16_round(ref)) < 1e-5, diff_report(out, ref)


def test_mxf4_grouped_contiguous_and_masked():
    g, n, k = 4, 512, 1280
    mt, actual, aligned, layout = oracle.make_contiguous_layout(g, 200, 128, actual_ms=[130, 256, 0, 77])
    a = seeded_bf16((mt, k), 5)
    a[layout < 0] = 0
    b = seeded_bf16((g, n, k), 6)
    qa, sfa = oracle.per_token_cast_to_fp4(a, True, 32)
    qs = [oracle.per_token_cast_to_fp4(b[i], True, 32) for i in range(g)]
    qb, sfb = np.stack([q for q, _ in qs]), np.stack([s for _, s in qs])
    d = torch.full((mt, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    dg.reset_kernel_status()
    dg.m_grouped_fp4_gemm_nt_contiguous((fp4_cuda(qa), packed_sf_cuda(sfa)), (fp4_cuda(qb), packed_sf_cuda(sfb)), d,
                                        torch.from_numpy(layout).cuda(), recipe_a=(1, 32), recipe_b=(1, 32))
    assert dg.kernel_status() == 0
    out = d.float().cpu().numpy()
    start = 0
    for i, (rows, padded) in enumerate(zip(actual, aligned)):
        if rows:
            want = oracle.dequant_gemm_nt(qa[start:start + rows], sfa[start:start + rows], qb[i], sfb[i], 32, 32, True, True)
            assert oracle.calc_diff(out[start:start + rows], oracle.bf16_round(want)) < 1e-5, i
        start += padded
    # masked: rows beyond masked_m untouched
    counts, max_m = (45, 128, 0, 83), 128
    am = seeded_bf16((g * max_m, k), 7)
    qam, sfam = oracle.per_token_cast_to_fp4(am, True, 32)
    qam, sfam = qam.reshape(g, max_m, -1), sfam.reshape(g, max_m, -1)
    dm = torch.full((g, max_m, n), -7.0, dtype=torch.bfloat16, device="cuda")
    dg.m_grouped_fp4_gemm_nt_masked((fp4_cuda(qam), packed_sf_cuda(sfam)), (fp4_cuda(qb), packed_sf_cuda(sfb)), dm,
                                    torch.tensor(counts, dtype=torch.int, device="cuda"), 64, recipe_a=(1, 32), recipe_b=(1, 32))
    assert dg.kernel_status() == 0
    outm = dm.float().cpu().numpy()
    for i, rows in enumerate(counts):
        if rows:
            want = oracle.dequant_gemm_nt(qam[i, :rows], sfam[i, :rows], qb[i], sfb[i], 32, 32, True, True)
            assert oracle.calc_diff(outm[i, :rows], oracle.bf16_round(want)) < 1e-5, i
        assert (outm[i, rows:] == -7.0).all()

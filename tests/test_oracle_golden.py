"""Pins the numpy oracle against outputs of the reference's own Python (tests/golden)."""
import numpy as np
import pytest

import oracle


def bits_to_f32(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def test_bf16_round_matches_bits(golden):
    x = bits_to_f32(golden["quant_x_bits"])
    assert np.array_equal(oracle.bf16_round(x), x)
    y = np.float32([1.00390625, 1.01171875, -3.0000001, 1e-40])
    r = oracle.bf16_round(y)
    assert (r.view(np.uint32) & 0xFFFF == 0).all()


def test_ceil_to_ue8m0(golden):
    assert np.array_equal(oracle.ceil_to_ue8m0(golden["ceil_in"]).view(np.int32), golden["ceil_out"].view(np.int32))


def test_e4m3_codec(golden):
    enc = oracle.e4m3_encode(golden["e4m3_sweep_in"])
    assert np.array_equal(enc, golden["e4m3_sweep_out"])
    dec = oracle.e4m3_decode(np.arange(256, dtype=np.uint8))
    ref = golden["e4m3_all_codes_value"]
    assert np.array_equal(np.isnan(dec), np.isnan(ref))
    assert np.array_equal(dec[~np.isnan(ref)], ref[~np.isnan(ref)])


@pytest.mark.parametrize("gran_k", [32, 128])
@pytest.mark.parametrize("ue", [False, True])
def test_per_token_cast_to_fp8(golden, gran_k, ue):
    x = bits_to_f32(golden["quant_x_bits"])
    q, sf = oracle.per_token_cast_to_fp8(x, use_ue8m0=ue, gran_k=gran_k)
    assert np.array_equal(q, golden[f"tok_fp8_g{gran_k}_ue{int(ue)}_q"])
    assert np.array_equal(sf.view(np.int32), golden[f"tok_fp8_g{gran_k}_ue{int(ue)}_sf"].view(np.int32))
    back = oracle.cast_back_from_fp8(q, sf, gran_k)
    assert np.array_equal(back.view(np.int32), golden[f"tok_fp8_g{gran_k}_ue{int(ue)}_back"].view(np.int32))
    if ue:
        _, psf = oracle.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=gran_k, use_packed_ue8m0=True)
        assert np.array_equal(psf, golden[f"tok_fp8_g{gran_k}_packed_sf"])
        assert np.array_equal(oracle.cast_back_from_fp8(q, psf, gran_k, use_packed_ue8m0=True)[:, :x.shape[1]], back)


@pytest.mark.parametrize("ue", [False, True])
def test_per_block_cast_to_fp8(golden, ue):
    x = bits_to_f32(golden["block_x_bits"])
    q, sf = oracle.per_block_cast_to_fp8(x, use_ue8m0=ue)
    assert np.array_equal(q, golden[f"blk_fp8_ue{int(ue)}_q"])
    assert np.array_equal(sf.view(np.int32), golden[f"blk_fp8_ue{int(ue)}_sf"].view(np.int32))


@pytest.mark.parametrize("gran_k", [32, 128])
def test_per_token_cast_to_fp4(golden, gran_k):
    x = bits_to_f32(golden["quant_x_bits"])
    q, sf = oracle.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=gran_k)
    assert np.array_equal(q, golden[f"tok_fp4_g{gran_k}_q"])
    assert np.array_equal(sf.view(np.int32), golden[f"tok_fp4_g{gran_k}_sf"].view(np.int32))
    back = oracle.cast_back_from_fp4(q, sf, gran_k)
    assert np.array_equal(back.view(np.int32), golden[f"tok_fp4_g{gran_k}_back"].view(np.int32))
    q0, sf0 = oracle.per_token_cast_to_fp4(x, use_ue8m0=False, gran_k=gran_k)
    assert np.array_equal(q0, golden[f"tok_fp4_g{gran_k}_ue0_q"])
    assert np.array_equal(sf0.view(np.int32), golden[f"tok_fp4_g{gran_k}_ue0_sf"].view(np.int32))
    _, psf = oracle.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=gran_k, use_packed_ue8m0=True)
    assert np.array_equal(psf, golden[f"tok_fp4_g{gran_k}_packed_sf"])


def test_fp4_helpers(golden):
    x = bits_to_f32(golden["quant_x_bits"])[:36]
    q, _ = oracle.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=32)
    assert np.array_equal(oracle.transpose_packed_fp4(q), golden["fp4_transposed"])
    assert np.array_equal(oracle.fp4_to_e4m3_bytes(q), golden["fp4_as_e4m3"])
    # E4M3 re-encoding represents every E2M1 value exactly (tests/test_fp8_fp4.py:95-100)
    assert np.array_equal(oracle.e4m3_decode(oracle.fp4_to_e4m3_bytes(q)),
                          oracle.cast_back_from_fp4(q, np.ones((36, 1), np.float32), gran_k=10 ** 9))


def test_packed_layout_values_shape_strides_storage(golden):
    for tag in golden["layout_cases"]:
        sf = golden[f"{tag}_sf"]
        view, strides = oracle.mn_major_tma_aligned_packed_ue8m0(sf)
        ref = golden[f"{tag}_packed"]
        assert view.shape == ref.shape, tag
        assert np.array_equal(view, ref), tag
        assert tuple(strides) == tuple(golden[f"{tag}_strides"]), tag
        # numpy's own byte strides describe the same memory layout
        assert all(vs // 4 == st for vs, st, n in zip(view.strides, strides, view.shape) if n > 1), tag
        storage = golden[f"{tag}_storage"]
        flat = np.lib.stride_tricks.as_strided(view, (storage.size,), (4,))
        assert np.array_equal(flat, storage), tag
        assert not (np.ascontiguousarray(view).view(np.uint8) == 0xFF).any()
        sf_k = sf.shape[-1]
        assert np.array_equal(oracle.unpack_mn_major_packed_ue8m0(view, sf_k).view(np.int32), sf.view(np.int32))


def test_dequant_gemm_and_calc_diff(golden):
    a = bits_to_f32(golden["gemm_a_bits"])
    b = bits_to_f32(golden["gemm_b_bits"])
    qa, sfa = oracle.per_token_cast_to_fp8(a, True, 128)
    qb, sfb = oracle.per_block_cast_to_fp8(b, True)
    sfb_rows = oracle.broadcast_sf_along_mn(sfb, 80, 128)
    d = oracle.dequant_gemm_nt(qa, sfa, qb, sfb_rows)
    ref = golden["gemm_fp8_ref_dequant"]
    assert oracle.calc_diff(d, ref) < 1e-12
    assert np.allclose(d, ref, rtol=1e-5, atol=1e-4)
    unq = a.astype(np.float64) @ b.astype(np.float64).T
    assert abs(oracle.calc_diff(unq, d) - float(golden["gemm_fp8_diff_unq_vs_deq"])) < 1e-7
    qb4, sfb4 = oracle.per_token_cast_to_fp4(b, True, 32)
    d4 = oracle.dequant_gemm_nt(qa, sfa, qb4, sfb4, 128, 32, False, True)
    assert oracle.calc_diff(d4, golden["gemm_fp4_ref_dequant"]) < 1e-12
    assert abs(oracle.calc_diff(unq, d4) - float(golden["gemm_fp4_diff_unq_vs_deq"])) < 1e-7
    assert oracle.calc_diff(np.zeros(4), np.zeros(4)) == float(golden["calc_diff_zero"]) == 0.0
    assert abs(oracle.calc_diff(oracle.bf16_round(ref), ref) - float(golden["calc_diff_bf16"])) < 1e-12


def test_grouped_refs_consistent():
    rng = np.random.default_rng(0)
    m, actual, aligned, layout = oracle.make_contiguous_layout(3, 40, 16, seed=1)
    assert m == sum(aligned) and (layout[:actual[0]] == 0).all() and (layout[actual[0]:aligned[0]] == -1).all()
    a = oracle.bf16_round(rng.standard_normal((m, 256)).astype(np.float32))
    a[layout < 0] = 0
    b = oracle.bf16_round(rng.standard_normal((3, 24, 256)).astype(np.float32))
    qa, sfa = oracle.per_token_cast_to_fp8(a, True, 128)
    qb = np.stack([oracle.per_token_cast_to_fp8(b[i], True, 128)[0] for i in range(3)])
    sfb = np.stack([oracle.per_token_cast_to_fp8(b[i], True, 128)[1] for i in range(3)])
    d = oracle.m_grouped_contiguous_ref(qa, sfa, qb, sfb, aligned)
    assert not np.isnan(d).any() and (d[layout < 0] == 0).all()
    dm = oracle.m_grouped_masked_ref(qa[:aligned[0]][None], sfa[:aligned[0]][None], qb[:1], sfb[:1], [actual[0]])
    assert np.array_equal(dm[0, :actual[0]], d[:actual[0]]) and np.isnan(dm[0, actual[0]:]).all()

"""CPU-side checks of the C-ABI library: exported symbols, settings, argument validation, heuristics
invariants, the host model of the tile scheduler, and the JIT runtime's compile / cache / error paths.
No compute call is made; no GPU is needed."""
import ctypes as C
import os
import re
import shutil

import numpy as np
import pytest

import deepgemm_amd_b200 as dg
from deepgemm_amd_b200 import _lib
from deepgemm_amd_b200._lib import GemmArgs, GemmConfig, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "deepgemm_b200.h")).read()
    declared = set(re.findall(r"DG_API\s+[\w\s\*]+?\b(dg_\w+)\s*\(", header))
    assert len(declared) >= 25
    raw = C.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(raw, name), f"{name} is declared in include/deepgemm_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)


def test_settings_defaults_and_setters():
    # defaults of the reference: alignment 128, theoretical 256 on sm_100, tc_util 100
    assert dg.get_mk_alignment_for_contiguous_layout() == 128
    assert dg.get_theoretical_mk_alignment_for_contiguous_layout() == 256
    assert dg.get_theoretical_mk_alignment_for_contiguous_layout(64) == 256
    assert dg.get_tc_util() == 100 and dg.get_pdl() is False
    dg.set_mk_alignment_for_contiguous_layout(256)
    assert dg.get_m_alignment_for_contiguous_layout() == 256 == dg.get_k_alignment_for_contiguous_layout()
    dg.set_mk_alignment_for_contiguous_layout(128)
    assert dg.get_num_sms() == 148            # no device here: B200's SM count
    with pytest.raises(RuntimeError, match="Assertion error"):
        dg.set_num_sms(147)                   # must be even (heuristics/config.hpp:60)
    dg.set_num_sms(132)
    assert dg.get_num_sms() == 132
    lib.dg_set_num_sms  # restore
    _lib.check(lib.dg_set_num_sms(148))
    dg.set_tc_util(80)
    assert dg.get_tc_util() == 80
    dg.set_tc_util(100)
    dg.set_pdl(True)
    assert dg.get_pdl() is True
    dg.set_pdl(False)
    assert dg.get_tma_aligned_size(4097, 4) == 4100 and dg.get_tma_aligned_size(129, 1) == 144
    with pytest.raises(RuntimeError):
        dg.get_tma_aligned_size(10, 3)


def _args(m=256, n=512, k=1024, groups=1, **kw):
    a = GemmArgs()
    a.m, a.n, a.k, a.num_groups = m, n, k, groups
    a.a_dtype, a.b_dtype, a.d_dtype = _lib.DG_FP8_E4M3, _lib.DG_FP8_E4M3, _lib.DG_BF16
    a.lda, a.ldb, a.ldd = k, k, n
    a.sfa_pitch, a.sfb_pitch = (m + 3) // 4 * 4, (n + 3) // 4 * 4
    a.gran_k_a = a.gran_k_b = 128
    a.expected_m = 64
    for key, v in kw.items():
        setattr(a, key, v)
    return a


@pytest.mark.parametrize("kw,kind,pattern", [
    (dict(gran_k_a=64), 0, "gran_k_a == 32"),
    (dict(d_dtype=_lib.DG_FP8_E4M3), 0, "sfd_pitch >= align_up"),                       # quantised D needs its scale tensor
    (dict(d_dtype=_lib.DG_FP8_E4M3, sfd_pitch=256, accumulate=1), 0, "!a->accumulate"),  # and never accumulates
    (dict(d_dtype=_lib.DG_FP8_E4M3, num_groups=2), 1, "d_dtype == DG_BF16"),
    (dict(ldd=500), 0, "ldd >= a->n"),
    (dict(n=513, ldd=513), 0, "% 16 == 0"),
    (dict(sfa_pitch=254), 0, "sfa_pitch"),
    (dict(sfb_pitch=514), 0, "sfb_pitch % 4"),
    (dict(lda=1000), 0, "lda >= k_bytes_a"),
    (dict(num_groups=2), 0, "num_groups == 1"),
    (dict(d_dtype=_lib.DG_FP32, num_groups=2), 1, "d_dtype == DG_BF16"),
    (dict(m=200, num_groups=2), 1, "m % 128 == 0"),
    (dict(num_groups=2, expected_m=0), 2, "expected_m > 0"),
    (dict(num_groups=2, accumulate=1), 2, "!a->accumulate"),
])
def test_argument_validation_fails_like_the_reference_asserts(kw, kind, pattern):
    cfg = GemmConfig()
    rc = lib.dg_get_gemm_config(kind, C.byref(_args(**kw)), C.byref(cfg))
    assert rc == 1, _lib.last_error()
    assert _lib.last_error().startswith("Assertion error (") and pattern in _lib.last_error(), _lib.last_error()


def test_unsupported_combinations_say_so():
    cfg = GemmConfig()
    rc = lib.dg_get_gemm_config(0, C.byref(_args(a_dtype=_lib.DG_FP4_E2M1_X2, major_a=_lib.DG_MAJOR_MN, lda=256)), C.byref(cfg))
    assert rc == 4 and "must be K-major" in _lib.last_error()
    # an MN-major packed FP4 B is built for FP8 x FP4 with whole 128-column blocks of N; FP4 x FP4 is K-major only
    rc = lib.dg_get_gemm_config(0, C.byref(_args(b_dtype=_lib.DG_FP4_E2M1_X2, major_b=_lib.DG_MAJOR_MN, n=704, ldb=352, gran_k_b=32)), C.byref(cfg))
    assert rc == 1 and "n % 128 == 0" in _lib.last_error()
    rc = lib.dg_get_gemm_config(0, C.byref(_args(b_dtype=_lib.DG_FP4_E2M1_X2, major_b=_lib.DG_MAJOR_MN, n=768, ldb=384, gran_k_b=32)), C.byref(cfg))
    assert rc == 0 and cfg.block_n == 128, _lib.last_error()
    rc = lib.dg_get_gemm_config(0, C.byref(_args(a_dtype=_lib.DG_FP4_E2M1_X2, b_dtype=_lib.DG_FP4_E2M1_X2, major_b=_lib.DG_MAJOR_MN, n=768,
                                                 lda=128, ldb=384, gran_k_a=32, gran_k_b=32)), C.byref(cfg))
    assert rc == 4 and "K-major" in _lib.last_error()


SHAPES = [(m, n, k) for m in (1, 64, 128, 129, 4096) for (n, k) in
          ((2112, 7168), (576, 7168), (24576, 1536), (32768, 512), (7168, 16384), (4096, 7168), (7168, 2048), (16, 128))]


@pytest.mark.parametrize("fp32", [False, True])
def test_heuristics_invariants(fp32):
    for m, n, k in SHAPES:
        cfg = dg.get_gemm_config(0, m, n, k, d_is_fp32=fp32)
        assert cfg["block_m"] in (128, 256) and cfg["block_k"] in (128, 256)
        # stages of 256 elements of K: only the swapped form's 16- and 32-column tiles, where a work item has 12 K-blocks or more
        if cfg["block_k"] == 256:
            assert cfg["swap_ab"] and m <= 32 and k % 256 == 0 and cfg["num_stages"] >= 4
            assert (cfg["kb_per_split"] if cfg["num_splits"] > 1 else -(-k // 128)) >= 12
        assert cfg["block_m"] == 128 or (m > 128 and cfg["num_splits"] == 1)
        # CTA pairs (one 256- or 512-row tile per pair) only for large dense GEMMs, never sliced along K
        assert cfg["cluster_size"] == 1 or (cfg["cluster_size"] == 2 and m >= 1024 and cfg["num_splits"] == 1 and cfg["num_ctas"] % 2 == 0)
        assert cfg["block_n"] % 16 == 0 and 16 <= cfg["block_n"] <= 240
        assert cfg["smem_bytes"] <= 232448, (m, n, k, cfg)
        assert cfg["tmem_cols"] in (32, 64, 128, 256, 512) and 2 * cfg["block_n"] + cfg["block_m"] // 32 + 4 * ((cfg["block_n"] + 127) // 128) <= cfg["tmem_cols"]
        assert 2 <= cfg["num_stages"] <= 32
        assert 1 <= cfg["num_ctas"] <= 148
        rows, cols = (n, m) if cfg["swap_ab"] else (m, n)        # operands swapped: the kernel's rows are the caller's N
        if cfg["swap_ab"]:
            # few rows only; one tile column as wide as the caller's M; K slices, if any, inside a cluster
            assert m <= 128 and cfg["block_m"] == 128 and cfg["block_n"] == -(-m // 16) * 16
            assert cfg["num_splits"] == 1 or cfg["split_in_cluster"]
        assert cfg["num_tiles"] == -(-rows // (cfg["block_m"] * cfg["cluster_size"])) * -(-cols // cfg["block_n"]) * cfg["num_splits"]
        kb = -(-k // 128)
        if cfg["num_splits"] > 1:
            # slices start on a packed scale word (4 K-blocks), cover K exactly once, and none is empty
            assert cfg["kb_per_split"] % 4 == 0 and cfg["kb_per_split"] >= 8
            assert (cfg["num_splits"] - 1) * cfg["kb_per_split"] < kb <= cfg["num_splits"] * cfg["kb_per_split"]
            assert cfg["num_tiles"] <= 148
            if cfg["split_in_cluster"]:
                # the slices of a tile are one thread-block cluster: portable size, one CTA per slice, and a parked FP32
                # accumulator fits the pipeline stages it overwrites
                assert cfg["num_splits"] <= 8 and cfg["num_ctas"] == cfg["num_tiles"] and cfg["cluster_size"] == 1
                # (what it receives: the slices of the 8-column chunks it owns; the area starts at the D staging buffers)
                recv = cfg["num_splits"] * -(-(cfg["block_n"] // 8) // cfg["num_splits"]) * 8 * 128 * 4
                assert recv <= cfg["store_buffers"] * 16384 + cfg["num_stages"] * (cfg["a_rows"] + cfg["block_n"]) * cfg["block_k"]
        else:
            assert cfg["kb_per_split"] == kb and not cfg["split_in_cluster"]
    for kind, groups in ((1, 32), (2, 16)):
        cfg = dg.get_gemm_config(kind, 256 if kind == 2 else 32 * 1024, 4096, 7168, num_groups=groups, expected_m=64)
        assert cfg["smem_bytes"] <= 232448 and cfg["num_ctas"] <= 148


@pytest.mark.parametrize("shape", [(8, 128, 128), (1, 16, 128), (16, 2112, 7168), (33, 1000, 512), (40, 128, 128), (64, 16, 128),
                                   (64, 7168, 2048), (48, 264, 1152), (64, 24576, 1536)])
def test_shortened_a_stages_keep_the_mma_read_inside_shared_memory(shape, monkeypatch):
    """A dense GEMM with at most 64 rows stages 16, 32 or 64 rows of A, but the MMA of every stage still reads 128 rows
    from the stage's base: the dynamic shared memory the kernel is launched with must reach the end of that read for the
    last stage too (small shapes have little behind the A stages)."""
    m, n, k = shape
    for swap in ("-1", "1"):
        monkeypatch.setenv("DG_FORCE_SWAP_AB", swap)
        cfg = dg.get_gemm_config(0, m, n, k)
        rows = n if cfg["swap_ab"] else m
        assert cfg["a_rows"] == (128 if rows > 64 else 16 if rows <= 16 else 32 if rows <= 32 else 64), cfg
        a_base = cfg["store_buffers"] * 16384                       # the A stages follow the D staging buffers
        assert cfg["smem_bytes"] >= a_base + (cfg["num_stages"] - 1) * cfg["a_rows"] * cfg["block_k"] + 128 * cfg["block_k"], cfg
        assert cfg["smem_bytes"] <= 232448
    monkeypatch.setenv("DG_FORCE_A_ROWS", "128")
    assert dg.get_gemm_config(0, m, n, k)["a_rows"] == 128


def test_256_element_k_stages(monkeypatch):
    """Stages of 256 elements of K: a stage row is two 128-byte swizzle atoms side by side, [atom][row][128 bytes].  Served for
    dense K-major FP8 GEMMs with one scale per 128 elements and K a multiple of 256, by 128-row CTAs; K may be sliced
    (slices stay multiples of 512 elements) and the operands swapped."""
    monkeypatch.setenv("DG_FORCE_BLOCK_K", "256")
    for m, n, k in [(128, 2112, 7168), (16, 2112, 7168), (64, 24576, 1536), (4096, 4096, 7168), (32, 4096, 512)]:
        cfg = dg.get_gemm_config(0, m, n, k)
        assert cfg["block_k"] == 256 and cfg["block_m"] == 128 and cfg["cluster_size"] == 1, cfg
        assert 2 <= cfg["num_stages"] and cfg["smem_bytes"] <= 232448
        # the MMAs on the second atom of the last stage read 128 rows of 128 bytes, starting one atom into the stage
        rows, a_base = cfg["a_rows"], cfg["store_buffers"] * 16384
        assert cfg["smem_bytes"] >= a_base + (cfg["num_stages"] - 1) * rows * 256 + rows * 128 + 128 * 128, cfg
        assert cfg["num_splits"] == 1 or cfg["kb_per_split"] % 4 == 0
    assert dg.get_gemm_config(0, 16, 2112, 7168)["swap_ab"] == 1
    monkeypatch.delenv("DG_FORCE_BLOCK_K")
    # without the request: chosen for the swapped form's narrow tiles when a work item is 12 K-blocks or longer
    assert [dg.get_gemm_config(0, m, n, k)["block_k"] for m, n, k in
            [(16, 2112, 7168), (32, 4096, 7168), (8, 24576, 1536), (16, 7168, 2048), (16, 32768, 512), (16, 4096, 7168 + 128), (64, 4096, 7168)]] == \
           [256, 256, 256, 128, 128, 128, 128]
    assert dg.get_gemm_config(0, 16, 4096, 7168, b_is_fp4=True, gran_k_b=32)["block_k"] == 128
    monkeypatch.setenv("DG_FORCE_BLOCK_K", "256")
    monkeypatch.setenv("DG_FORCE_SWAP_AB", "-1")
    for m, n, k in [(16, 2112, 2048), (32, 384, 512), (8, 128, 256)]:
        cfg = dg.get_gemm_config(0, m, n, k)
        rows, a_base = cfg["a_rows"], cfg["store_buffers"] * 16384
        assert cfg["block_k"] == 256 and rows == (16 if m <= 16 else 32), cfg
        assert cfg["smem_bytes"] >= a_base + (cfg["num_stages"] - 1) * rows * 256 + rows * 128 + 128 * 128, cfg
    monkeypatch.delenv("DG_FORCE_SWAP_AB")
    for kw in (dict(kind=0, m=128, n=2112, k=7168 + 128), dict(kind=0, m=128, n=2112, k=7168, b_is_fp4=True, gran_k_b=32),
               dict(kind=1, m=4096, n=4096, k=7168, num_groups=4)):
        with pytest.raises(RuntimeError, match="no tile configuration"):
            dg.get_gemm_config(**kw)


def test_operand_swap_can_be_forced_and_forbidden(monkeypatch):
    """DG_FORCE_SWAP_AB: 1 = swap whenever the form applies (dense K-major FP8, M <= 128, no accumulation), -1 = never."""
    monkeypatch.setenv("DG_FORCE_SWAP_AB", "1")
    assert dg.get_gemm_config(0, 16, 4096, 7168)["swap_ab"] == 1
    assert dg.get_gemm_config(0, 128, 4096, 7168)["swap_ab"] == 1           # up to 128 rows on request
    assert dg.get_gemm_config(0, 129, 4096, 7168)["swap_ab"] == 0           # too many rows
    assert dg.get_gemm_config(0, 16, 4096, 7168, b_is_fp4=True, gran_k_b=32)["swap_ab"] == 1     # an FP4 weight becomes the A side
    assert dg.get_gemm_config(1, 4096, 4096, 7168, num_groups=4)["swap_ab"] == 0
    monkeypatch.setenv("DG_FORCE_SWAP_AB", "-1")
    assert dg.get_gemm_config(0, 16, 4096, 7168)["swap_ab"] == 0
    monkeypatch.delenv("DG_FORCE_SWAP_AB")
    assert dg.get_gemm_config(0, 16, 4096, 7168)["swap_ab"] == 1            # chosen by cost up to 64 rows
    assert dg.get_gemm_config(0, 64, 4096, 7168)["swap_ab"] == 1            # (here: modelled 19 % cheaper)
    assert dg.get_gemm_config(0, 64, 24576, 1536)["swap_ab"] == 0           # (here: modelled dearer)
    assert dg.get_gemm_config(0, 65, 4096, 7168)["swap_ab"] == 0            # on request only beyond


def test_second_staging_buffer_is_given_up_only_for_a_third_stage(monkeypatch):
    """(One CTA per tile.)  MN-major operands are staged as whole 128-byte atoms (a 240-column B tile takes 32 KB), so 256 x 240 tiles fit two
    stages beside two D staging buffers per epilogue warpgroup and three beside one; K-major tiles fit three either way."""
    monkeypatch.setenv("DG_FORCE_CLUSTER", "1")
    cfg = GemmConfig()
    _lib.check(lib.dg_get_gemm_config(0, C.byref(_args(m=4096, n=4096, k=7168, lda=7168, ldb=7168, ldd=4096)), C.byref(cfg)))
    assert (cfg.block_m, cfg.num_stages, cfg.store_buffers) == (256, 3, 2)
    _lib.check(lib.dg_get_gemm_config(0, C.byref(_args(m=4096, n=4096, k=7168, lda=7168, ldb=4096, ldd=4096, major_b=_lib.DG_MAJOR_MN)), C.byref(cfg)))
    assert (cfg.block_m, cfg.num_stages, cfg.store_buffers) == (256, 3, 1) and cfg.smem_bytes <= 232448


def test_split_reduction_mode_can_be_forced(monkeypatch):
    """DG_FORCE_SPLIT_CLUSTER: 1 = slices reduced inside a cluster, -1 = through the workspace and a second kernel."""
    m, n, k = 128, 2112, 7168
    monkeypatch.setenv("DG_FORCE_SPLIT_CLUSTER", "1")
    cfg = dg.get_gemm_config(0, m, n, k)
    assert cfg["num_splits"] > 1 and cfg["split_in_cluster"] == 1 and cfg["num_splits"] <= 8
    monkeypatch.setenv("DG_FORCE_SPLIT_CLUSTER", "-1")
    cfg = dg.get_gemm_config(0, m, n, k)
    assert cfg["num_splits"] > 1 and cfg["split_in_cluster"] == 0
    monkeypatch.setenv("DG_FORCE_SPLIT_K", "1")
    cfg = dg.get_gemm_config(0, m, n, k)
    assert cfg["num_splits"] == 1 and cfg["split_in_cluster"] == 0


def _enumerate(kind, bn, rg, m, n, groups, layout, num_ctas):
    tiles = []
    lay = np.ascontiguousarray(layout, dtype=np.int32) if layout is not None else None
    ptr = lay.ctypes.data_as(C.c_void_p) if lay is not None else None
    for cta in range(num_ctas):
        buf = (C.c_uint32 * (4 * 8192))()
        cnt = lib.dg_enumerate_tiles(kind, bn, rg, m, n, groups, ptr, cta, num_ctas, buf, 8192)
        assert 0 <= cnt <= 8192
        tiles += [tuple(buf[4 * i: 4 * i + 4]) + (cta, i) for i in range(cnt)]
    return tiles


@pytest.mark.parametrize("m,n,bn,rg,ctas", [(4096, 4096, 240, 16, 148), (129, 2112, 16, 16, 132), (1, 16, 16, 16, 1),
                                            (1000, 1000, 64, 4, 7), (4096, 7168, 224, 8, 148)])
def test_scheduler_dense_visits_every_tile_once(m, n, bn, rg, ctas):
    tiles = _enumerate(0, bn, rg, m, n, 1, None, ctas)
    seen = sorted((t[0], t[1]) for t in tiles)
    want = sorted((i, j) for i in range(-(-m // 128)) for j in range(-(-n // bn)))
    assert seen == want
    assert all(t[2] == 0 and t[3] == 128 for t in tiles)
    # static round-robin: CTA c's i-th tile is global tile i * ctas + c, so loads are balanced to within one tile
    per_cta = np.bincount([t[4] for t in tiles], minlength=ctas)
    assert per_cta.max() - per_cta.min() <= 1


def test_scheduler_contiguous_maps_row_blocks_to_experts():
    import oracle
    m, actual, aligned, layout = oracle.make_contiguous_layout(6, 300, 128, seed=2)
    tiles = _enumerate(1, 128, 16, m, 512, 6, layout, 20)
    assert sorted((t[0], t[1]) for t in tiles) == sorted((i, j) for i in range(m // 128) for j in range(4))
    for mb, nb, group, valid, _, _ in tiles:
        assert group == max(0, int(layout[mb * 128])) and valid == 128
    # with alignment 256 every second block may start on padding (-1): it still belongs to the expert before it
    m2, _, aligned2, layout2 = oracle.make_contiguous_layout(3, 100, 256, actual_ms=[100, 0, 300])
    tiles2 = _enumerate(1, 64, 16, m2, 128, 3, layout2, 3)
    blocks = {t[0]: t[2] for t in tiles2}
    assert blocks[0] == 0 and blocks[1] == 0 and blocks[2] == 2 and blocks[3] == 2 and blocks[4] == 2


@pytest.mark.parametrize("actual_ms,alignment", [((100, 150, 114), 128), ((130, 0, 256, 77, 300), 128), ((1, 1, 1), 256), ((0, 0), 128)])
def test_scheduler_prefix_sum_layout_walks_each_group_from_its_aligned_start(actual_ms, alignment):
    import oracle
    import deepgemm_amd_b200 as dg
    dg.set_mk_alignment_for_contiguous_layout(alignment)
    try:
        m, starts, ends = oracle.make_psum_layout(actual_ms, alignment)
        n, bn = 1000, 112
        tiles = _enumerate(3, bn, 16, max(m, 1), n, len(actual_ms), ends, 37)
        want = {}
        for g, (s0, e) in enumerate(zip(starts, ends)):
            for mb in range(-(-(int(e) - s0) // 128)):
                for nb in range(-(-n // bn)):
                    want[(g, s0 // 128 + mb, nb)] = min(128, int(e) - s0 - mb * 128)
        got = {(t[2], t[0], t[1]): t[3] for t in tiles}
        assert len(tiles) == len(got) == len(want) and got == want
    finally:
        dg.set_mk_alignment_for_contiguous_layout(128)


def test_scheduler_k_grouped_and_batched_give_every_group_the_full_tile_grid():
    m, n, bn = 300, 1000, 112
    ks = (256, 0, 1024, 128)
    tiles = _enumerate(4, bn, 16, m, n, len(ks), ks, 37)
    want = {(g, mb, nb): k // 128 for g, k in enumerate(ks) for mb in range(3) for nb in range(9)}
    got = {(t[2], t[0], t[1]): t[3] for t in tiles}
    assert len(tiles) == len(got) == len(want) and got == want
    tiles = _enumerate(5, bn, 16, m, n, 5, None, 37)
    assert sorted((t[2], t[0], t[1]) for t in tiles) == sorted((b, mb, nb) for b in range(5) for mb in range(3) for nb in range(9))


@pytest.mark.parametrize("counts,max_m", [((45, 83, 0, 256, 129), 256), ((0, 0, 0), 128), ((300, 1), 256), ((64,) * 16, 256)])
def test_scheduler_masked_follows_device_counts(counts, max_m):
    n, bn = 4096, 240
    tiles = _enumerate(2, bn, 16, max_m, n, len(counts), counts, 148)
    want = {}
    for g, c in enumerate(counts):
        c = min(c, max_m)
        for mb in range(-(-c // 128)):
            for nb in range(-(-n // bn)):
                want[(g, mb, nb)] = min(128, c - mb * 128)
    got = {(t[2], t[0], t[1]): t[3] for t in tiles}
    assert len(tiles) == len(got) == len(want) and got == want      # each tile exactly once, none beyond masked_m


TRIVIAL = 'extern "C" __global__ void k(int* p) { if (p) *p = %d; }\n'


def test_jit_compile_cache_and_errors(tmp_path, monkeypatch):
    monkeypatch.setenv("DG_JIT_CACHE_DIR", str(tmp_path))
    h1, h2, h3 = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _lib.check(lib.dg_jit_compile(b"trivial", b"k", (TRIVIAL % 1).encode(), b"", C.byref(h1)))
    path = lib.dg_jit_kernel_path(h1).decode()
    assert path.startswith(str(tmp_path)) and os.path.getsize(path) > 0
    assert not [d for d in os.listdir(tmp_path) if d.startswith("tmp.")]       # published by rename, no leftovers
    mtime = os.path.getmtime(path)
    _lib.check(lib.dg_jit_compile(b"trivial", b"k", (TRIVIAL % 1).encode(), b"", C.byref(h2)))
    assert h1.value == h2.value and os.path.getmtime(path) == mtime             # cache hit
    _lib.check(lib.dg_jit_compile(b"trivial", b"k", (TRIVIAL % 2).encode(), b"", C.byref(h3)))
    assert lib.dg_jit_kernel_path(h3).decode() != path                          # different source, different key
    bad = C.c_void_p()
    rc = lib.dg_jit_compile(b"broken", b"k", b"this is not CUDA", b"", C.byref(bad))
    assert rc == 3 and "nvcc failed" in _lib.last_error() and "error" in _lib.last_error()
    assert not [d for d in os.listdir(tmp_path) if d.startswith("tmp.")]
    # launching needs a driver: without one the call fails cleanly instead of crashing
    import torch
    if not torch.cuda.is_available():
        rc = lib.dg_jit_launch(h1, 1, 32, 1, 0, 0, None, None)
        assert rc == 2 and "driver" in _lib.last_error().lower()


def test_gemm_kernel_source_compiles_for_every_family(tmp_path, monkeypatch):
    monkeypatch.setenv("DG_JIT_CACHE_DIR", str(tmp_path))
    dg.precompile_gemm(0, 128, 2112, 7168)
    dg.precompile_gemm(0, 4096, 4096, 7168, d_is_fp32=True, accumulate=True)
    dg.precompile_gemm(1, 1024, 4096, 7168, num_groups=4)
    dg.precompile_gemm(2, 256, 4096, 7168, num_groups=16, expected_m=64)
    dg.precompile_gemm(0, 4096, 7168, 2048, b_is_fp4=True, gran_k_b=32)
    # kernels already shipped in the in-tree cache are found there; anything else lands in the override directory
    for d in os.listdir(tmp_path):
        assert d.startswith("kernel.gemm_fp8_fp4_") and os.path.getsize(tmp_path / d / "kernel.cubin") > 0

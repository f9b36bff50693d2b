"""The compiled Python binding (deepgemm_amd_b200/_C.so, csrc/python_binding.cpp): it loads without a GPU and words
its failures like the interpreter path; on a GPU it gives the same bits as the ctypes path for dense, m-grouped
contiguous and masked GEMMs, refuses what the ctypes path refuses, and costs the host a few microseconds per call."""
import time

import numpy as np
import pytest
import torch

import deepgemm_amd_b200 as dg
from deepgemm_amd_b200 import api


def test_binding_is_built_and_loaded():
    assert dg.HAS_COMPILED_BINDING, "deepgemm_amd_b200/_C.so is missing: run python deepgemm_amd_b200/build.py"
    for name in ("dense_nt", "m_grouped_contiguous", "m_grouped_masked"):
        assert callable(getattr(api._C, name))


def test_binding_words_its_failures_like_the_reference():
    t, sf = torch.zeros(4, 4), torch.zeros(4, 1, dtype=torch.int)
    with pytest.raises(RuntimeError, match=r"Assertion error \(deepgemm_amd_b200/csrc/python_binding.cpp:\d+\): t.is_cuda\(\)"):
        api._C.dense_nt((t, sf), (t, sf), t, None, None, None, None, False, None, None)
    with pytest.raises(RuntimeError, match="Assertion error"):
        api._C.m_grouped_masked((t, sf), (t, sf), t, sf, 1, None, None, None, False, None)
    with pytest.raises(RuntimeError, match="Assertion error"):
        api._C.m_grouped_contiguous((t, sf), (t, sf), t, sf, None, None, None, False, False, True, None, None)


def test_calls_the_binding_serves():
    """Packed scales with gran_mn == 1 and no epilogue object; everything else is handed back untouched (False), and the
    interpreter path words the error or runs the transform kernel."""
    t, i32, f32 = torch.zeros(4, 4), torch.zeros(4, 1, dtype=torch.int), torch.zeros(4, 1)

    def served(sfa=i32, sfb=i32, recipe=None, recipe_a=None, recipe_b=None, disable=False, epilogue=None, c=None):
        try:
            return api._C.dense_nt((t, sfa), (t, sfb), t, c, recipe, recipe_a, recipe_b, disable, None, epilogue)
        except RuntimeError as e:           # accepted: the first check then refuses the CPU tensors
            assert "t.is_cuda()" in str(e)
            return True

    assert served() and served(recipe=(1, 1, 32)) and served(recipe=[1, 1, 128]) and served(recipe_a=(1, 32), recipe_b=(1, 128))
    assert served(c=t)
    assert not served(sfa=f32) and not served(sfb=f32)
    assert not served(recipe=(1, 128, 128)) and not served(recipe=(1, 1, 64)) and not served(recipe=(1, 1))
    assert not served(recipe=(1, 1, 128), recipe_a=(1, 128), recipe_b=(1, 128))
    assert not served(recipe_a=(1, 128)) and not served(recipe_a=(1, 64), recipe_b=(1, 128)) and not served(recipe_a=(2, 128), recipe_b=(1, 128))
    assert not served(recipe="abc") and not served(disable=True) and not served(epilogue=dg.epilogue.Identity())
    assert not served(c=torch.zeros(4, 4))              # a C that is not D itself is copied by the general path


# ------------------------------------------------------------------------------------------------------------------
# GPU
# ------------------------------------------------------------------------------------------------------------------
def _dense_inputs(m, n, k, b_fp4=False, seed=0):
    from gpu_helpers import fp4_cuda, fp8_cuda, packed_sf_cuda, quantise_dense, seeded_bf16
    a, b = seeded_bf16((m, k), seed), seeded_bf16((n, k), seed + 1)
    qa, sfa, qb, sfb_rows, _ = quantise_dense(a, b, b_fp4)
    return (fp8_cuda(qa), packed_sf_cuda(sfa)), ((fp4_cuda(qb) if b_fp4 else fp8_cuda(qb)), packed_sf_cuda(sfb_rows))


def _both_paths(monkeypatch, call):
    """Runs `call(d)` through the compiled binding and through the ctypes path; returns both outputs."""
    outs = []
    for compiled in (True, False):
        with monkeypatch.context() as mp:
            if not compiled:
                mp.setattr(api, "_C", None)
                api._validated_calls().clear()
            outs.append(call())
    return outs


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k,b_fp4", [(128, 256, 512, False), (200, 2112, 1024, False), (64, 576, 1152, True), (1, 4096, 2048, False)])
@pytest.mark.parametrize("out_dtype,accumulate,alpha", [(torch.bfloat16, False, None), (torch.float, True, None), (torch.bfloat16, False, 0.5)])
def test_dense_same_bits_as_the_ctypes_path(m, n, k, b_fp4, out_dtype, accumulate, alpha, monkeypatch):
    a, b = _dense_inputs(m, n, k, b_fp4)
    gran_b = 32 if b_fp4 else 128

    def call():
        d = torch.full((m, n), 0.25 if accumulate else float("nan"), dtype=out_dtype, device="cuda")
        dg.fp8_fp4_gemm_nt(a, b, d, c=d if accumulate else None, recipe_a=(1, 128), recipe_b=(1, gran_b), alpha=alpha)
        return d

    compiled, interpreted = _both_paths(monkeypatch, call)
    assert not torch.isnan(compiled.float()).any()
    assert torch.equal(compiled.view(torch.uint8), interpreted.view(torch.uint8))


@pytest.mark.gpu
def test_grouped_same_bits_as_the_ctypes_path(monkeypatch):
    from gpu_helpers import fp8_cuda, packed_sf_cuda, seeded_bf16
    import oracle
    groups, n, k, rows = 3, 384, 640, [128, 0, 256]
    m = sum(rows)
    a = seeded_bf16((m, k), 7)
    b = seeded_bf16((groups, n, k), 8)
    qa, sfa = oracle.per_token_cast_to_fp8(a, True, 128)
    qb, sfb = zip(*[oracle.per_token_cast_to_fp8(b[g], True, 128) for g in range(groups)])
    a_t = (fp8_cuda(qa), packed_sf_cuda(sfa))
    b_t = (fp8_cuda(np.stack(qb)), packed_sf_cuda(np.stack(sfb)))
    layout = torch.tensor(np.repeat(np.arange(groups), rows).astype(np.int32), device="cuda")

    def contiguous():
        d = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_nt_contiguous(a_t, b_t, d, layout, recipe_a=(1, 128), recipe_b=(1, 128))
        return d

    compiled, interpreted = _both_paths(monkeypatch, contiguous)
    assert not torch.isnan(compiled.float()).any()
    assert torch.equal(compiled.view(torch.int16), interpreted.view(torch.int16))

    # masked: the same weights, A reshaped to [groups, max_m, k]
    max_m = 128
    am = seeded_bf16((groups, max_m, k), 9)
    qam, sfam = zip(*[oracle.per_token_cast_to_fp8(am[g], True, 128) for g in range(groups)])
    am_t = (fp8_cuda(np.stack(qam)), packed_sf_cuda(np.stack(sfam)))
    masked_m = torch.tensor([100, 0, 37], dtype=torch.int, device="cuda")

    def masked():
        d = torch.zeros((groups, max_m, n), dtype=torch.bfloat16, device="cuda")
        dg.m_grouped_fp8_fp4_gemm_nt_masked(am_t, b_t, d, masked_m, 64, recipe_a=(1, 128), recipe_b=(1, 128))
        return d

    compiled, interpreted = _both_paths(monkeypatch, masked)
    assert compiled[0, :100].float().abs().sum() > 0 and compiled[1].float().abs().sum() == 0
    assert torch.equal(compiled.view(torch.int16), interpreted.view(torch.int16))


@pytest.mark.gpu
def test_binding_refuses_what_the_ctypes_path_refuses():
    a, b = _dense_inputs(128, 256, 1024)          # two packed scale words per row
    d = torch.empty((128, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="m == m_ and n == n_ and k == k_"):
        dg.fp8_fp4_gemm_nt(a, b, d[:, :128], recipe_a=(1, 128), recipe_b=(1, 128))
    with pytest.raises(RuntimeError, match=r"t.stride\(-1\) == 1"):
        dg.fp8_fp4_gemm_nt(a, b, torch.empty((256, 128), dtype=torch.bfloat16, device="cuda").t(), recipe_a=(1, 128), recipe_b=(1, 128))
    with pytest.raises(RuntimeError, match=r"sf.size\(-1\) == ceil_div"):
        dg.fp8_fp4_gemm_nt(a, b, d, recipe_a=(1, 32), recipe_b=(1, 128))
    with pytest.raises(RuntimeError, match=r"d.scalar_type\(\) == torch::kBFloat16 or"):
        dg.fp8_fp4_gemm_nt(a, b, d.to(torch.half), recipe_a=(1, 128), recipe_b=(1, 128))
    with pytest.raises(RuntimeError, match="sf.stride"):
        dg.fp8_fp4_gemm_nt((a[0], a[1].contiguous()), b, d, recipe_a=(1, 128), recipe_b=(1, 128))
    # degenerate shapes return early, as the reference does (csrc/apis/gemm.hpp:17-53)
    dg.fp8_fp4_gemm_nt((a[0][:0], a[1][:0]), b, d[:0], recipe_a=(1, 128), recipe_b=(1, 128))


@pytest.mark.gpu
def test_host_cost_of_a_call(monkeypatch):
    """Host time of one enqueue (the call returns before the kernel runs).  The compiled binding has to stay well under
    the interpreter path; the absolute bound is loose because test boxes differ."""
    a, b = _dense_inputs(128, 2112, 7168)
    d = torch.empty((128, 2112), dtype=torch.bfloat16, device="cuda")

    def per_call_us(calls=2000):
        for _ in range(50):
            dg.fp8_fp4_gemm_nt(a, b, d, recipe_a=(1, 128), recipe_b=(1, 128))
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            # short bursts: the launch queue must not fill up, or the host would be timing the GPU
            t = 0.0
            for _ in range(calls // 100):
                t0 = time.perf_counter()
                for _ in range(100):
                    dg.fp8_fp4_gemm_nt(a, b, d, recipe_a=(1, 128), recipe_b=(1, 128))
                t += time.perf_counter() - t0
                torch.cuda.synchronize()
            best = min(best, t / calls * 1e6)
        return best

    compiled = per_call_us()
    with monkeypatch.context() as mp:
        mp.setattr(api, "_C", None)
        interpreted = per_call_us()
    print(f"host us per call: compiled binding {compiled:.2f}, ctypes path {interpreted:.2f}")
    assert compiled < interpreted
    assert compiled < 12.0

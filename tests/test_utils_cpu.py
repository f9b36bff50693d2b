"""Torch-side helpers of the reference's deep_gemm.utils / deep_gemm.testing that the GEMM path's callers use, checked on
the CPU against the numpy oracle."""
import os

import numpy as np
import pytest
import torch

import oracle
from deepgemm_amd_b200 import testing, utils


def _bf16(shape, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    return oracle.bf16_round((rng.standard_normal(shape) * scale).astype(np.float32))


@pytest.mark.parametrize("gran_k", [32, 128])
@pytest.mark.parametrize("ue8m0", [True, False])
def test_per_channel_cast_is_the_per_token_cast_of_the_transpose(gran_k, ue8m0):
    x = _bf16((256, 72), 5, 2.0)
    x[:, 3] = 0                                         # an all-zero channel: the 1e-4 clamp
    q, sf = utils.per_channel_cast_to_fp8(torch.from_numpy(x).bfloat16(), ue8m0, gran_k)
    want_q, want_sf = oracle.per_token_cast_to_fp8(np.ascontiguousarray(x.T), ue8m0, gran_k)
    assert q.shape == (256, 72) and sf.shape == (256 // gran_k, 72)
    assert np.array_equal(q.view(torch.uint8).numpy(), want_q.T)
    assert np.array_equal(sf.numpy(), want_sf.T)


def test_per_custom_dims_cast_keeps_one_scale_per_kept_index():
    x = _bf16((6, 5, 64), 6, 3.0)
    xt = torch.from_numpy(x).bfloat16()
    q, sf = utils.per_custom_dims_cast_to_fp8(xt, (0,), True)
    assert sf.shape == (6,) and q.shape == x.shape
    for i in range(6):
        want_q, want_sf = oracle.per_token_cast_to_fp8(x[i].reshape(1, -1), True, gran_k=x[i].size)
        assert sf[i].item() == want_sf[0, 0]
        assert np.array_equal(q[i].view(torch.uint8).numpy().reshape(1, -1), want_q)
    _, sf2 = utils.per_custom_dims_cast_to_fp8(xt, (0, 1), False)
    assert sf2.shape == (6, 5)
    assert torch.allclose(sf2, xt.abs().float().amax(dim=2).clamp(1e-4) / 448.0)


def test_transpose_packed_fp4_matches_oracle():
    x = _bf16((36, 64), 7, 2.0)
    q, _ = oracle.per_token_cast_to_fp4(x, True, 32)
    got = utils.transpose_packed_fp4(torch.from_numpy(q))
    assert got.dtype == torch.int8 and got.shape == (64, 18)
    assert np.array_equal(got.numpy(), oracle.transpose_packed_fp4(q))
    assert np.array_equal(utils.transpose_packed_fp4(got).numpy(), q)      # an involution


def test_test_script_decorators(monkeypatch, capsys):
    calls = []

    @testing.test_filter(lambda: False)
    def skipped():
        calls.append("skipped")

    @testing.test_filter(lambda: True)
    def kept():
        calls.append("kept")

    skipped(); kept()
    assert calls == ["kept"] and "Filtered by" in capsys.readouterr().out

    monkeypatch.setenv("DG_SOME_SETTING", "7")

    @testing.ignore_env("DG_SOME_SETTING", lambda: True)
    def without():
        return os.environ.get("DG_SOME_SETTING")

    @testing.ignore_env("DG_SOME_SETTING", lambda: False)
    def with_it():
        return os.environ.get("DG_SOME_SETTING")

    assert without() is None and with_it() == "7" and os.environ["DG_SOME_SETTING"] == "7"
    with testing.empty_suppress():
        pass


def test_suppress_stdout_stderr_restores_the_descriptors(capfd):
    with testing.suppress_stdout_stderr():
        os.write(1, b"hidden\n")
    os.write(1, b"shown\n")
    out = capfd.readouterr().out
    assert "shown" in out and "hidden" not in out


def test_k_grouped_nt_form_is_rejected_like_the_reference_on_this_architecture():
    import deepgemm_amd_b200 as dg
    with pytest.raises(RuntimeError, match="Unsupported architecture"):
        dg.k_grouped_fp8_gemm_nt_contiguous(None, None, None, [128], None)


def test_import_touches_no_cuda_context_and_shutdown_is_final():
    """tests/test_lazy_init.py of the reference: importing must leave CUDA uninitialised (worker processes pick their
    device afterwards); shutdown() may be called twice, and nothing recreates the runtime after it."""
    import subprocess
    import sys
    import textwrap
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    child = textwrap.dedent("""
        import torch
        import deepgemm_amd_b200 as dg
        assert not torch.cuda.is_initialized()
        assert dg.get_tc_util() == 100
        dg.set_tc_util(90); assert dg.get_tc_util() == 90
        assert not torch.cuda.is_initialized()
        dg.shutdown(); dg.shutdown()
        for call in (dg.get_tc_util, lambda: dg.set_tc_util(80), dg.get_num_sms, lambda: dg.set_mk_alignment_for_contiguous_layout(256)):
            try:
                call()
            except RuntimeError as e:
                assert "shut down" in str(e)
            else:
                raise AssertionError("the runtime was recreated after shutdown")
        print("DG_CHILD_OK")
    """)
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""))
    result = subprocess.run([sys.executable, "-c", child], env=env, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0 and "DG_CHILD_OK" in result.stdout, result.stdout + result.stderr


def test_chunked_parallel_oracle_quantisers_give_the_bytes_of_one_call():
    """oracle/parallel.py applies the oracle's casts to row chunks on a thread pool; the pieces must stack to exactly what
    one call over the whole array gives (per-token casts for any chunking, the 128 x 128 block cast for chunks of whole
    128-row bands), and the chunk-seeded generator must not depend on the thread count."""
    import numpy as np
    import oracle
    a = oracle.seeded_bf16_rows((700, 640), 5, rows_per_chunk=256)
    assert np.array_equal(a, oracle.seeded_bf16_rows((700, 640), 5, rows_per_chunk=256, threads=1))
    assert np.array_equal(a, oracle.bf16_round(a)) and abs(float(a.std()) - 1.0) < 0.02
    b = oracle.seeded_bf16_rows((1000, 640), 6, rows_per_chunk=256)
    for b_fp4 in (False, True):
        qa, sfa, qb, sfb = oracle.quantise_dense_parallel(a, b, b_fp4=b_fp4)
        wa, wsfa = oracle.per_token_cast_to_fp8(a, True, 128)
        assert np.array_equal(qa, wa) and np.array_equal(sfa, wsfa)
        if b_fp4:
            wb, wsfb = oracle.per_token_cast_to_fp4(b, True, 32)
        else:
            wb, raw = oracle.per_block_cast_to_fp8(b, True, 128)
            wsfb = oracle.broadcast_sf_along_mn(raw, b.shape[0], 128)
        assert np.array_equal(qb, wb) and np.array_equal(sfb, wsfb)

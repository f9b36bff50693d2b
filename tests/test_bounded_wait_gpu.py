"""A bounded device-side wait that really runs out.

Every mbarrier wait in the kernels has a time limit after which the waiting role records a code in a host-visible
status word, raises its CTA's abort flag and returns, so that a lost signal ends in an error the host can read rather
than in a hung GPU.  The library's self-test builds a one-CTA kernel from the very same wait primitive with the limit
lowered to a millisecond or so and lets it wait on a barrier nobody arrives at.  Nothing traps, faults or spins without
bound: the kernel returns normally and the context stays usable, which the test checks by running a GEMM afterwards.
(The reference's only timed wait prints and traps after 60 s: deep_gemm/include/deep_gemm/comm/barrier.cuh:11-24.)
"""
import pytest
import torch

import oracle
from gpu_helpers import fp8_cuda, packed_sf_cuda, quantise_dense, seeded_bf16

pytestmark = pytest.mark.gpu

dg = pytest.importorskip("deepgemm_amd_b200")


@pytest.mark.parametrize("timeout_us", [500, 2000])
def test_a_wait_on_a_barrier_nobody_arrives_at_gives_up_and_reports(timeout_us):
    assert dg.kernel_status() == 0
    try:
        status, waited_ns, bystander_ns = dg.selftest_bounded_wait(timeout_us)
        # [31] failure, [30:24] role 7 (self-test), [23:16] site 3, [15:0] CTA 0
        assert status == 0x87030000, hex(status)
        # the waiter gave up after its limit, not long after it (the limit is checked every 256 polls)
        assert timeout_us * 1000 <= waited_ns < 50 * timeout_us * 1000, waited_ns
        # the second waiter (which starts half a limit later) left through the CTA's abort flag about when the first gave
        # up, i.e. before its own limit, without reporting
        assert bystander_ns < timeout_us * 1000, bystander_ns
        assert dg.kernel_status() == 0x87030000          # first failure wins and stays until it is reset
    finally:
        dg.reset_kernel_status()
    assert dg.kernel_status() == 0
    # the kernel returned normally: the context still runs GEMMs
    m, n, k = 128, 256, 512
    qa, sfa, qb, sfb, _ = quantise_dense(seeded_bf16((m, k), 5), seeded_bf16((n, k), 6))
    d = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt((fp8_cuda(qa), packed_sf_cuda(sfa)), (fp8_cuda(qb), packed_sf_cuda(sfb)), d, recipe=(1, 1, 128))
    assert dg.kernel_status() == 0
    assert oracle.calc_diff(d.float().cpu().numpy(), oracle.dequant_gemm_nt(qa, sfa, qb, sfb)) < 1e-3

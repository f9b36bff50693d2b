"""Two-GPU check of the sharded GEMM path: column-parallel dense and expert-parallel grouped GEMMs, one process per
GPU, no collective inside the GEMM; NCCL only gathers the shards for verification (the reference's helper does the
same, deep_gemm/utils/dist.py:38-66).  The gathered result must pass the oracle check and equal the single-GPU
result bit for bit: K is accumulated per output element, independently of how N or the experts are split."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    import oracle
    import deepgemm_amd_b200 as dg
    from deepgemm_amd_b200.dist import expert_rows, shard_columns, shard_experts, uneven_all_gather
    from gpu_helpers import fp8_cuda, packed_sf_cuda, quantise_dense, seeded_bf16

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    results = {}

    # ---- dense, column-parallel along N -----------------------------------------------------------
    m, n, k = 256, 2112, 1024
    qa, sfa, qb, sfb, _ = quantise_dense(seeded_bf16((m, k), 70), seeded_bf16((n, k), 71))
    lo, hi = shard_columns(n, world, rank)
    d_full = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    # every rank writes its column slice straight into a full-pitch D (the D tensor map takes the row pitch)
    dg.fp8_gemm_nt((fp8_cuda(qa), packed_sf_cuda(sfa)), (fp8_cuda(qb[lo:hi]), packed_sf_cuda(sfb[lo:hi])),
                   d_full[:, lo:hi], recipe=(1, 1, 128))
    gathered = uneven_all_gather(d_full[:, lo:hi].contiguous(), dim=1)
    single = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    dg.fp8_gemm_nt((fp8_cuda(qa), packed_sf_cuda(sfa)), (fp8_cuda(qb), packed_sf_cuda(sfb)), single, recipe=(1, 1, 128))
    ref = oracle.dequant_gemm_nt(qa, sfa, qb, sfb)
    results["dense_diff"] = oracle.calc_diff(gathered.float().cpu().numpy(), ref)
    results["dense_bitwise"] = bool(torch.equal(gathered.view(torch.int16), single.view(torch.int16)))

    # ---- m-grouped contiguous, expert-parallel ----------------------------------------------------
    g, n2, k2 = 4, 512, 768
    mt, actual, aligned, layout = oracle.make_contiguous_layout(g, 200, 128, actual_ms=[130, 256, 0, 77])
    a = seeded_bf16((mt, k2), 72)
    a[layout < 0] = 0
    b = seeded_bf16((g, n2, k2), 73)
    qa2, sfa2 = oracle.per_token_cast_to_fp8(a, True, 128)
    qs = [oracle.per_block_cast_to_fp8(b[i], True) for i in range(g)]
    qb2 = np.stack([q for q, _ in qs])
    sfb2 = np.stack([oracle.broadcast_sf_along_mn(s, n2, 128) for _, s in qs])
    g0, g1 = shard_experts(g, world, rank)
    r0, r1 = expert_rows(aligned, g0, g1)
    local_layout = layout[r0:r1].copy()
    local_layout[local_layout >= 0] -= g0                      # re-based expert ids
    d_local = torch.zeros((r1 - r0, n2), dtype=torch.bfloat16, device="cuda")
    if r1 > r0:
        dg.m_grouped_fp8_gemm_nt_contiguous((fp8_cuda(qa2[r0:r1]), packed_sf_cuda(sfa2[r0:r1])),
                                            (fp8_cuda(qb2[g0:g1]), packed_sf_cuda(sfb2[g0:g1])), d_local,
                                            torch.from_numpy(local_layout).cuda(), recipe=(1, 1, 128))
    gathered2 = uneven_all_gather(d_local, dim=0)
    ref2 = oracle.m_grouped_contiguous_ref(qa2, sfa2, qb2, sfb2, aligned)
    valid = layout >= 0
    results["grouped_diff"] = oracle.calc_diff(gathered2.float().cpu().numpy()[valid], ref2[valid])
    results["status"] = dg.kernel_status()
    dist.barrier()
    if rank == 0:
        import json
        json.dump(results, open(os.path.join(out_dir, "results.json"), "w"))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_gemms_gather_to_the_single_gpu_result(tmp_path):
    import json
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    r = json.load(open(tmp_path / "results.json"))
    assert r["status"] == 0
    assert r["dense_diff"] < 1e-5 and r["dense_bitwise"]
    assert r["grouped_diff"] < 1e-5

"""Partitioning logic of the multi-GPU path, run as two gloo ranks on CPU: shards cover the problem exactly,
and gathering per-rank results reproduces the unsharded result (checked with the oracle standing in for the GEMM)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deepgemm_amd_b200.dist import expert_rows, shard_columns, shard_experts, uneven_all_gather


@pytest.mark.parametrize("n", [2112, 4096, 128, 100, 24576])
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_column_shards_partition_n(n, world):
    cuts = [shard_columns(n, world, r) for r in range(world)]
    assert cuts[0][0] == 0 and cuts[-1][1] == n
    for (b0, e0), (b1, e1) in zip(cuts, cuts[1:]):
        assert e0 == b1 and b0 <= e0
    for b, e in cuts:
        assert b == e or (b % 128 == 0 and (e % 128 == 0 or e == n))       # shard starts stay 16-byte aligned for TMA
    sizes = [-(-(e - b) // 128) for b, e in cuts]
    assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("experts,world", [(32, 8), (16, 8), (16, 3), (5, 8)])
def test_expert_shards_partition_groups(experts, world):
    cuts = [shard_experts(experts, world, r) for r in range(world)]
    assert cuts[0][0] == 0 and cuts[-1][1] == experts
    assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
    aligned = [128 * (i % 3 + 1) for i in range(experts)]
    rows = [expert_rows(aligned, b, e) for b, e in cuts]
    assert rows[0][0] == 0 and rows[-1][1] == sum(aligned) and all(a[1] == b[0] for a, b in zip(rows, rows[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(0)                               # same inputs on every rank
    m, n, k = 64, 300, 256
    a = oracle.bf16_round(rng.standard_normal((m, k)).astype(np.float32))
    b = oracle.bf16_round(rng.standard_normal((n, k)).astype(np.float32))
    qa, sfa = oracle.per_token_cast_to_fp8(a, True, 128)
    qb, sfb = oracle.per_token_cast_to_fp8(b, True, 128)
    full = oracle.dequant_gemm_nt(qa, sfa, qb, sfb)
    # dense: column-parallel
    lo, hi = shard_columns(n, world, rank)
    part = oracle.dequant_gemm_nt(qa, sfa, qb[lo:hi], sfb[lo:hi])
    gathered = uneven_all_gather(torch.from_numpy(part), dim=1).numpy()
    ok_dense = np.array_equal(gathered, full)
    # grouped: expert-parallel over 3 experts with uneven row counts
    aligned = [128, 256, 128]
    g0, g1 = shard_experts(3, world, rank)
    r0, r1 = expert_rows(aligned, g0, g1)
    A = oracle.bf16_round(rng.standard_normal((sum(aligned), k)).astype(np.float32))
    B = oracle.bf16_round(rng.standard_normal((3, 40, k)).astype(np.float32))
    qA, sfA = oracle.per_token_cast_to_fp8(A, True, 128)
    qB = np.stack([oracle.per_token_cast_to_fp8(B[i], True, 128)[0] for i in range(3)])
    sfB = np.stack([oracle.per_token_cast_to_fp8(B[i], True, 128)[1] for i in range(3)])
    full_g = oracle.m_grouped_contiguous_ref(qA, sfA, qB, sfB, aligned)
    part_g = oracle.m_grouped_contiguous_ref(qA[r0:r1], sfA[r0:r1], qB[g0:g1], sfB[g0:g1], aligned[g0:g1])
    gathered_g = uneven_all_gather(torch.from_numpy(part_g), dim=0).numpy()
    ok_grouped = np.array_equal(gathered_g, full_g)
    dist.barrier()
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(f"{int(ok_dense)} {int(ok_grouped)}")
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    world, port = 2, _free_port()
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert open(tmp_path / f"rank{r}.txt").read() == "1 1"

"""The N-partition over ranks (host logic of the multi-GPU mode) on CPU: the shard plan, and a
world_size-2 gloo run in which each rank computes its column slab with the CPU checker standing in
for the GPU kernel, the slabs are all-gathered and the step time is reduced as max over ranks --
the same plumbing bench.py uses with NCCL."""
import os
import socket
import sys

import numpy as np
import pytest

import helpers as h
from fp8_quant_matmul_b200.shard import gather_columns_of_C, plan_n_shards, shard_columns_of_B


@pytest.mark.parametrize("N", [7168, 4608, 4096, 3072, 1536, 576, 512, 64])
@pytest.mark.parametrize("G", [1, 2, 4, 8])
def test_plan_covers_and_respects_granule(N, G):
    plan = plan_n_shards(N, G)
    assert len(plan) == G
    pos = 0
    for n0, n_local in plan:
        if n_local == 0:
            continue
        assert n0 == pos and n0 % 64 == 0 and n_local % 16 == 0
        pos += n_local
    assert pos == N
    sizes = [c for _, c in plan if c]
    assert max(sizes) - min(sizes) <= 64 + (N % 64)


def test_shards_reassemble_to_the_unsharded_result():
    M, N, K = 32, 576, 256
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=77)
    full = h.oracle_gemm(A, B, a_s, b_s, M, N, K)
    for G in (2, 4, 8):
        plan = plan_n_shards(N, G)
        slabs = [h.oracle_gemm(A, shard_columns_of_B(B, N, K, n0, nl), a_s, b_s, M, nl, K, n0=n0, n_total=N)
                 if nl else np.empty((M, 0), np.uint16) for (n0, nl) in plan]
        assert np.array_equal(gather_columns_of_C(slabs, plan, M, N), full)


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        M, N, K = 32, 576, 256
        A, B, a_s, b_s = h.make_inputs(M, N, K, seed=5)          # A and the scales are replicated
        plan = plan_n_shards(N, world)
        n0, nl = plan[rank]
        mine = h.oracle_gemm(A, shard_columns_of_B(B, N, K, n0, nl), a_s, b_s, M, nl, K, n0=n0, n_total=N)
        # all-gather of ragged slabs: pad to the widest, as bench.py does for the NCCL gather
        width = max(c for _, c in plan)
        pad = np.zeros((M, width), np.uint16)
        pad[:, :nl] = mine
        bufs = [torch.zeros((M, width * 2), dtype=torch.uint8) for _ in range(world)]     # bf16 bits as bytes
        dist.all_gather(bufs, torch.from_numpy(pad.view(np.uint8)))
        slabs = [b.numpy().view(np.uint16)[:, :plan[r][1]] for r, b in enumerate(bufs)]
        C = gather_columns_of_C(slabs, plan, M, N)
        t = torch.tensor([10.0 + rank])                          # per-rank step time -> max over ranks
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        ok = np.array_equal(C, h.oracle_gemm(A, B, a_s, b_s, M, N, K)) and float(t) == 10.0 + world - 1
        q.put((rank, bool(ok)))
    except Exception as e:  # report instead of leaving the parent waiting
        q.put((rank, repr(e)))
        raise
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo_partition_and_gather():
    torch = pytest.importorskip("torch")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def _leaving_worker(rank, world, port, q):
    """Three steps; rank 1 leaves after the first one (between steps, nothing of its in flight).  The others learn of
    it on the host: their next collective ends with an error after the short process-group timeout."""
    import datetime
    import time
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    steps_done, noticed = 0, None
    try:
        for step in range(3):
            t = torch.tensor([float(rank)])
            dist.all_reduce(t, op=dist.ReduceOp.MAX)             # stands for the step's barrier / max-over-ranks
            steps_done += 1
            if rank == 1 and step == 0:
                q.put((rank, steps_done, "left"))
                return                                           # leaves without calling any further collective
            time.sleep(0.1)
    except Exception as e:                                       # the survivor's next collective fails: detected
        noticed = type(e).__name__
    q.put((rank, steps_done, noticed))


def test_a_rank_that_leaves_between_steps_is_noticed_by_the_others():
    torch = pytest.importorskip("torch")
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_leaving_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.terminate()
    assert results[1] == (1, 1, "left")
    rank, steps_done, noticed = results[0]
    assert rank == 0 and steps_done == 1 and noticed is not None, results     # no second step was completed alone

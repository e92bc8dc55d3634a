"""Fused distribution of C (fp8bs_gemm_scatter): an N-sharded GEMM whose epilogue stores every finished tile into the
full-width C of several destinations.  On one GPU the destinations are separate local buffers; with two or more
GPUs the test runs one process per GPU and the destinations are the ranks' peer-mapped buffers."""
import os
import sys

import numpy as np
import pytest
import torch

import fp8_quant_matmul_b200 as f
from fp8_quant_matmul_b200.shard import plan_n_shards

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import helpers as h  # noqa: E402

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda:0")


@pytest.mark.parametrize("shape,shards,ndest", [((256, 512, 512), 2, 2), ((384, 1152, 1024), 3, 3), ((1024, 576, 1024), 4, 8),
                                                ((144, 320, 384), 2, 1)],
                         ids=["256x512-2shards", "384x1152-3shards", "1024x576-4shards-8dest", "ragged-1dest"])
def test_every_destination_receives_every_shard(shape, shards, ndest):
    M, N, K = shape
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=41)
    ref = h.oracle_gemm(A, B, a_s, b_s, M, N, K)
    dA = torch.from_numpy(A).to(dev())
    dAs, dBs = torch.from_numpy(a_s).to(dev()), torch.from_numpy(b_s).to(dev())
    dests = [torch.full((M + 2, N), float("nan"), dtype=torch.bfloat16, device=dev()) for _ in range(ndest)]
    Bm = B.reshape(K, N)
    for (n0, nl) in plan_n_shards(N, shards):
        dB = torch.from_numpy(np.ascontiguousarray(Bm[:, n0:n0 + nl]).ravel()).to(dev())
        f.gemm_scatter(dA, dB, dAs, dBs, [d[1:M + 1] for d in dests], M, nl, K, n0, N)
    f.last_device_status()
    for d in dests:
        bits = d.view(torch.int16).cpu().numpy().view(np.uint16)
        assert np.isnan(h.bf16_bits_to_f32(bits[0])).all() and np.isnan(h.bf16_bits_to_f32(bits[M + 1])).all()   # guard rows
        bad, first, maxerr = h.mismatches(ref, bits[1:M + 1])
        assert bad == 0, "%d mismatches, first %d, max err %g" % (bad, first, maxerr)


def test_pair_tile_stores_to_every_destination():
    # a column shard large enough for the dispatcher to pick the 256 x 256 CTA-pair tile (long K): both CTAs of a pair
    # store their own 128 rows into every destination
    M, N, K, shards = 2048, 2560, 4096, 2
    assert f.select_path(M, N // shards, K)[2] & f.TILE_PAIR
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=45)
    rows = np.arange(5, M, 37, dtype=np.int32)
    ref = h.oracle_gemm(A, B, a_s, b_s, M, N, K, rows=rows)
    dA = torch.from_numpy(A).to(dev())
    dAs, dBs = torch.from_numpy(a_s).to(dev()), torch.from_numpy(b_s).to(dev())
    dests = [torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev()) for _ in range(2)]
    Bm = B.reshape(K, N)
    for (n0, nl) in plan_n_shards(N, shards):
        dB = torch.from_numpy(np.ascontiguousarray(Bm[:, n0:n0 + nl]).ravel()).to(dev())
        f.gemm_scatter(dA, dB, dAs, dBs, dests, M, nl, K, n0, N)
    f.last_device_status()
    for d in dests:
        assert not torch.isnan(d).any()
        bad, first, maxerr = h.mismatches(ref, d.view(torch.int16).cpu().numpy().view(np.uint16)[rows])
        assert bad == 0, "%d mismatches, first %d, max err %g" % (bad, first, maxerr)


def test_scatter_argument_errors():
    M, N, K = 128, 256, 256
    z8 = torch.zeros(M * K, dtype=torch.uint8, device=dev())
    zb = torch.zeros(N * K, dtype=torch.uint8, device=dev())
    s1 = torch.ones(M * 2, dtype=torch.float32, device=dev())
    s2 = torch.ones(2 * 2, dtype=torch.float32, device=dev())
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=dev())
    with pytest.raises(f.Fp8bsError) as e:
        f.gemm_scatter(z8, zb, s1, s2, [C] * 9, M, N, K, 0, N)        # more than 8 destinations
    assert e.value.code == -5
    with pytest.raises(f.Fp8bsError) as e:
        f.gemm_scatter(z8, zb, s1, s2, [C.data_ptr() + 2], M, N, K, 0, N)   # misaligned destination
    assert e.value.code == -3
    with pytest.raises(f.Fp8bsError) as e:
        f.gemm_scatter(z8, zb, s1, s2, [C], M, 128, K, 32, N)           # shard boundary not on 64 columns
    assert e.value.code == -5


def _rank_main(rank, world, port, q):
    """One rank of the peer-write test.  Every step that can fail on one rank alone is followed by a collective
    agreement (an all-reduce of a success flag), so that all ranks take the same exit path: none is left inside a
    collective that a failed peer never joins, and none exits while a peer still maps its memory."""
    import datetime
    import traceback
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0",
                      TORCH_SYMM_MEM_DISABLE_MULTICAST="1")       # plain peer mappings, no NVLink multicast objects
    joined = False
    try:
        torch.cuda.set_device(rank)
        d = torch.device("cuda", rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=d,
                                timeout=datetime.timedelta(seconds=60))
        joined = True

        def all_ok(ok):
            t = torch.tensor([0.0 if ok else 1.0], device=d)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item() == 0.0

        M, N, K = 512, 1024, 1024
        A, B, a_s, b_s = h.make_inputs(M, N, K, seed=43)
        n0, nl = plan_n_shards(N, world)[rank]
        err, Cfull, hdl = "", None, None
        try:
            import torch.distributed._symmetric_memory as symm
            Cfull = symm.empty((M, N), dtype=torch.bfloat16, device=d)
            Cfull.fill_(float("nan"))
        except Exception:
            err = traceback.format_exc()[-1500:]
        if not all_ok(Cfull is not None):                  # before the rendezvous, which is itself collective
            q.put((rank, -1, err or "symmetric memory unavailable on another rank"))
            return
        hdl = symm.rendezvous(Cfull, dist.group.WORLD.group_name)
        dist.barrier()
        torch.cuda.synchronize()
        bad = -1
        try:
            dA = torch.from_numpy(A).to(d)
            dB = torch.from_numpy(np.ascontiguousarray(B.reshape(K, N)[:, n0:n0 + nl]).ravel()).to(d)
            f.gemm_scatter(dA, dB, torch.from_numpy(a_s).to(d), torch.from_numpy(b_s).to(d),
                           [int(p) for p in hdl.buffer_ptrs], M, nl, K, n0, N)
            torch.cuda.synchronize()
            f.last_device_status()
            bad = 0
        except Exception:
            err = traceback.format_exc()[-1500:]
        wrote = all_ok(bad == 0)                           # doubles as the barrier: every rank's stores have drained
        torch.cuda.synchronize()
        if wrote:
            bits = Cfull.view(torch.int16).cpu().numpy().view(np.uint16)
            bad, first, maxerr = h.mismatches(h.oracle_gemm(A, B, a_s, b_s, M, N, K), bits)
            err = "" if bad == 0 else "first mismatch at %d, max err %g" % (first, maxerr)
        q.put((rank, bad if wrote else -1, err or "a peer failed"))
        all_ok(True)                                       # nobody unmaps while a peer is still reading its copy
        del hdl, Cfull
    except Exception:                 # report instead of hanging the parent
        q.put((rank, -1, traceback.format_exc()[-1500:]))
    finally:
        if joined:
            try:
                dist.destroy_process_group()
            except Exception:
                pass


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_write_each_others_c():
    import queue
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            try:
                results.append(q.get(timeout=240))
            except queue.Empty:
                break
    finally:
        for p in procs:                # the children have reported (or timed out): reap them, whatever happened
            p.join(timeout=90)
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(timeout=30)
    assert len(results) == world, "only %d of %d ranks reported" % (len(results), world)
    for rank, bad, msg in results:
        assert bad == 0, "rank %d: %s %s" % (rank, bad, msg)

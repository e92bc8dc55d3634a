"""The allocation-free split-K entry point, fp8bs_gemm_mn_small_static.

Some callers cannot give the library scratch memory when they call it: their device memory belongs to another
allocator, they are forbidden to call cudaMalloc, or they cannot afford the synchronisation an allocation brings.
For them the library carries its own fixed scratch array.  This test calls the entry point through the C ABI twice
in a row (the second call finds the array as the first one left it) and compares each result with what the ordinary
entry point, fp8bs_gemm_mn_small with a caller-owned workspace, produces for the same inputs.

The file name sorts last on purpose: if this addition fails, a run that stops at the first failure has already
executed every other test.
"""
import numpy as np
import pytest

import fp8_quant_matmul_b200 as f
import helpers as h

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _inputs(M, N, K, seed):
    dev = torch.device("cuda:0")
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=seed)
    return [torch.from_numpy(x).to(dev) for x in (A, B, a_s, b_s)], (A, B, a_s, b_s)


def _bits(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.parametrize("M,N,K,splits", [(1024, 512, 7168, 4), (1024, 576, 7168, 3), (256, 256, 1024, 0)])
def test_static_scratch_matches_the_workspace_entry_point(M, N, K, splits):
    dev = torch.device("cuda:0")
    lib = f.lib()
    need = f.workspace_bytes(M, N, K, f.PATH_MN_SMALL, splits, f.SPLIT_WORKSPACE)     # what the static entry point uses
    assert 0 < need <= f.STATIC_SCRATCH_BYTES
    ws = torch.zeros(max(need, 65536), dtype=torch.uint8, device=dev)
    for call in range(2):                                   # two calls in a row, different data each time
        (dA, dB, dAs, dBs), host = _inputs(M, N, K, seed=40 + call)
        want = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        same = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        args = (dA.data_ptr(), dB.data_ptr(), dAs.data_ptr(), dBs.data_ptr())
        # the existing entry point (it may pick the cluster reduction: another kernel, same split order) ...
        assert lib.fp8bs_gemm_mn_small(*args, want.data_ptr(), M, N, K, splits, ws.data_ptr(), ws.numel(), None) == 0
        # ... and the same kernel the static entry point runs, on a caller-owned workspace
        assert lib.fp8bs_gemm_ex(*args, same.data_ptr(), M, N, K, 0, N, f.PATH_MN_SMALL, splits, f.SPLIT_WORKSPACE,
                                 ws.data_ptr(), ws.numel(), None) == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        assert lib.fp8bs_gemm_mn_small_static(*args, got.data_ptr(), M, N, K, splits, None) == 0
        torch.cuda.synchronize()
        if call == 1:       # the first call on a device may do one-time set-up; the second must not touch the allocator
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        f.last_device_status()
        got_bits = _bits(got)
        # same kernel, same summation order: every bit agrees
        assert np.array_equal(_bits(same), got_bits), "call %d: differs from the workspace split-K kernel" % call
        bad, first, maxerr = h.mismatches(_bits(want), got_bits)     # |d| <= 1e-3 + 2e-2*|ref|, the suite's tolerance
        assert bad == 0, "call %d: %d mismatches, first %d, max err %g" % (call, bad, first, maxerr)
        # and both agree with the CPU checker
        rows = np.arange(0, M, 8, dtype=np.int32)
        bad, first, maxerr = h.mismatches(h.oracle_gemm(*host, M, N, K, rows=rows), got_bits[rows])
        assert bad == 0, "call %d vs checker: %d mismatches" % (call, bad)


def test_static_scratch_is_usable_after_a_reported_timeout():
    """The wait-timeout self-test leaves a status behind; once it has been read, the built-in scratch works as before."""
    dev = torch.device("cuda:0")
    lib = f.lib()
    M, N, K, splits = 256, 256, 1024, 4
    (dA, dB, dAs, dBs), host = _inputs(M, N, K, seed=47)
    assert lib.fp8bs_selftest_wait_timeout(None) == 0
    with pytest.raises(f.Fp8bsError):
        f.last_device_status()
    got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    assert lib.fp8bs_gemm_mn_small_static(dA.data_ptr(), dB.data_ptr(), dAs.data_ptr(), dBs.data_ptr(), got.data_ptr(),
                                          M, N, K, splits, None) == 0
    torch.cuda.synchronize()
    f.last_device_status()
    bad, first, maxerr = h.mismatches(h.oracle_gemm(*host, M, N, K), _bits(got))
    assert bad == 0


def test_static_scratch_refuses_what_does_not_fit():
    dev = torch.device("cuda:0")
    M, N, K = 6144, 4608, 256
    assert f.workspace_bytes(M, N, K, f.PATH_MN_SMALL, 2, f.SPLIT_WORKSPACE) > f.STATIC_SCRATCH_BYTES
    dummy = torch.zeros(M * K + N * K, dtype=torch.uint8, device=dev)
    scales = torch.ones(M * 2 + 36 * 2, dtype=torch.float32, device=dev)
    C = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
    rc = f.lib().fp8bs_gemm_mn_small_static(dummy.data_ptr(), dummy.data_ptr(), scales.data_ptr(), scales.data_ptr(),
                                            C.data_ptr(), M, N, K, 2, None)
    assert rc == -4                                           # FP8BS_ERR_WORKSPACE
    assert "workspace" in f.status_string(rc)

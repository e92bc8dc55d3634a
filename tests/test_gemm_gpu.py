"""Parity of the CUDA kernels with the CPU checker, through the C ABI (ctypes -> libfp8bs.so).

Tolerance: |got - ref| <= 1e-3 + 2e-2 * |ref| on the bf16 outputs, zero mismatches allowed
(fp32 accumulation in a different order than the checker, then one bf16 rounding)."""
import os

import numpy as np
import pytest

import fp8_quant_matmul_b200 as f
import helpers as h

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def dev():
    return torch.device("cuda:0")


def to_dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(dev()) for a in arrays]


def run_gemm(A, B, a_s, b_s, M, N, K, **kw):
    """Runs the library on device copies of the inputs; returns bf16 bits [M, N] and checks that the
    rows before and after C were not touched."""
    dA, dB, dAs, dBs = to_dev(A, B, a_s, b_s)
    guard = torch.full((M + 2, N), float("nan"), dtype=torch.bfloat16, device=dev())
    guard[0].fill_(12288.0)
    guard[M + 1].fill_(-12288.0)
    C = guard[1:M + 1]
    f.gemm(dA, dB, dAs, dBs, C, M, N, K, **kw)
    f.last_device_status()
    out = guard.view(torch.int16).cpu().numpy().view(np.uint16)
    assert (h.bf16_bits_to_f32(out[0]) == 12288.0).all() and (h.bf16_bits_to_f32(out[M + 1]) == -12288.0).all()
    return out[1:M + 1]


def assert_parity(ref_bits, got_bits, what=""):
    bad, first, maxerr = h.mismatches(ref_bits, got_bits)
    assert bad == 0, "%s: %d mismatches, first at flat index %d, max |err| %g" % (what, bad, first, maxerr)


FORCED = [
    dict(path=f.PATH_MN_LARGE, splits=1, tile_n=128),
    dict(path=f.PATH_MN_LARGE, splits=1, tile_n=256),
    dict(path=f.PATH_MN_SMALL, splits=1, tile_n=128),
    dict(path=f.PATH_MN_SMALL, splits=2, tile_n=128),
    dict(path=f.PATH_MN_SMALL, splits=2, tile_n=256),
    dict(path=f.PATH_MN_LARGE, splits=1, tile_n=256 | f.TILE_PAIR),      # 256 x 256 tile on a pair of CTAs
    dict(path=f.PATH_MN_SMALL, splits=2, tile_n=256 | f.TILE_PAIR),
    dict(path=f.PATH_MN_SMALL, splits=2, tile_n=128 | f.SPLIT_WORKSPACE),  # split-K reduced through the workspace
    dict(path=f.PATH_MN_SMALL, splits=2, tile_n=256 | f.SPLIT_WORKSPACE),
    dict(path=f.PATH_MN_SMALL, splits=1, tile_n=128 | f.STREAM_K),         # K blocks of all tiles dealt out over the SMs
    dict(path=f.PATH_MN_SMALL, splits=1, tile_n=256 | f.STREAM_K),
]


def ids(cfgs):
    return ["p%d-s%d-t%d%s%s" % (c["path"], c["splits"], c["tile_n"] & 0xFFF, "pair" if c["tile_n"] & f.TILE_PAIR else "",
                                 "ws" if c["tile_n"] & f.SPLIT_WORKSPACE else ("sk" if c["tile_n"] & f.STREAM_K else
                                                                                 ("short" if c["tile_n"] & f.SHORT_K else "")))
            for c in cfgs]


# ------------------------------------------------------------------ known answers ----------
@pytest.mark.parametrize("cfg", FORCED, ids=ids(FORCED))
def test_kat_all_ones_counts_every_k(cfg):
    M, N, K = 128, 256, 512
    one = h.e4m3fn_byte(1.0)
    A, B = np.full(M * K, one, np.uint8), np.full(N * K, one, np.uint8)
    a_s, b_s = np.ones(M * K // 128, np.float32), np.ones(2 * K // 128, np.float32)
    got = h.bf16_bits_to_f32(run_gemm(A, B, a_s, b_s, M, N, K, **cfg))
    assert (got == float(K)).all()


@pytest.mark.parametrize("cfg", FORCED, ids=ids(FORCED))
def test_kat_small_integers_are_exact(cfg):
    # unit scales, operands in {-2..2}: block sums are small integers -> any lost accumulation shows
    M, N, K = 128, 256, 256
    rng = np.random.default_rng(5)
    vals = np.array([h.e4m3fn_byte(v) for v in (-2.0, -1.0, 0.0, 1.0, 2.0)], dtype=np.uint8)
    ai, bi = rng.integers(0, 5, (K, M)), rng.integers(0, 5, (K, N))
    want = ((ai - 2).T.astype(np.int64) @ (bi - 2).astype(np.int64)).astype(np.float32)
    assert np.abs(want).max() < 256
    got = h.bf16_bits_to_f32(run_gemm(vals[ai].ravel(), vals[bi].ravel(), np.ones(M * 2, np.float32),
                                      np.ones(2 * 2, np.float32), M, N, K, **cfg))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("cfg", FORCED[:3], ids=ids(FORCED[:3]))
def test_kat_one_hot_pins_index_formulas(cfg):
    # one non-zero in A and in B: exactly one non-zero in C, scaled by a_scale[m + M*kb] * b_scale[nb + sn*kb]
    M, N, K = 144, 576, 384                        # ragged: M % 128 = 16, N % 128 = 64, sn = 5
    sn, KB = 5, 3
    a_s = 1.0 + np.arange(M * KB, dtype=np.float32) / 64
    b_s = (0.5 + np.arange(sn * KB, dtype=np.float32)) * 0.25
    for (m, n, k) in [(0, 0, 0), (143, 575, 383), (7, 513, 130), (130, 127, 255), (3, 128, 256)]:
        A, B = np.zeros(M * K, np.uint8), np.zeros(N * K, np.uint8)
        A[m + M * k] = h.e4m3fn_byte(3.0)
        B[n + N * k] = h.e4m3fn_byte(-1.5)
        got = run_gemm(A, B, a_s, b_s, M, N, K, **cfg)
        assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), got, "one-hot %s" % ((m, n, k),))
        assert np.count_nonzero(h.bf16_bits_to_f32(got)) == 1 and h.bf16_bits_to_f32(got)[m, n] != 0


# ------------------------------------------------------------------ short K (K <= 256) ------
SHORT = dict(path=f.PATH_MN_LARGE, splits=1, tile_n=f.SHORT_K)      # a tile's partial sums stay in tensor memory
SHORT_K_SHAPES = [(128, 128, 128), (128, 128, 256), (16, 16, 128), (144, 80, 256), (128, 64, 256), (512, 1024, 256),
                  (2048, 2064, 256), (1024, 7168, 256), (1024, 7168, 128)]


@pytest.mark.parametrize("shape", SHORT_K_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_short_k_kernel_matches_the_oracle_and_the_full_k_kernel_bit_for_bit(shape):
    M, N, K = shape
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=300 + M + N + K)
    got = run_gemm(A, B, a_s, b_s, M, N, K, **SHORT)
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), got, "short K %s" % (shape,))
    # same arithmetic in the same order as the K loop of the other kernels: equal bits, not only equal within tolerance
    full = run_gemm(A, B, a_s, b_s, M, N, K, path=f.PATH_MN_LARGE, splits=1, tile_n=256)
    assert np.array_equal(got, full)


def test_short_k_kat_small_integers_and_one_hot():
    M, N, K = 128, 256, 256
    rng = np.random.default_rng(6)
    vals = np.array([h.e4m3fn_byte(v) for v in (-2.0, -1.0, 0.0, 1.0, 2.0)], dtype=np.uint8)
    ai, bi = rng.integers(0, 5, (K, M)), rng.integers(0, 5, (K, N))
    want = ((ai - 2).T.astype(np.int64) @ (bi - 2).astype(np.int64)).astype(np.float32)
    got = h.bf16_bits_to_f32(run_gemm(vals[ai].ravel(), vals[bi].ravel(), np.ones(M * 2, np.float32),
                                      np.ones(2 * 2, np.float32), M, N, K, **SHORT))
    assert np.array_equal(got, want)
    # one non-zero in A and in B on a ragged shape: exactly one non-zero in C, scaled by a_scale[m + M*kb] * b_scale[nb + sn*kb]
    M, N, K = 144, 576, 256
    sn, KB = 5, 2
    a_s = 1.0 + np.arange(M * KB, dtype=np.float32) / 64
    b_s = (0.5 + np.arange(sn * KB, dtype=np.float32)) * 0.25
    for (m, n, k) in [(0, 0, 0), (143, 575, 255), (7, 513, 130), (130, 127, 127), (3, 128, 128)]:
        A, B = np.zeros(M * K, np.uint8), np.zeros(N * K, np.uint8)
        A[m + M * k] = h.e4m3fn_byte(3.0)
        B[n + N * k] = h.e4m3fn_byte(-1.5)
        got = run_gemm(A, B, a_s, b_s, M, N, K, **SHORT)
        assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), got, "one-hot %s" % ((m, n, k),))
        assert np.count_nonzero(h.bf16_bits_to_f32(got)) == 1 and h.bf16_bits_to_f32(got)[m, n] != 0


def test_short_k_column_shard_uses_the_global_scale_columns():
    # columns [n0, n0 + nl) of a wider problem: b_scale is indexed by the global column
    M, N, K, n0, nl = 256, 1024, 256, 192, 448
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=77)
    full = h.oracle_gemm(A, B, a_s, b_s, M, N, K)
    from fp8_quant_matmul_b200.shard import shard_columns_of_B
    got = run_gemm(A, shard_columns_of_B(B, N, K, n0, nl), a_s, b_s, M, nl, K, n0=n0, n_total=N, **SHORT)
    assert_parity(np.ascontiguousarray(full[:, n0:n0 + nl]), got, "short K shard")


# ------------------------------------------------------------------ random parity ----------
SMALL_SHAPES = [(128, 128, 128), (128, 128, 256), (256, 256, 512), (16, 16, 128), (144, 80, 384),
                (384, 576, 1024), (128, 64, 256), (512, 1024, 256)]


@pytest.mark.parametrize("shape", SMALL_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("cfg", FORCED, ids=ids(FORCED))
def test_forced_paths_small_shapes(shape, cfg):
    M, N, K = shape
    if cfg["splits"] > K // 128:
        pytest.skip("more splits than K blocks")
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=100 + M + N + K)
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), run_gemm(A, B, a_s, b_s, M, N, K, **cfg), str((shape, cfg)))


def test_reference_style_inputs_negative_scales():
    # check.cu:155-162 draws elements AND scales from U(-5, 5): scales may be negative
    M, N, K = 256, 320, 512
    rng = np.random.default_rng(2)
    A = f.float_to_e4m3fn(rng.uniform(-5, 5, M * K).astype(np.float32))
    B = f.float_to_e4m3fn(rng.uniform(-5, 5, N * K).astype(np.float32))
    a_s = rng.uniform(-5, 5, M * K // 128).astype(np.float32)
    b_s = rng.uniform(-5, 5, 3 * K // 128).astype(np.float32)
    ref = h.oracle_gemm(A, B, a_s, b_s, M, N, K)
    for cfg in FORCED:
        assert_parity(ref, run_gemm(A, B, a_s, b_s, M, N, K, **cfg), str(cfg))


@pytest.mark.parametrize("name", ["check_case.npz", "quantize_case.npz"])
def test_golden_fixtures_on_gpu(name):
    # expected values produced by the reference's own host code (see tests/golden/make_golden.py)
    g = np.load(os.path.join(h.GOLDEN_DIR, name))
    M, N, K = int(g["M"]), int(g["N"]), int(g["K"])
    want = g["C_gemmcpu_bf16"] if "C_gemmcpu_bf16" in g else g["C_bf16"]
    for cfg in (dict(), FORCED[0], FORCED[3]):
        assert_parity(want, run_gemm(g["A"], g["B"], g["a_scale"], g["b_scale"], M, N, K, **cfg), name)


def test_ref_kernel_is_bit_identical_to_the_checker():
    # the ground-truth kernel restated in CUDA (check.cu:30-49) performs the checker's operations in order
    M, N, K = 96, 576, 384
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=8, scale_lo=-2.0, scale_hi=2.0)
    dA, dB, dAs, dBs = to_dev(A, B, a_s, b_s)
    C = f.gemm_ref(dA, dB, dAs, dBs, M, N, K)
    got = C.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, h.oracle_gemm(A, B, a_s, b_s, M, N, K))


@pytest.mark.parametrize("shape", f.SHAPES_18, ids=lambda s: "x".join(map(str, s)))
def test_auto_dispatch_on_the_18_benchmark_shapes(shape):
    M, N, K = shape
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=7 + 13 * f.SHAPES_18.index(shape))
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), run_gemm(A, B, a_s, b_s, M, N, K), str(shape))


@pytest.mark.parametrize("shape", [(1024, 512, 7168), (1024, 576, 7168), (1024, 1536, 7168), (6144, 4608, 7168)],
                         ids=lambda s: "x".join(map(str, s)))
def test_both_kernels_forced_on_named_configs(shape):
    M, N, K = shape
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=31)
    rows = np.arange(0, M, max(1, M // 512), dtype=np.int32)
    ref = h.oracle_gemm(A, B, a_s, b_s, M, N, K, rows=rows)
    for cfg in (FORCED[0], FORCED[1], FORCED[5], dict(path=f.PATH_MN_SMALL, splits=0, tile_n=0),
                dict(path=f.PATH_MN_SMALL, splits=4, tile_n=128), dict(path=f.PATH_MN_SMALL, splits=3, tile_n=256 | f.TILE_PAIR)):
        if cfg["splits"] > 1 and M * N > 4096 * 4096:
            continue
        assert_parity(ref, run_gemm(A, B, a_s, b_s, M, N, K, **cfg)[rows], str((shape, cfg)))


# ------------------------------------------------------------------ properties -------------
@pytest.mark.parametrize("shape,splits,tile_n", [((1024, 576, 7168), 7, 128), ((6144, 512, 7168), 6, 128),
                                                 ((6144, 512, 7168), 3, 256 | 0x1000), ((6144, 512, 7168), 7, 256),
                                                 ((1024, 576, 7168), 7, 128 | 0x2000), ((6144, 512, 7168), 6, 128 | 0x2000),
                                                 ((6144, 512, 7168), 9, 128), ((6144, 512, 7168), 7, 256 | 0x2000),
                                                 ((1024, 576, 7168), 1, 128 | 0x4000), ((6144, 512, 7168), 1, 256 | 0x4000),
                                                 ((1024, 1536, 7168), 1, 256 | 0x4000), ((1024, 7168, 2304), 1, 256 | 0x4000)],
                         ids=["1024x576-s7-t128", "6144x512-s6-t128", "6144x512-s3-pair", "6144x512-s7-t256",
                              "1024x576-s7-t128-ws", "6144x512-s6-t128-ws", "6144x512-s9-t128-ws", "6144x512-s7-t256-ws",
                              "1024x576-t128-streamk", "6144x512-t256-streamk", "1024x1536-t256-streamk",
                              "1024x7168x2304-t256-streamk"])
def test_split_k_is_bit_deterministic(shape, splits, tile_n):
    # several work units per CTA; the workspace is poisoned with NaN before every run so that a partial sum
    # read before it was written, or left over from another run, cannot go unnoticed
    M, N, K = shape
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=3)
    dA, dB, dAs, dBs = to_dev(A, B, a_s, b_s)
    ws = torch.zeros(max(65536, f.workspace_bytes(M, N, K, f.PATH_MN_SMALL, splits, tile_n)), dtype=torch.uint8, device=dev())
    first = None
    for i in range(20):
        ws[65536:].fill_(0xFF)
        C = torch.empty((M, N), dtype=torch.bfloat16, device=dev())
        f.gemm(dA, dB, dAs, dBs, C, M, N, K, path=f.PATH_MN_SMALL, splits=splits, tile_n=tile_n, workspace=ws)
        bits = C.view(torch.int16)
        if first is None:
            first = bits.clone()
        else:
            assert torch.equal(first, bits), "run %d differs" % i
    f.last_device_status()
    rows = np.arange(0, M, max(1, M // 512), dtype=np.int32)
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K, rows=rows), first.cpu().numpy().view(np.uint16)[rows])


def test_power_of_two_scale_linearity_at_full_size():
    # doubling a_scale doubles every partial product exactly, so C doubles bit-exactly (size-independent)
    M, N, K = 6144, 4608, 7168
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=17)
    dA, dB, dAs, dBs = to_dev(A, B, a_s, b_s)
    C1 = f.gemm(dA, dB, dAs, dBs, None, M, N, K)
    C2 = f.gemm(dA, dB, dAs * 2.0, dBs, None, M, N, K)
    f.last_device_status()
    assert torch.equal((C1.float() * 2.0).to(torch.bfloat16).view(torch.int16), C2.view(torch.int16))
    rows = np.array([0, 1, 127, 128, 3071, 6143], dtype=np.int32)
    got = C1.view(torch.int16).cpu().numpy().view(np.uint16)[rows]
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K, rows=rows), got)


def test_column_shards_equal_the_unsharded_result():
    # the multi-GPU partition, emulated on one GPU: every shard is bit-identical to the same columns
    # of the unsharded call (same kernel, same per-element operation order)
    from fp8_quant_matmul_b200.shard import plan_n_shards, shard_columns_of_B, gather_columns_of_C
    M, K = 512, 1024
    for N in (576, 1536):
        A, B, a_s, b_s = h.make_inputs(M, N, K, seed=N)
        ref = h.oracle_gemm(A, B, a_s, b_s, M, N, K)
        for G in (2, 4, 8):
            plan = plan_n_shards(N, G)
            slabs = [run_gemm(A, shard_columns_of_B(B, N, K, n0, nl), a_s, b_s, M, nl, K, n0=n0, n_total=N)
                     for (n0, nl) in plan]
            assert_parity(ref, gather_columns_of_C(slabs, plan, M, N), "N=%d G=%d" % (N, G))


@pytest.mark.parametrize("NK", [(512, 7168), (7168, 256), (4608, 7168)], ids=lambda s: "x".join(map(str, s)))
def test_m16384_variant_sampled_rows(NK):
    # multi-GPU workload shape (M = 16384), one GPU's 1/8 column shard, 256 seeded sample rows checked
    from fp8_quant_matmul_b200.shard import plan_n_shards, shard_columns_of_B
    N, K = NK
    M = 16384
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=99)
    n0, nl = plan_n_shards(N, 8)[3]
    Bs = shard_columns_of_B(B, N, K, n0, nl)
    rows = np.sort(np.random.default_rng(0).choice(M, 256, replace=False)).astype(np.int32)
    got = run_gemm(A, Bs, a_s, b_s, M, nl, K, n0=n0, n_total=N)
    assert_parity(h.oracle_gemm(A, Bs, a_s, b_s, M, nl, K, n0=n0, n_total=N, rows=rows), got[rows])


# ------------------------------------------------------------------ boundary behaviour -----
def test_workspace_rules():
    M, N, K = 256, 256, 1024
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=1)
    dA, dB, dAs, dBs = to_dev(A, B, a_s, b_s)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=dev())
    lib = f.lib()
    args = (dA.data_ptr(), dB.data_ptr(), dAs.data_ptr(), dBs.data_ptr(), C.data_ptr(), M, N, K)
    small = torch.zeros(1024, dtype=torch.uint8, device=dev())
    # forced split-K through the workspace with too little of it is an error, never a silent other path
    assert lib.fp8bs_gemm_ex(*args, 0, N, f.PATH_MN_SMALL, 4, 128 | f.SPLIT_WORKSPACE, small.data_ptr(), small.numel(), None) == -4
    # the cluster reduction needs none
    assert lib.fp8bs_gemm_mn_small(*args, 4, None, 0, None) == 0
    # auto dispatch without workspace falls back to a full-K configuration and is still right
    assert lib.fp8bs_gemm(*args, None, 0, None) == 0
    torch.cuda.synchronize()
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), C.view(torch.int16).cpu().numpy().view(np.uint16))
    # an explicit caller-owned workspace
    need = f.workspace_bytes(M, N, K, f.PATH_MN_SMALL, 4, 128 | f.SPLIT_WORKSPACE)
    ws = torch.empty(need, dtype=torch.uint8, device=dev())
    assert lib.fp8bs_workspace_init(ws.data_ptr(), need, None) == 0
    for _ in range(3):     # the counters re-arm themselves between calls
        C.fill_(float("nan"))
        assert lib.fp8bs_gemm_ex(*args, 0, N, f.PATH_MN_SMALL, 4, 128 | f.SPLIT_WORKSPACE, ws.data_ptr(), need, None) == 0
        torch.cuda.synchronize()
        assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), C.view(torch.int16).cpu().numpy().view(np.uint16))
    assert lib.fp8bs_last_device_status(None, None) == 0


def test_runs_on_a_side_stream_and_counts_launches():
    M, N, K = 256, 256, 256
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=12)
    dA, dB, dAs, dBs = to_dev(A, B, a_s, b_s)
    before = f.launch_count()
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        C = f.gemm(dA, dB, dAs, dBs, None, M, N, K)
    s.synchronize()
    assert f.launch_count() == before + 1
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), C.view(torch.int16).cpu().numpy().view(np.uint16))


def test_gemmGPU_mirror_with_host_buffers():
    # the reference's host wrapper (check.cu:51-130): fp32 host arrays in, device-side fp8 conversion
    M, N, K = 128, 128, 256          # check.cu's own active shape (check.cu:137-139)
    rng = np.random.default_rng(7)
    Af = rng.uniform(-5, 5, M * K).astype(np.float32)
    Bf = rng.uniform(-5, 5, N * K).astype(np.float32)
    a_s = rng.uniform(-5, 5, M * K // 128).astype(np.float32)
    b_s = rng.uniform(-5, 5, K // 128).astype(np.float32)
    ref = h.oracle_gemm(f.float_to_e4m3fn(Af), f.float_to_e4m3fn(Bf), a_s, b_s, M, N, K)
    c_ref_kernel = f.gemmGPU(Af, Bf, a_s, b_s, M, N, K, option=2)
    assert np.array_equal(c_ref_kernel, ref)                       # device conversion == host conversion too
    for option in (0, 1):
        got = f.gemmGPU(Af, Bf, a_s, b_s, M, N, K, option=option)
        assert_parity(ref, got, "gemmGPU option %d" % option)
        # the reference's own acceptance test: absolute tolerance 100 against the ref kernel (check.cu:174)
        assert np.abs(h.bf16_bits_to_f32(got) - h.bf16_bits_to_f32(c_ref_kernel)).max() <= 100.0


def test_host_context_end_to_end():
    M, N, K = 1024, 576, 7168
    ctx = f.HostContext(M, N, K)
    try:
        A, B, a_s, b_s = h.make_inputs(M, N, K, seed=55)
        hA = ctx.buffer(0, M * K, np.uint8); hA[:] = A
        hB = ctx.buffer(1, N * K, np.uint8); hB[:] = B
        hAs = ctx.buffer(2, a_s.nbytes, np.float32); hAs[:] = a_s
        hBs = ctx.buffer(3, b_s.nbytes, np.float32); hBs[:] = b_s
        hC = ctx.buffer(4, M * N * 2, np.uint16)
        for _ in range(2):
            hC[:] = 0x7FC0
            ctx.gemm(hC, hA, hB, hAs, hBs, M, N, K)
            assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), hC.reshape(M, N))
    finally:
        ctx.close()


@pytest.mark.parametrize("shape,n0,n_total", [((512, 4096, 1024), 0, 4096), ((2048, 256, 4096), 0, 256),
                                              ((2048, 192, 4096), 64, 320), ((2064, 272, 4096), 0, 272)],
                         ids=["column-chunks", "row-chunks", "row-chunks-of-a-shard", "row-chunks-ragged"])
def test_host_context_pipelined_paths(shape, n0, n_total):
    # large enough for the host call to pipeline copy-in, GEMM and copy-out over column or row chunks
    M, N, K = shape
    ctx = f.HostContext(M, N, K)
    try:
        A, Bfull, a_s, b_s = h.make_inputs(M, n_total, K, seed=57)
        B = np.ascontiguousarray(Bfull.reshape(K, n_total)[:, n0:n0 + N]).ravel()
        hA = ctx.buffer(0, M * K, np.uint8); hA[:] = A
        hB = ctx.buffer(1, N * K, np.uint8); hB[:] = B
        hAs = ctx.buffer(2, a_s.nbytes, np.float32); hAs[:] = a_s
        hBs = ctx.buffer(3, b_s.nbytes, np.float32); hBs[:] = b_s
        hC = ctx.buffer(4, M * N * 2, np.uint16)
        ref = h.oracle_gemm(A, Bfull, a_s, b_s, M, n_total, K)[:, n0:n0 + N]
        for _ in range(2):
            hC[:] = 0x7FC0
            ctx.gemm(hC, hA, hB, hAs, hBs, M, N, K, n0, n_total)
            assert_parity(np.ascontiguousarray(ref), hC.reshape(M, N))
    finally:
        ctx.close()


def test_bounded_wait_reports_a_timeout_and_leaves_the_context_usable():
    # failure detection without a GPU fault: a wait on a barrier nothing sets runs out, the kernel returns a status
    lib = f.lib()
    f.last_device_status()                                   # start from a clean record
    assert lib.fp8bs_selftest_wait_timeout(None) == 0
    with pytest.raises(f.Fp8bsError) as e:
        f.last_device_status()
    assert e.value.code == -8 and (e.value.detail & 0xFF) == 9
    f.last_device_status()                                   # the record was cleared
    # and the GPU still computes
    M, N, K = 128, 128, 256
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=2)
    assert_parity(h.oracle_gemm(A, B, a_s, b_s, M, N, K), run_gemm(A, B, a_s, b_s, M, N, K))

"""Host-side logic of the library, runnable without a GPU: the shared library loads and exports every
symbol include/fp8bs.h declares, the shape dispatch, argument checking, the input generator and the
fp8 conversions.  No kernel is launched here."""
import ctypes
import os
import re

import numpy as np
import pytest

import fp8_quant_matmul_b200 as f
from fp8_quant_matmul_b200 import api
import helpers as h

ROOT = h.ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "fp8bs.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fp8bs_[A-Za-z0-9_]+)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = f.lib()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(lib, name), "libfp8bs.so does not export " + name
    # and the Python binding covers the whole header
    assert sorted(api.exported_symbols()) == declared


def test_status_strings():
    for code in range(0, -10, -1):
        s = f.status_string(code)
        assert isinstance(s, str) and s and s != "unknown status"
    assert f.status_string(-99) == "unknown status"


def test_dispatch_policy_on_the_18_shapes():
    # large M*N -> the persistent full-K kernel; small M*N with K = 7168 -> split-K (README.md:99, 161)
    for (M, N, K) in f.SHAPES_18:
        path, splits, tile_n = f.select_path(M, N, K)
        assert path in (f.PATH_MN_LARGE, f.PATH_MN_SMALL)
        assert (tile_n & ~(f.SPLIT_WORKSPACE | f.STREAM_K | f.SHORT_K)) in (128, 256, 256 | f.TILE_PAIR)
        assert 1 <= splits <= K // 128
        # the mn_small family cuts K: into `splits` ranges per tile, or (stream-K) evenly over the SMs
        assert (path == f.PATH_MN_SMALL) == (splits > 1 or bool(tile_n & f.STREAM_K))
        ws = f.workspace_bytes(M, N, K)
        assert (ws > 0) == bool(tile_n & (f.SPLIT_WORKSPACE | f.STREAM_K))   # cluster reductions need no workspace
        if tile_n & f.STREAM_K:
            assert ws == 65536 + min(148, (M // 128) * -(-N // (tile_n & 0xFFF)) * (K // 128) // 4) * (tile_n & 0xFFF) * 128 * 4
    assert f.select_path(6144, 4608, 7168)[0] == f.PATH_MN_LARGE
    assert f.select_path(1024, 512, 7168)[0] == f.PATH_MN_SMALL
    assert f.select_path(1024, 576, 7168)[0] == f.PATH_MN_SMALL
    assert f.select_path(6144, 7168, 256)[:2] == (f.PATH_MN_LARGE, 1)
    # K <= 256: the kernel that keeps a tile's partial sums in tensor memory, up to three tiles per SM at K = 256
    assert f.select_path(1024, 7168, 256) == (f.PATH_MN_LARGE, 1, 256 | f.SHORT_K)
    assert f.select_path(6144, 7168, 256) == (f.PATH_MN_LARGE, 1, 256)
    assert f.select_path(6144, 7168, 128) == (f.PATH_MN_LARGE, 1, 256 | f.SHORT_K)


def test_dispatch_is_deterministic_and_validates():
    assert f.select_path(1024, 1536, 7168) == f.select_path(1024, 1536, 7168)
    with pytest.raises(f.Fp8bsError) as e:
        f.select_path(1024, 1536, 100)          # K % 128 != 0 (mn_large.hip:17)
    assert e.value.code == -2
    with pytest.raises(f.Fp8bsError) as e:
        f.select_path(1000, 1536, 128)          # M % 16 != 0
    assert e.value.code == -3
    assert f.workspace_bytes(1024, 512, 7168, f.PATH_MN_SMALL, 4, 128 | f.SPLIT_WORKSPACE) == 65536 + 8 * 4 * 4 * 128 * 128 * 4
    assert f.workspace_bytes(1024, 512, 7168, f.PATH_MN_SMALL, 4, 128) == 0          # reduced inside a cluster
    assert f.workspace_bytes(1024, 512, 7168, f.PATH_MN_SMALL, 9, 128) > 0           # more than 8 splits: workspace
    assert f.workspace_bytes(1024, 512, 7168, f.PATH_MN_LARGE, 1, 0) == 0
    assert f.workspace_bytes(1024, 512, 7168, f.PATH_MN_LARGE, 2, 0) == 0     # invalid combination -> 0


def test_argument_errors_come_back_as_codes_without_touching_a_device():
    lib = f.lib()
    fake = ctypes.c_void_p(0x1000)
    # NULL pointers
    assert lib.fp8bs_gemm(None, fake, fake, fake, fake, 128, 128, 128, None, 0, None) == -1
    assert lib.fp8bs_gemm_ref(fake, fake, fake, fake, None, 128, 128, 128, None) == -1
    # shape and alignment
    assert lib.fp8bs_gemm(fake, fake, fake, fake, fake, 128, 128, 100, None, 0, None) == -2
    assert lib.fp8bs_gemm(fake, fake, fake, fake, fake, 0, 128, 128, None, 0, None) == -2
    assert lib.fp8bs_gemm(fake, fake, fake, fake, fake, 120, 128, 128, None, 0, None) == -3
    assert lib.fp8bs_gemm(ctypes.c_void_p(0x1001), fake, fake, fake, fake, 128, 128, 128, None, 0, None) == -3
    # path / splits / tile / shard arguments
    ex = lib.fp8bs_gemm_ex
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 7, 0, 0, None, 0, None) == -5
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 2, 3, 0, None, 0, None) == -5    # splits > K/128
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 1, 2, 0, None, 0, None) == -5    # mn_large cannot split
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 0, 0, 192, None, 0, None) == -5  # tile width
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 0, 0, 128 | f.TILE_PAIR, None, 0, None) == -5  # pairs are 256 wide
    assert ex(fake, fake, fake, fake, fake, 128, 128, 384, 0, 128, 0, 0, f.SHORT_K, None, 0, None) == -5        # short K: K <= 256
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 0, 0, 128 | f.SHORT_K, None, 0, None) == -5  # ... 256 wide
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 2, 2, f.SHORT_K, None, 0, None) == -5        # ... K is not cut
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 32, 256, 0, 0, 0, None, 0, None) == -5   # n0 % 64
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 192, 256, 0, 0, 0, None, 0, None) == -5  # shard beyond n_total
    # forced split-K without a workspace
    assert ex(fake, fake, fake, fake, fake, 128, 128, 256, 0, 128, 2, 2, 128 | f.SPLIT_WORKSPACE, None, 0, None) == -4
    assert lib.fp8bs_workspace_init(None, 1 << 20, None) == -1
    assert lib.fp8bs_workspace_init(fake, 16, None) == -4


def test_no_device_is_an_error_not_a_fallback():
    torch = pytest.importorskip("torch")
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    fake = ctypes.c_void_p(0x1000)
    assert f.lib().fp8bs_gemm_mn_large(fake, fake, fake, fake, fake, 128, 128, 128, None) == -6
    with pytest.raises(RuntimeError):
        f.gemm(torch.zeros(128 * 128, dtype=torch.uint8), torch.zeros(128 * 128, dtype=torch.uint8),
               torch.ones(128), torch.ones(1), M=128, N=128, K=128)


def test_float_to_e4m3fn_matches_torch_rounding():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(1)
    x = np.concatenate([
        rng.standard_normal(4000).astype(np.float32),
        (rng.standard_normal(4000) * 100).astype(np.float32),
        (rng.standard_normal(2000) * 0.01).astype(np.float32),
        f.e4m3fn_to_float(np.arange(256, dtype=np.uint8)[np.r_[0:0x7F, 0x80:0xFF]]),        # every finite value
        np.array([2.0 ** -10, 2.0 ** -9 * 1.5, 2.0 ** -9 * 2.5, 447.9, 448.0, 1.0625, 1.1875, -1.0625], np.float32),
    ])
    x = x[np.abs(x) <= 448]
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = f.float_to_e4m3fn(x)
    # +0/-0: both encodings of zero are accepted for values that round to zero
    same = (want == got) | (((want | got) & 0x7F) == 0)
    assert same.all(), (x[~same][:5], want[~same][:5], got[~same][:5])
    # saturation instead of NaN above the range
    assert f.float_to_e4m3fn(np.array([1e6, -1e6, np.inf], np.float32)).tolist() == [0x7E, 0xFE, 0x7E]
    assert f.float_to_e4m3fn(np.array([np.nan], np.float32))[0] == 0x7F


def test_decode_matches_oracle_table():
    got = f.e4m3fn_to_float(np.arange(256, dtype=np.uint8))
    want = np.array([h.oracle_lib().oracle_e4m3fn_to_float(i) for i in range(256)], dtype=np.float32)
    assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)]) and np.array_equal(np.isnan(got), np.isnan(want))


def test_generator_distribution_and_value_set():
    b = f.gen_normal_e4m3(200000, 7)
    assert np.array_equal(b, f.gen_normal_e4m3(200000, 7))                  # seeded
    assert not np.array_equal(b, f.gen_normal_e4m3(200000, 8))
    assert np.array_equal(b[:1001], f.gen_normal_e4m3(1001, 7))             # counter-based: prefix-stable
    v = f.e4m3fn_to_float(b)
    assert not np.isnan(v).any() and abs(v.mean()) < 0.02 and abs(v.std() - 1.0) < 0.02
    nz = np.abs(v[v != 0])
    assert nz.min() >= 2.0 ** -6 and nz.max() <= 240.0 and not (b == 0x80).any()     # common to fn and fnuz
    # every generated value also exists in e4m3fnuz with byte + 8
    L = h.oracle_lib()
    for byte in np.unique(b):
        if byte & 0x7F:
            assert L.oracle_e4m3fnuz_to_float(int(byte) + 8) == L.oracle_e4m3fn_to_float(int(byte))
    s = f.gen_uniform_f32(100000, 3, 0.01, 1.0)
    assert s.min() >= 0.01 and s.max() < 1.0 and abs(s.mean() - 0.505) < 0.01


def test_fnuz_to_fn_preserves_values():
    L = h.oracle_lib()
    ok_bytes, bad_bytes = [], []
    fn_values = {L.oracle_e4m3fn_to_float(i) for i in range(256) if i not in (0x7F, 0xFF)}
    for bb in range(256):
        v = L.oracle_e4m3fnuz_to_float(bb)
        (ok_bytes if (v == v and v in fn_values) else bad_bytes).append(bb)
    assert len(bad_bytes) == 1 + 16          # NaN, and the 8 odd multiples of 2^-10 below 2^-6 with either sign
    src = np.array(ok_bytes, dtype=np.uint8)
    dst = f.fnuz_to_fn(src)
    for s, d in zip(src, dst):
        assert L.oracle_e4m3fnuz_to_float(int(s)) == L.oracle_e4m3fn_to_float(int(d))
    for bb in bad_bytes:
        with pytest.raises(f.Fp8bsError) as e:
            f.fnuz_to_fn(np.array([0x40, bb], dtype=np.uint8))
        assert e.value.code == -9 and e.value.bad_index == 1


def test_stream_k_is_never_chosen_above_one_wave_of_tiles():
    # measured: with more tiles than SMs the stream-K schedule loses its L2 sharing and runs up to 2x slower than the
    # tile-per-CTA kernel, so the dispatcher offers it only on request there
    from fp8_quant_matmul_b200.shard import plan_n_shards
    for M in (1024, 6144, 16384):
        for (N, K) in ((1536, 7168), (3072, 1536), (576, 7168), (7168, 256), (7168, 2048), (4608, 7168), (7168, 2304),
                       (512, 7168), (4096, 512)):
            for g in (1, 2, 4, 8):
                for (_, nl) in set(plan_n_shards(N, g)):
                    path, splits, tile_n = f.select_path(M, nl, K)
                    if tile_n & f.STREAM_K:
                        assert (M // 128) * -(-nl // (tile_n & 0xFFF)) <= 148
                    # the library only ever asks for a workspace it would use
                    assert (f.workspace_bytes(M, nl, K) > 0) == bool(tile_n & (f.SPLIT_WORKSPACE | f.STREAM_K))
    # forcing it is always possible, and it then reports its workspace
    assert f.workspace_bytes(16384, 1536, 7168, f.PATH_MN_SMALL, 1, 256 | f.STREAM_K) == 65536 + 148 * 256 * 128 * 4


def test_dispatch_for_a_smaller_gpu_never_needs_more_resident_ctas_than_sms():
    # stream-K CTAs wait (bounded) for partial tiles of other CTAs and the CTAs of a cluster wait for each other at a
    # hardware barrier: both need all of them resident together, whatever the SM count the context exposes
    from fp8_quant_matmul_b200.shard import plan_n_shards
    shapes = set()
    for M in (1024, 6144):
        for (N, K) in ((1536, 7168), (576, 7168), (7168, 256), (4608, 7168), (512, 7168), (4096, 512)):
            for g in (1, 8):
                shapes |= {(M, nl, K) for (_, nl) in plan_n_shards(N, g)}
    for sms in (148, 132, 74, 36, 8, 1):
        for (M, N, K) in sorted(shapes):
            path, splits, tile_n, ctas = f.select_path_sms(M, N, K, sms)
            assert ctas <= sms, (sms, M, N, K, splits, tile_n, ctas)
            assert path in (f.PATH_MN_LARGE, f.PATH_MN_SMALL) and 1 <= splits <= K // 128
    # a full B200 and the default model agree
    for (M, N, K) in f.SHAPES_18:
        assert f.select_path_sms(M, N, K, 148)[:3] == f.select_path(M, N, K)
    with pytest.raises(f.Fp8bsError):
        f.select_path_sms(1024, 512, 7168, 0)


def test_short_k_dispatch_rule():
    # K = 128: always the kernel that keeps a tile's partial sums in tensor memory; K = 256: up to three 128 x 256 tiles per SM
    for (M, N) in ((128, 64), (1024, 7168), (6144, 7168), (16384, 7168)):
        path, splits, tile_n = f.select_path(M, N, 128)
        assert (path, splits, tile_n) == (f.PATH_MN_LARGE, 1, 256 | f.SHORT_K)
    sms = 148
    for (M, N) in ((1024, 7168), (2048, 7168), (1536, 9472), (6144, 7168), (6144, 3584), (6144, 1792)):
        tiles = -(-M // 128) * -(-N // 256)
        path, splits, tile_n = f.select_path(M, N, 256)
        assert path == f.PATH_MN_LARGE and splits == 1
        assert bool(tile_n & f.SHORT_K) == (tiles <= 3 * sms), (M, N, tiles, hex(tile_n))
        assert f.workspace_bytes(M, N, 256) == 0
    # the rule follows the SM count it is asked about
    p, s_, t, _ = f.select_path_sms(6144, 7168, 256, 148)
    assert not (t & f.SHORT_K)
    p, s_, t, _ = f.select_path_sms(1024, 7168, 256, 36)
    assert not (t & f.SHORT_K)                                          # 224 tiles on 36 SMs: more than three per SM
    # longer K never takes it
    for K in (384, 512, 7168):
        assert not (f.select_path(1024, 7168, K)[2] & f.SHORT_K)
    assert f.workspace_bytes(1024, 7168, 256, f.PATH_MN_LARGE, 1, f.SHORT_K) == 0

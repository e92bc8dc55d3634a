"""The CPU checker (oracle/) pinned against everything the reference gives for this operator:
torch's float8 decode tables, the reference's own host code (genMat, gemmCPU, quantize.py,
through the committed golden fixtures) and hand-derived known answers for each index formula
of ref_kernel (check.cu:36-48)."""
import os

import numpy as np
import pytest

import helpers as h

GOLD = h.GOLDEN_DIR


def _load(name):
    return np.load(os.path.join(GOLD, name))


def test_e4m3_decode_tables_match_torch_golden():
    t = _load("e4m3_tables.npz")
    L = h.oracle_lib()
    fn = np.array([L.oracle_e4m3fn_to_float(i) for i in range(256)], dtype=np.float32)
    fnuz = np.array([L.oracle_e4m3fnuz_to_float(i) for i in range(256)], dtype=np.float32)
    assert np.array_equal(np.isnan(fn), np.isnan(t["fn"])) and np.array_equal(np.isnan(fnuz), np.isnan(t["fnuz"]))
    assert np.array_equal(fn[~np.isnan(fn)], t["fn"][~np.isnan(fn)])
    assert np.array_equal(fnuz[~np.isnan(fnuz)], t["fnuz"][~np.isnan(fnuz)])


def test_e4m3_decode_tables_match_torch_live():
    torch = pytest.importorskip("torch")
    b = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    L = h.oracle_lib()
    for dt, fn in ((torch.float8_e4m3fn, L.oracle_e4m3fn_to_float), (torch.float8_e4m3fnuz, L.oracle_e4m3fnuz_to_float)):
        want = b.view(dt).to(torch.float32).numpy()
        got = np.array([fn(i) for i in range(256)], dtype=np.float32)
        ok = np.isnan(want) == np.isnan(got)
        assert ok.all() and np.array_equal(want[~np.isnan(want)], got[~np.isnan(want)])


def test_dialect_relation_fn_is_twice_fnuz():
    # for every byte except the NaN encodings, e4m3fn(b) == 2 * e4m3fnuz(b)
    L = h.oracle_lib()
    for b in range(256):
        if b in (0x7F, 0x80, 0xFF):
            continue
        assert L.oracle_e4m3fn_to_float(b) == 2.0 * L.oracle_e4m3fnuz_to_float(b)


def test_bf16_round_to_nearest_even():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 50,
                        np.array([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.3895314e38, np.inf, -np.inf], np.float32)])
    want = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got = np.array([h.oracle_lib().oracle_float_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(want, got)
    assert np.array_equal(h.f32_to_bf16_bits(x), want)


@pytest.mark.parametrize("M,N,K", [(16, 16, 128), (48, 208, 384), (33, 576, 256), (130, 70, 128)])
def test_blocked_routine_is_bit_identical_to_naive_statement(M, N, K):
    rng = np.random.default_rng(M * 1000 + N)
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=11 + M)
    a_s = rng.uniform(-5, 5, a_s.size).astype(np.float32)      # negative scales occur in check.cu:161-162
    b_s = rng.uniform(-5, 5, b_s.size).astype(np.float32)
    assert np.array_equal(h.oracle_gemm(A, B, a_s, b_s, M, N, K), h.oracle_gemm_naive(A, B, a_s, b_s, M, N, K))


def test_row_subset_and_shard_offsets():
    M, N, K = 64, 320, 256
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=3)
    full = h.oracle_gemm(A, B, a_s, b_s, M, N, K)
    rows = np.array([5, 0, 63, 17], dtype=np.int32)
    assert np.array_equal(h.oracle_gemm(A, B, a_s, b_s, M, N, K, rows=rows), full[rows])
    # columns [192, 320) as an N-shard with n0 = 192 (straddles a 128-wide b_scale block)
    Bm = B.reshape(K, N)
    shard = np.ascontiguousarray(Bm[:, 192:320]).ravel()
    got = h.oracle_gemm(A, shard, a_s, b_s, M, 128, K, n0=192, n_total=N)
    assert np.array_equal(got, full[:, 192:320])


def test_kat_unit_scales_small_integers_exact():
    # K = 128, unit scales, operands in {-2..2}: every block sum is a small integer, exact in bf16
    M, N, K = 32, 48, 128
    rng = np.random.default_rng(5)
    vals = np.array([h.e4m3fn_byte(v) for v in (-2.0, -1.0, 0.0, 1.0, 2.0)], dtype=np.uint8)
    ai, bi = rng.integers(0, 5, (K, M)), rng.integers(0, 5, (K, N))
    A, B = vals[ai].ravel(), vals[bi].ravel()
    want = (ai - 2).T.astype(np.int64) @ (bi - 2).astype(np.int64)
    assert np.abs(want).max() < 256
    got = h.bf16_bits_to_f32(h.oracle_gemm(A, B, np.ones(M, np.float32), np.ones(1, np.float32), M, N, K))
    assert np.array_equal(got, want.astype(np.float32))


def test_kat_one_hot_pins_every_index_formula():
    # A is non-zero at one (m, k), B at one (n, k): C has exactly one non-zero element and its value
    # names the a_scale / b_scale entries used (check.cu:42-48, sn = ceil(N/128) for N = 576)
    M, N, K = 32, 576, 384
    sn, KB = (N + 127) // 128, K // 128
    a_s = (1.0 + np.arange(M * KB, dtype=np.float32))            # a_scale[m + M*kb] = 1 + m + M*kb
    b_s = (0.5 + np.arange(sn * KB, dtype=np.float32)) * 0.25      # b_scale[nb + sn*kb]
    for (m, n, k) in [(0, 0, 0), (31, 575, 383), (7, 513, 130), (20, 127, 255), (3, 128, 256)]:
        A = np.zeros(M * K, np.uint8)
        B = np.zeros(N * K, np.uint8)
        A[m + M * k] = h.e4m3fn_byte(3.0)
        B[n + N * k] = h.e4m3fn_byte(-1.5)
        C = h.bf16_bits_to_f32(h.oracle_gemm(A, B, a_s, b_s, M, N, K))
        kb, nb = k // 128, n // 128
        want = np.float32(np.float32(np.float32(-4.5) * a_s[m + M * kb]) * b_s[nb + sn * kb])
        assert np.count_nonzero(C) == 1
        assert C[m, n] == h.bf16_bits_to_f32(h.f32_to_bf16_bits(np.array([want])))[0]


def test_kat_scale_only():
    # all elements 1.0: C[m,n] = 128 * sum_kb a_scale[m,kb] * b_scale[n/128,kb]
    M, N, K = 16, 256, 512
    one = h.e4m3fn_byte(1.0)
    A, B = np.full(M * K, one, np.uint8), np.full(N * K, one, np.uint8)
    _, _, a_s, b_s = h.make_inputs(M, N, K, seed=9, scale_lo=-1.0, scale_hi=1.0)
    got = h.bf16_bits_to_f32(h.oracle_gemm(A, B, a_s, b_s, M, N, K))
    a2, b2 = a_s.reshape(K // 128, M), b_s.reshape(K // 128, 2)
    want = np.zeros((M, N), np.float32)
    for kb in range(K // 128):
        want += (np.float32(128.0) * a2[kb][:, None]) * np.repeat(b2[kb], 128)[None, :]
    assert np.array_equal(got, h.bf16_bits_to_f32(h.f32_to_bf16_bits(want)))


def test_golden_genmat_first_values():
    # the reference's seeded generator (utils.h:25-33) under libstdc++
    ref = h.ref_lib()
    first = _load("genmat_kat.npz")["first64"]
    assert np.allclose(first[:8], [-4.99945, 4.20765, -2.10763, -2.89449, 2.29371, 0.327143, -1.70688, 2.52053],
                       atol=1e-5)
    if ref is not None:
        out = np.empty(64, np.float32)
        ref.ref_genMat(out.ctypes.data, out.size)
        assert np.array_equal(out, first)


def test_golden_check_case_against_reference_gemmcpu():
    # check.cu's own configuration; expected values came from the reference's gemmCPU on dequantised operands
    g = _load("check_case.npz")
    M, N, K = int(g["M"]), int(g["N"]), int(g["K"])
    got = h.oracle_gemm(g["A"], g["B"], g["a_scale"], g["b_scale"], M, N, K)
    bad, first, maxerr = h.mismatches(g["C_gemmcpu_bf16"], got)
    assert bad == 0, (bad, first, maxerr)
    # and under the reference's own criterion: absolute tolerance 100 (check.cu:174)
    assert np.abs(h.bf16_bits_to_f32(got) - g["C_gemmcpu_f32"]).max() <= 100.0


def test_golden_quantize_case_against_reference_quantizer():
    # operands and inverse scales produced by the reference's quantize.py; expected C from float64
    g = _load("quantize_case.npz")
    M, N, K = int(g["M"]), int(g["N"]), int(g["K"])
    got = h.oracle_gemm(g["A"], g["B"], g["a_scale"], g["b_scale"], M, N, K)
    bad, first, maxerr = h.mismatches(g["C_bf16"], got)
    assert bad == 0, (bad, first, maxerr)


def test_reference_gemmcpu_path_agrees_live():
    # second, independent CPU path: dequantise -> the reference's gemmCPU (utils.h:65-76) -> bf16
    ref = h.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built (no reference checkout)")
    import fp8_quant_matmul_b200 as f
    M, N, K = 64, 192, 256
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=21)
    Av = f.e4m3fn_to_float(A).reshape(K, M).T * np.repeat(a_s.reshape(K // 128, M).T, 128, axis=1)
    Bv = f.e4m3fn_to_float(B).reshape(K, N) * np.repeat(np.repeat(b_s.reshape(K // 128, 2), 128, axis=0), 128, axis=1)[:, :N]
    Ad, Bd = np.ascontiguousarray(Av, np.float32), np.ascontiguousarray(Bv, np.float32)
    Cf = np.empty((M, N), np.float32)
    ref.ref_gemmCPU(Cf.ctypes.data, Ad.ctypes.data, Bd.ctypes.data, M, N, K)
    Cm = np.empty((M, N), np.float32)
    ref.ref_gemmCPU_mt(Cm.ctypes.data, Ad.ctypes.data, Bd.ctypes.data, M, N, K, 3)
    assert np.array_equal(Cf, Cm)
    bad, first, maxerr = h.mismatches(h.f32_to_bf16_bits(Cf), h.oracle_gemm(A, B, a_s, b_s, M, N, K))
    assert bad == 0, (bad, first, maxerr)


def test_f64_tiebreaker_close_to_fp32_oracle():
    M, N, K = 16, 64, 512
    A, B, a_s, b_s = h.make_inputs(M, N, K, seed=4)
    out = np.empty((M, N), np.float64)
    rc = h.oracle_lib().oracle_gemm_rows_f64(A.ctypes.data, B.ctypes.data, a_s.ctypes.data, b_s.ctypes.data,
                                             M, N, K, 0, 1, None, M, out.ctypes.data, 0)
    assert rc == 0
    _, f32 = h.oracle_gemm(A, B, a_s, b_s, M, N, K, want_f32=True)
    assert np.abs(out - f32).max() <= 1e-4 * max(1.0, np.abs(out).max())

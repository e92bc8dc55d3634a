"""Shared test helpers: ctypes access to the CPU checker in oracle/, bf16 bit helpers, seeded inputs.

Only tests (and the benchmark's CPU-baseline leg) may touch oracle/; the library never does.
"""
import ctypes as C
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")

RTOL, ATOL = 2e-2, 1e-3      # the parity tolerance of the operator (bf16 output, fp32 accumulation)

_oracle = None
_ref = None


def oracle_lib():
    global _oracle
    if _oracle is None:
        L = C.CDLL(os.path.join(ORACLE_DIR, "liboracle.so"))
        L.oracle_gemm_rows_ex.restype = C.c_int
        L.oracle_gemm_rows_ex.argtypes = ([C.c_void_p] * 4 + [C.c_int] * 5 +
                                          [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_int])
        L.oracle_gemm_naive.restype = C.c_int
        L.oracle_gemm_naive.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4
        L.oracle_gemm_rows_f64.restype = C.c_int
        L.oracle_gemm_rows_f64.argtypes = ([C.c_void_p] * 4 + [C.c_int] * 5 + [C.c_void_p, C.c_int, C.c_void_p, C.c_int])
        L.oracle_e4m3fn_to_float.restype = C.c_float
        L.oracle_e4m3fn_to_float.argtypes = [C.c_uint8]
        L.oracle_e4m3fnuz_to_float.restype = C.c_float
        L.oracle_e4m3fnuz_to_float.argtypes = [C.c_uint8]
        L.oracle_float_to_bf16.restype = C.c_uint16
        L.oracle_float_to_bf16.argtypes = [C.c_float]
        L.oracle_allclose_bf16.restype = C.c_size_t
        L.oracle_allclose_bf16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float,
                                           C.POINTER(C.c_size_t), C.POINTER(C.c_float)]
        L.oracle_num_threads.restype = C.c_int
        _oracle = L
    return _oracle


def ref_lib():
    """The reference's own host helpers (oracle/_ref), or None when they were not built."""
    global _ref
    path = os.path.join(ORACLE_DIR, "_ref", "libfp8bs_ref.so")
    if _ref is None and os.path.exists(path):
        L = C.CDLL(path)
        L.ref_genMat.argtypes = [C.c_void_p, C.c_size_t]
        L.ref_gemmCPU.argtypes = [C.c_void_p] * 3 + [C.c_size_t] * 3
        L.ref_gemmCPU_mt.argtypes = [C.c_void_p] * 3 + [C.c_size_t] * 3 + [C.c_int]
        L.ref_row_to_col_major.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        L.ref_allClose.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_float]
        _ref = L
    return _ref


def oracle_gemm(A, B, a_scale, b_scale, M, N, K, n0=0, n_total=None, rows=None, dialect=0, want_f32=False):
    """bf16 bit patterns [rows, N] of the checker's result (all rows when rows is None)."""
    n_total = N if n_total is None else n_total
    sn = (n_total + 127) // 128
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    a_scale = np.ascontiguousarray(a_scale, dtype=np.float32)
    b_scale = np.ascontiguousarray(b_scale, dtype=np.float32)
    assert A.size == M * K and B.size == N * K and a_scale.size == M * (K // 128) and b_scale.size == sn * (K // 128)
    if rows is None:
        nrows, rp = M, None
    else:
        rows = np.ascontiguousarray(rows, dtype=np.int32)
        nrows, rp = len(rows), rows.ctypes.data
    out = np.empty((nrows, N), dtype=np.uint16)
    f32 = np.empty((nrows, N), dtype=np.float32) if want_f32 else None
    rc = oracle_lib().oracle_gemm_rows_ex(A.ctypes.data, B.ctypes.data, a_scale.ctypes.data, b_scale.ctypes.data,
                                          M, N, K, n0, sn, rp, nrows, out.ctypes.data,
                                          f32.ctypes.data if want_f32 else None, dialect, 0)
    assert rc == 0
    return (out, f32) if want_f32 else out


def oracle_gemm_naive(A, B, a_scale, b_scale, M, N, K, dialect=0):
    out = np.empty((M, N), dtype=np.uint16)
    rc = oracle_lib().oracle_gemm_naive(A.ctypes.data, B.ctypes.data, a_scale.ctypes.data, b_scale.ctypes.data,
                                        out.ctypes.data, M, N, K, dialect)
    assert rc == 0
    return out


def bf16_bits_to_f32(u):
    return (np.ascontiguousarray(u, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    f = oracle_lib().oracle_float_to_bf16
    u = x.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r[nan] = 0x7FC0
    return r


def mismatches(ref_bits, got_bits, rtol=RTOL, atol=ATOL):
    """Number of elements with |got - ref| > atol + rtol*|ref| (NaN counts), plus the first index."""
    ref_bits = np.ascontiguousarray(ref_bits, dtype=np.uint16)
    got_bits = np.ascontiguousarray(got_bits, dtype=np.uint16)
    assert ref_bits.shape == got_bits.shape
    first, maxerr = C.c_size_t(0), C.c_float(0)
    bad = oracle_lib().oracle_allclose_bf16(ref_bits.ctypes.data, got_bits.ctypes.data, ref_bits.size, rtol, atol,
                                            C.byref(first), C.byref(maxerr))
    return int(bad), int(first.value), float(maxerr.value)


def make_inputs(M, N, K, seed, n_total=None, scale_lo=0.01, scale_hi=1.0):
    """Seeded operator inputs with the benchmark's distributions (see fp8bs_gen_* in include/fp8bs.h)."""
    import fp8_quant_matmul_b200 as f
    n_total = N if n_total is None else n_total
    A = f.gen_normal_e4m3(M * K, seed)
    B = f.gen_normal_e4m3(N * K, seed + 1)
    a_scale = f.gen_uniform_f32(M * (K // 128), seed + 2, scale_lo, scale_hi)
    b_scale = f.gen_uniform_f32(((n_total + 127) // 128) * (K // 128), seed + 3, scale_lo, scale_hi)
    return A, B, a_scale, b_scale


def e4m3fn_byte(value):
    """The e4m3fn byte of an exactly representable value."""
    import fp8_quant_matmul_b200 as f
    b = int(f.float_to_e4m3fn(np.array([value], dtype=np.float32))[0])
    assert float(f.e4m3fn_to_float(np.array([b], dtype=np.uint8))[0]) == float(value)
    return b

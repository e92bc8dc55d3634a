"""Generates the golden fixtures in this directory.  Run once, on a machine that has a checkout of the
reference project, after `make -C oracle REF=/path/to/reference` has built oracle/_ref:

    python tests/golden/make_golden.py /path/to/reference

The reference stores no expected outputs for its operator, so every fixture here is an
output of reference CODE run on seeded inputs:
  e4m3_tables.npz     decode tables of torch.float8_e4m3fn / float8_e4m3fnuz (all 256 bytes),
                      the two element dialects involved (check.cu:17-21 uses fnuz)
  genmat_kat.npz      first 64 values of the reference's genMat (utils.h:25-33, seed 7)
  check_case.npz      check.cu's own test configuration (M = N = 128, K = 256, inputs from
                      genMat exactly as check.cu:155-167 builds them), fp8 bytes made by
                      torch's float8_e4m3fn cast, expected C from the reference's gemmCPU
                      (utils.h:65-76) on the dequantised operands -> bf16
  quantizer_case.npz  fp32 matrices X, W and what the reference's quantize.py makes of them (e4m3fn bytes and inverse
                      scales, re-laid out as the GEMM reads them): the expected output of the device-side quantisers
  quantize_case.npz   inputs produced by the reference's quantize.py (row-wise 1x128 scales
                      for A, quantize.py:43-67; 128x128 block scales for B, quantize.py:16-41,
                      dtype e4m3fn) from a seeded fp32 matrix pair, expected C from a
                      float64 matmul of the dequantised operands
"""
import ctypes as C
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if len(sys.argv) != 2 or not os.path.isfile(os.path.join(sys.argv[1], "quantize.py")):
    raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference   (the checkout that holds quantize.py)")
REF = sys.argv[1]
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import helpers  # noqa: E402


def f32_to_bf16_bits(x):
    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32)).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def tables():
    b = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    fn = b.view(torch.float8_e4m3fn).to(torch.float32).numpy()
    fnuz = b.view(torch.float8_e4m3fnuz).to(torch.float32).numpy()
    np.savez(os.path.join(HERE, "e4m3_tables.npz"), fn=fn, fnuz=fnuz)


def genmat(ref):
    out = np.empty(64, dtype=np.float32)
    ref.ref_genMat(out.ctypes.data, out.size)
    np.savez(os.path.join(HERE, "genmat_kat.npz"), first64=out)


def check_case(ref):
    M, N, K = 128, 128, 256
    g = np.empty(max(M * K, K * N), dtype=np.float32)
    ref.ref_genMat(g.ctypes.data, g.size)
    matA = g[:M * K].copy()                      # row-major M x K                (check.cu:155)
    matB = g[:K * N].copy()                      # K x N row-major = N x K col-major (check.cu:156)
    matAs = g[:M * K // 128].copy()              # check.cu:161, passed untransposed (check.cu:171)
    matBs = g[:(K // 128) * ((N + 127) // 128)].copy()   # check.cu:162
    A_col = np.empty_like(matA)
    ref.ref_row_to_col_major(matA.ctypes.data, A_col.ctypes.data, M, K)   # check.cu:164-165
    A8 = torch.from_numpy(A_col).to(torch.float8_e4m3fn)
    B8 = torch.from_numpy(matB).to(torch.float8_e4m3fn)
    A_bytes = A8.view(torch.uint8).numpy().copy()
    B_bytes = B8.view(torch.uint8).numpy().copy()
    # dequantise: A[m,k]*as[m,kb], B[n,k]*bs[nb,kb]; then the reference's fp32 gemmCPU
    Av = A8.to(torch.float32).numpy().reshape(K, M).T            # [M, K]
    Bv = B8.to(torch.float32).numpy().reshape(K, N)              # [K, N]
    as_mk = np.repeat(matAs.reshape(K // 128, M).T, 128, axis=1)             # [M, K]
    bs_kn = np.repeat(np.repeat(matBs.reshape(K // 128, (N + 127) // 128), 128, axis=0), 128, axis=1)[:, :N]
    Ad = np.ascontiguousarray(Av * as_mk, dtype=np.float32)
    Bd = np.ascontiguousarray(Bv * bs_kn, dtype=np.float32)
    Cf = np.empty((M, N), dtype=np.float32)
    ref.ref_gemmCPU(Cf.ctypes.data, Ad.ctypes.data, Bd.ctypes.data, M, N, K)
    np.savez(os.path.join(HERE, "check_case.npz"), M=M, N=N, K=K, A=A_bytes, B=B_bytes, a_scale=matAs,
             b_scale=matBs, C_gemmcpu_bf16=f32_to_bf16_bits(Cf), C_gemmcpu_f32=Cf)


def quantize_case():
    spec = importlib.util.spec_from_file_location("ref_quantize", os.path.join(REF, "quantize.py"))
    q = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(q)
    M, N, K = 256, 384, 512
    gen = torch.Generator().manual_seed(7)
    X = torch.randn(M, K, generator=gen) * 3.0
    W = torch.randn(N, K, generator=gen) * 0.5
    A8, a_inv = q.to_float8_rowwise_scale(X, dtype=torch.float8_e4m3fn)      # [M,K], [M,K/128]
    B8, b_inv = q.to_float8_block_scale(W, dtype=torch.float8_e4m3fn)        # [N,K], [N/128,K/128]
    A_bytes = A8.view(torch.uint8).numpy().T.copy().ravel()                  # column-major: A[m + M*k]
    B_bytes = B8.view(torch.uint8).numpy().T.copy().ravel()
    a_scale = a_inv.numpy().T.copy().ravel().astype(np.float32)              # a_scale[m + M*kb]
    b_scale = b_inv.numpy().T.copy().ravel().astype(np.float32)              # b_scale[nb + sn*kb]
    Ad = A8.to(torch.float64) * a_inv.to(torch.float64).repeat_interleave(128, dim=1)
    Bd = B8.to(torch.float64) * b_inv.to(torch.float64).repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
    Cd = (Ad @ Bd.T).numpy()
    np.savez(os.path.join(HERE, "quantize_case.npz"), M=M, N=N, K=K, A=A_bytes, B=B_bytes, a_scale=a_scale,
             b_scale=b_scale, C_f64=Cd, C_bf16=f32_to_bf16_bits(Cd.astype(np.float32)))


def quantizer_case():
    """Inputs AND outputs of the reference's quantisers (fp32 input, e4m3fn output), for the device-side quantiser."""
    spec = importlib.util.spec_from_file_location("ref_quantize", os.path.join(REF, "quantize.py"))
    q = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(q)
    gen = torch.Generator().manual_seed(11)
    X = torch.randn(144, 256, generator=gen) * torch.rand(144, 1, generator=gen) * 8.0
    W = torch.randn(256, 256, generator=gen) * 0.3
    X[3, 128:] = 0.0                                         # an all-zero group: exercises the 1e-12 clamp
    A8, a_inv = q.to_float8_rowwise_scale(X, dtype=torch.float8_e4m3fn)
    B8, b_inv = q.to_float8_block_scale(W, dtype=torch.float8_e4m3fn)
    np.savez(os.path.join(HERE, "quantizer_case.npz"), X=X.numpy(), W=W.numpy(),
             A=A8.view(torch.uint8).numpy().T.copy().ravel(), a_scale=a_inv.numpy().T.copy().ravel().astype(np.float32),
             B=B8.view(torch.uint8).numpy().T.copy().ravel(), b_scale=b_inv.numpy().T.copy().ravel().astype(np.float32))


if __name__ == "__main__":
    ref = helpers.ref_lib()
    if ref is None:
        raise SystemExit("oracle/_ref/libfp8bs_ref.so missing: run `make -C oracle` with the reference mounted")
    tables()
    genmat(ref)
    check_case(ref)
    quantize_case()
    quantizer_case()
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))

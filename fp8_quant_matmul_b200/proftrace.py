"""Where the time goes inside one GEMM launch: reads the counters of the instrumented library.

    python -m fp8_quant_matmul_b200.build --profile          # builds lib/libfp8bs_prof.so (-DFP8BS_PROFILE=3)
    python -m fp8_quant_matmul_b200.proftrace M,N,K[,path,splits,tile_n] ... [--kblocks 40]

For every shape: one timed launch, per-CTA phase stamps and wait counters, and the per-K-block time line of CTA 0
(the buffer layout is documented next to the PROF_* macros in csrc/gemm_kernel.cuh).  The instrumentation costs
10-15 % per K block, so the cycle counts show proportions, not the speed of the production library.
"""
import ctypes
import os
import sys

import numpy as np

from . import api

PROF_LIB = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libfp8bs_prof.so")
COUNTERS = ["producer wait: free stage", "MMA wait: free TMEM buffer", "MMA wait: operands", "MMA loop total",
            "promotion wait: a_scale", "promotion wait: partial sums", "promotion loads + FMAs", "epilogue"]
STAMPS = ["start", "set-up done", "first operands (lead CTA)", "MMA loop done", "promotion loop done", "all stores issued",
          "exit"]


def trace(M, N, K, path=0, splits=0, tile_n=0, kblocks=40):
    import torch
    lib = api.load(PROF_LIB)
    lib.fp8bs_debug_prof.restype = ctypes.c_int
    lib.fp8bs_debug_prof.argtypes = [ctypes.c_void_p, ctypes.c_int]
    dev = torch.device("cuda:0")
    A = torch.from_numpy(api.gen_normal_e4m3(M * K, 1)).to(dev)
    B = torch.from_numpy(api.gen_normal_e4m3(N * K, 2)).to(dev)
    a_s = torch.from_numpy(api.gen_uniform_f32(M * (K // 128), 3, 0.01, 1.0)).to(dev)
    b_s = torch.from_numpy(api.gen_uniform_f32(((N + 127) // 128) * (K // 128), 4, 0.01, 1.0)).to(dev)
    C = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    for _ in range(3):
        api.gemm(A, B, a_s, b_s, C, M, N, K, path=path, splits=splits, tile_n=tile_n)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    api.gemm(A, B, a_s, b_s, C, M, N, K, path=path, splits=splits, tile_n=tile_n)
    e1.record()
    torch.cuda.synchronize()
    out = np.zeros(4096 + 16 * 128, dtype=np.int64)
    lib.fp8bs_debug_prof(ctypes.c_void_p(out.ctypes.data), out.size)
    per_cta = out[:148 * 16].reshape(148, 16)
    tr = out[4096:].reshape(16, 128)
    active = per_cta[per_cta[:, 8] > 0]
    print("M=%d N=%d K=%d path=%d splits=%d tile_n=%#x: %.1f us (one launch, instrumented build), %d CTAs" %
          (M, N, K, path, splits, tile_n, e0.elapsed_time(e1) * 1e3, len(active)))
    for i, name in enumerate(COUNTERS):
        col = active[:, i]
        print("   %-32s mean %10.0f clk   max %10d" % (name, col.mean(), col.max()))
    t0 = active[:, 8].min()
    for i, name in enumerate(STAMPS):
        col = active[:, 8 + i]
        col = col[col > 0]
        if len(col):
            print("   t[%-26s] min %8d ns   mean %8.0f   max %8d" % (name, col.min() - t0, col.mean() - t0, col.max() - t0))
    z = tr[1, 0]
    KB = K // 128
    print("   kb : stage free | TMEM free  operands  MMAs issued | a_scale  partial sums  FMAs done | warp 5: partial sums  FMAs done"
          "   (clock cycles of CTA 0, relative to its first operands)")
    for i in range(min(128, kblocks)):
        if tr[2, i] == 0:
            break
        r = [int(tr[e, i] - z) if tr[e, i] else 0 for e in (6, 0, 1, 2, 3, 4, 5, 7, 8)]
        print("   %3d: %9d | %9d %9d %9d | %9d %9d %9d | %9d %9d" % ((i,) + tuple(r)))
    units = [(int(tr[9, i] - z), int(tr[10, i] - z)) for i in range(128) if tr[9, i]]
    if units and KB <= 16:
        print("   epilogue of CTA 0's units (start, end): " + " ".join("(%d, %d)" % u for u in units[:16]))


def main(argv):
    kblocks = 40
    shapes = []
    it = iter(argv)
    for a in it:
        if a == "--kblocks":
            kblocks = int(next(it))
        else:
            shapes.append([int(x, 0) for x in a.split(",")])
    if not shapes:
        raise SystemExit(__doc__)
    for s in shapes:
        trace(*s, kblocks=kblocks)


if __name__ == "__main__":
    main(sys.argv[1:])

"""fp8_quant_matmul_b200 -- B200-native row-wise block-scaled FP8 GEMM.

    C[M,N] (bf16) = sum_kb a_scale[m,kb] * b_scale[n/128,kb] * (A[m, kb-block] . B[n, kb-block])

The work is done by hand-written sm_100a CUDA kernels in ``lib/libfp8bs.so`` (C ABI in
``include/fp8bs.h``).  This package is the Python host side: it loads that library with
ctypes and mirrors the reference's operator surface (the 8-argument kernel signature of
mn_large.hip:11 / mn_small.hip:10 and the gemmGPU wrapper of check.cu:51-130).
There is no fallback path: if the library is missing or no B200 is present, calls raise.
"""
from .api import (  # noqa: F401
    Fp8bsError,
    PATH_AUTO,
    PATH_MN_LARGE,
    PATH_MN_SMALL,
    TILE_PAIR,
    SPLIT_WORKSPACE,
    STREAM_K,
    SHORT_K,
    gemm,
    gemm_ref,
    gemm_mn_small_static,
    gemm_scatter,
    STATIC_SCRATCH_BYTES,
    gemmGPU,
    quantize_rowwise,
    quantize_block,
    HostContext,
    select_path,
    select_path_sms,
    workspace_bytes,
    gen_normal_e4m3,
    gen_uniform_f32,
    float_to_e4m3fn,
    e4m3fn_to_float,
    fnuz_to_fn,
    fnuz_to_fn_device,
    status_string,
    launch_count,
    last_device_status,
    lib,
    SHAPES_18,
)

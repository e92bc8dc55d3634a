"""ctypes binding of libfp8bs.so and the Python mirror of the reference's operator surface.

Device memory, streams and (in the benchmark) torch.distributed come from PyTorch; all
arithmetic happens in the library's CUDA kernels.
"""
import ctypes
import os

import numpy as np

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_PKG_DIR, "lib", "libfp8bs.so")

PATH_AUTO, PATH_MN_LARGE, PATH_MN_SMALL = 0, 1, 2
TILE_PAIR = 0x1000      # tile_n = 256 | TILE_PAIR: a 256 x 256 tile owned by a pair of CTAs
SPLIT_WORKSPACE = 0x2000  # OR into tile_n: reduce split-K partial sums through the workspace, not in a cluster
STREAM_K = 0x4000         # OR into tile_n: deal the K blocks of all tiles out evenly over the SMs (needs the workspace)
SHORT_K = 0x8000          # OR into tile_n (0 or 256): K <= 256, both K blocks of a tile stay in tensor memory

# The 18 benchmark shapes (M, N, K) of the reference's results table (README.md:15-25).
SHAPES_18 = [(m, n, k) for m in (1024, 6144)
             for (n, k) in ((1536, 7168), (3072, 1536), (576, 7168), (7168, 256), (7168, 2048),
                            (4608, 7168), (7168, 2304), (512, 7168), (4096, 512))]


class Fp8bsError(RuntimeError):
    def __init__(self, code, where):
        self.code = code
        super().__init__("%s failed: %d (%s)" % (where, code, status_string(code)))


_lib = None

_c = ctypes
_SIGS = {
    "fp8bs_gemm": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 3 + [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fp8bs_gemm_mn_large": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 3 + [_c.c_void_p]),
    "fp8bs_gemm_mn_small": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 4 + [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fp8bs_gemm_mn_small_static": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 4 + [_c.c_void_p]),
    "fp8bs_gemm_ex": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 8 + [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fp8bs_gemm_scatter": (_c.c_int, [_c.c_void_p] * 4 + [_c.POINTER(_c.c_void_p)] + [_c.c_int] * 6 + [_c.c_void_p]),
    "fp8bs_gemm_ref": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_int] * 3 + [_c.c_void_p]),
    "fp8bs_select_path": (_c.c_int, [_c.c_int] * 3 + [_c.POINTER(_c.c_int)] * 2),
    "fp8bs_select_path_sms": (_c.c_int, [_c.c_int] * 4 + [_c.POINTER(_c.c_int)] * 3),
    "fp8bs_workspace_bytes": (_c.c_size_t, [_c.c_int] * 3),
    "fp8bs_workspace_bytes_ex": (_c.c_size_t, [_c.c_int] * 6),
    "fp8bs_workspace_init": (_c.c_int, [_c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "fp8bs_last_device_status": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_uint)]),
    "fp8bs_selftest_wait_timeout": (_c.c_int, [_c.c_void_p]),
    "fp8bs_status_string": (_c.c_char_p, [_c.c_int]),
    "fp8bs_last_cuda_error": (_c.c_int, []),
    "fp8bs_launch_count": (_c.c_ulonglong, []),
    "fp8bs_gemmGPU": (_c.c_int, [_c.c_void_p] * 5 + [_c.c_size_t] * 3 + [_c.c_int]),
    "fp8bs_host_ctx_create": (_c.c_int, [_c.POINTER(_c.c_void_p)] + [_c.c_size_t] * 3),
    "fp8bs_host_ctx_destroy": (_c.c_int, [_c.c_void_p]),
    "fp8bs_host_ctx_buffer": (_c.c_void_p, [_c.c_void_p, _c.c_int]),
    "fp8bs_gemm_host": (_c.c_int, [_c.c_void_p] * 6 + [_c.c_int] * 5),
    "fp8bs_quantize_rowwise": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_float, _c.c_void_p]),
    "fp8bs_quantize_block": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int, _c.c_float, _c.c_void_p]),
    "fp8bs_gen_normal_e4m3": (_c.c_int, [_c.c_void_p, _c.c_size_t, _c.c_uint64]),
    "fp8bs_gen_uniform_f32": (_c.c_int, [_c.c_void_p, _c.c_size_t, _c.c_uint64, _c.c_float, _c.c_float]),
    "fp8bs_float_to_e4m3fn": (_c.c_uint8, [_c.c_float]),
    "fp8bs_e4m3fn_to_float": (_c.c_float, [_c.c_uint8]),
    "fp8bs_fnuz_to_fn_device": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p, _c.c_void_p]),
    "fp8bs_fnuz_to_fn": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.POINTER(_c.c_size_t)]),
}


def load(path):
    """Load the library from `path` and make it the one every call of this module uses (e.g. the instrumented
    build lib/libfp8bs_prof.so).  Raises if the file is missing: there is no other code path."""
    global _lib
    if not os.path.exists(path):
        raise RuntimeError("libfp8bs.so is not built (%s); run `python -m fp8_quant_matmul_b200.build`. "
                           "There is no fallback implementation." % path)
    handle = ctypes.CDLL(path)
    for name, (res, args) in _SIGS.items():
        fn = getattr(handle, name)
        fn.restype = res
        fn.argtypes = args
    _lib = handle
    return _lib


def lib():
    """The loaded library.  Raises if it has not been built: there is no other code path."""
    if _lib is None:
        load(_LIB_PATH)
    return _lib


def exported_symbols():
    """Names this binding expects the library to export (all of include/fp8bs.h)."""
    return sorted(_SIGS)


def status_string(code):
    try:
        return lib().fp8bs_status_string(int(code)).decode()
    except Exception:  # library absent: still give a usable message
        return "status %d" % code


def _check(code, where):
    if code != 0:
        raise Fp8bsError(code, where)


def launch_count():
    return int(lib().fp8bs_launch_count())


# ---------------------------------------------------------------- host-only helpers ----
def select_path(M, N, K):
    """(path, splits, tile_n) the run-time dispatch picks for a shape (pure host function)."""
    s, t = _c.c_int(0), _c.c_int(0)
    rc = lib().fp8bs_select_path(M, N, K, _c.byref(s), _c.byref(t))
    if rc < 0:
        raise Fp8bsError(rc, "fp8bs_select_path")
    return rc, s.value, t.value


def select_path_sms(M, N, K, sm_count):
    """(path, splits, tile_n, ctas that must be co-resident) for a GPU with sm_count SMs (pure host function)."""
    s, t, c = _c.c_int(0), _c.c_int(0), _c.c_int(0)
    rc = lib().fp8bs_select_path_sms(M, N, K, sm_count, _c.byref(s), _c.byref(t), _c.byref(c))
    if rc < 0:
        raise Fp8bsError(rc, "fp8bs_select_path_sms")
    return rc, s.value, t.value, c.value


def workspace_bytes(M, N, K, path=None, splits=0, tile_n=0):
    if path is None:
        return int(lib().fp8bs_workspace_bytes(M, N, K))
    return int(lib().fp8bs_workspace_bytes_ex(M, N, K, path, splits, tile_n))


def gen_normal_e4m3(n, seed):
    """n e4m3fn bytes: N(0,1) rounded to nearest even, |x| <= 240, |x| < 2^-6 -> +0."""
    out = np.empty(int(n), dtype=np.uint8)
    _check(lib().fp8bs_gen_normal_e4m3(out.ctypes.data, out.size, int(seed)), "fp8bs_gen_normal_e4m3")
    return out


def gen_uniform_f32(n, seed, lo, hi):
    out = np.empty(int(n), dtype=np.float32)
    _check(lib().fp8bs_gen_uniform_f32(out.ctypes.data, out.size, int(seed), float(lo), float(hi)),
           "fp8bs_gen_uniform_f32")
    return out


def float_to_e4m3fn(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    f = lib().fp8bs_float_to_e4m3fn
    return np.array([f(float(v)) for v in x.ravel()], dtype=np.uint8).reshape(x.shape)


def e4m3fn_to_float(b):
    b = np.ascontiguousarray(b, dtype=np.uint8)
    f = lib().fp8bs_e4m3fn_to_float
    table = np.array([f(i) for i in range(256)], dtype=np.float32)
    return table[b]


def fnuz_to_fn(src):
    """Re-encode e4m3fnuz bytes as e4m3fn bytes of equal value; raises on a byte that has none."""
    src = np.ascontiguousarray(src, dtype=np.uint8)
    dst = np.empty_like(src)
    bad = _c.c_size_t(0)
    rc = lib().fp8bs_fnuz_to_fn(dst.ctypes.data, src.ctypes.data, src.size, _c.byref(bad))
    if rc != 0:
        err = Fp8bsError(rc, "fp8bs_fnuz_to_fn")
        err.bad_index = bad.value
        raise err
    return dst


def fnuz_to_fn_device(src, dst=None):
    """Re-encode a CUDA uint8 tensor of e4m3fnuz bytes as e4m3fn bytes; returns (dst, number of inexact bytes)."""
    torch = _torch()
    if dst is None:
        dst = torch.empty_like(src)
    count = torch.zeros(1, dtype=torch.int32, device=src.device)
    stream = torch.cuda.current_stream(src.device).cuda_stream
    _check(lib().fp8bs_fnuz_to_fn_device(dst.data_ptr(), src.data_ptr(), src.numel(), count.data_ptr(), stream),
           "fp8bs_fnuz_to_fn_device")
    return dst, int(count.item())


# ---------------------------------------------------------------- the operator ---------
def _torch():
    import torch
    return torch


_workspaces = {}
_retired = []


def _workspace(device, nbytes):
    """A zero-initialised per-device workspace, grown on demand and reused between calls."""
    torch = _torch()
    key = (device.type, device.index)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _retired.append(ws)      # a captured CUDA graph may still point at the old one: keep it alive
        ws = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _check(lib().fp8bs_workspace_init(ws.data_ptr(), ws.numel(),
                                          torch.cuda.current_stream(device).cuda_stream), "fp8bs_workspace_init")
        _workspaces[key] = ws
    return ws


def gemm(A, B, a_scale, b_scale, C=None, M=None, N=None, K=None, path=PATH_AUTO, splits=0, tile_n=0,
         n0=0, n_total=None, workspace=None):
    """C = (A . a_scale) @ (B . b_scale)^T on the current CUDA stream.

    Arguments follow the kernel signature (A, B, As, Bs, C, M, N, K) of mn_large.hip:11:
      A        uint8/float8_e4m3fn CUDA tensor, M*K bytes, column-major  A[m + M*k]
      B        same, N*K bytes, column-major                             B[n + N*k]
      a_scale  float32 CUDA tensor [K/128, M] (memory order a_scale[m + M*kb])
      b_scale  float32 CUDA tensor [K/128, ceil(n_total/128)]
      C        bfloat16 CUDA tensor [M, N] (allocated if None)
    path / splits / tile_n force a kernel; n0 / n_total describe an N-shard.
    """
    torch = _torch()
    if not A.is_cuda:
        raise RuntimeError("fp8bs.gemm needs CUDA tensors; there is no CPU implementation")
    if M is None or N is None or K is None:
        raise ValueError("M, N, K are required (operands are flat column-major buffers)")
    if C is None:
        C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    if n_total is None:
        n_total = N
    need = workspace_bytes(M, N, K, path, splits, tile_n) if (path or splits or tile_n) else workspace_bytes(M, N, K)
    ws_ptr, ws_bytes = None, 0
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    elif need:
        ws = _workspace(A.device, need)
        ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    stream = torch.cuda.current_stream(A.device).cuda_stream
    rc = lib().fp8bs_gemm_ex(A.data_ptr(), B.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), C.data_ptr(),
                             M, N, K, n0, n_total, path, splits, tile_n, ws_ptr, ws_bytes, stream)
    _check(rc, "fp8bs_gemm_ex")
    return C


def gemm_scatter(A, B, a_scale, b_scale, dests, M, N, K, n0, n_total, stream=None):
    """N-sharded GEMM with the distribution of C fused into the epilogue: computes columns [n0, n0 + N) of an
    n_total-wide C and stores them into every buffer of `dests` (device pointers as ints, or torch tensors of shape
    [M, n_total] bf16): this GPU's own C and the peer-mapped C of the other GPUs."""
    import torch
    ptrs = [d.data_ptr() if hasattr(d, "data_ptr") else int(d) for d in dests]
    arr = (_c.c_void_p * len(ptrs))(*ptrs)
    if stream is None:
        stream = torch.cuda.current_stream(A.device).cuda_stream
    with torch.cuda.device(A.device):
        rc = lib().fp8bs_gemm_scatter(A.data_ptr(), B.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), arr, len(ptrs),
                                      M, N, K, n0, n_total, stream)
    _check(rc, "fp8bs_gemm_scatter")


STATIC_SCRATCH_BYTES = (32 << 20) + 65536


def gemm_mn_small_static(A, B, a_scale, b_scale, M, N, K, splits=0, C=None):
    """Split-K GEMM on the library's built-in scratch array: nothing is allocated, no workspace is passed.

    For callers that cannot allocate device memory when they call.  Problems whose partial sums exceed
    STATIC_SCRATCH_BYTES raise Fp8bsError(-4).  Calls share the scratch: keep them ordered on the GPU.
    C must be given if the caller truly cannot allocate; it is created here only as a convenience.
    """
    torch = _torch()
    if C is None:
        C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    stream = torch.cuda.current_stream(A.device).cuda_stream
    _check(lib().fp8bs_gemm_mn_small_static(A.data_ptr(), B.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(),
                                            C.data_ptr(), M, N, K, splits, stream), "fp8bs_gemm_mn_small_static")
    return C


def gemm_ref(A, B, a_scale, b_scale, M, N, K, C=None):
    """The ground-truth kernel restated in CUDA (ref_kernel, check.cu:30-49)."""
    torch = _torch()
    if C is None:
        C = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    stream = torch.cuda.current_stream(A.device).cuda_stream
    _check(lib().fp8bs_gemm_ref(A.data_ptr(), B.data_ptr(), a_scale.data_ptr(), b_scale.data_ptr(), C.data_ptr(),
                                M, N, K, stream), "fp8bs_gemm_ref")
    return C


def _quantize(fn_name, X, fp8_max):
    torch = _torch()
    if not X.is_cuda or X.dim() != 2 or not X.is_contiguous():
        raise ValueError("expected a contiguous 2-D CUDA tensor [rows, K]")
    if X.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("fp32 or bf16 input")
    rows, K = X.shape
    q = torch.empty(rows * K, dtype=torch.uint8, device=X.device)
    block = fn_name.endswith("block")
    n_scales = (K // 128) * (((rows + 127) // 128) if block else rows)
    scales = torch.empty(n_scales, dtype=torch.float32, device=X.device)
    stream = torch.cuda.current_stream(X.device).cuda_stream
    _check(getattr(lib(), fn_name)(X.data_ptr(), int(X.dtype == torch.bfloat16), q.data_ptr(), scales.data_ptr(),
                                   rows, K, float(fp8_max), stream), fn_name)
    return q, scales


def quantize_rowwise(X, fp8_max=448.0):
    """A and a_scale of the GEMM from a row-major [M, K] activation matrix (quantize.py:43-67).
    Returns (A bytes column-major, flat; inverse scales laid out a_scale[m + M*kb])."""
    return _quantize("fp8bs_quantize_rowwise", X, fp8_max)


def quantize_block(W, fp8_max=448.0):
    """B and b_scale of the GEMM from a row-major [N, K] weight matrix (128 x 128 blocks, quantize.py:16-41).
    Returns (B bytes column-major, flat; inverse scales laid out b_scale[nb + ceil(N/128)*kb])."""
    return _quantize("fp8bs_quantize_block", W, fp8_max)


def last_device_status(stream=None):
    """Synchronises and raises if a kernel recorded a barrier timeout."""
    detail = _c.c_uint(0)
    rc = lib().fp8bs_last_device_status(stream, _c.byref(detail))
    if rc != 0:
        err = Fp8bsError(rc, "fp8bs_last_device_status")
        err.detail = detail.value
        raise err


def gemmGPU(A, B, a_scale, b_scale, M, N, K, option=0):
    """Mirror of the reference's gemmGPU (check.cu:51-130): HOST fp32 arrays in, HOST bf16 bits out.

    A is fp32 M x K column-major, B fp32 N x K column-major (flat numpy arrays); they are
    converted to fp8 on the device as the reference does.  option: 0 auto, 1 mn_small, 2 ref kernel.
    Returns a uint16 array [M, N] of bf16 bit patterns.
    """
    A = np.ascontiguousarray(A, dtype=np.float32)
    B = np.ascontiguousarray(B, dtype=np.float32)
    a_scale = np.ascontiguousarray(a_scale, dtype=np.float32)
    b_scale = np.ascontiguousarray(b_scale, dtype=np.float32)
    C = np.empty((M, N), dtype=np.uint16)
    _check(lib().fp8bs_gemmGPU(C.ctypes.data, A.ctypes.data, B.ctypes.data, a_scale.ctypes.data,
                               b_scale.ctypes.data, M, N, K, option), "fp8bs_gemmGPU")
    return C


class HostContext:
    """Reusable end-to-end context: pinned host staging + device buffers, no allocation per call."""

    def __init__(self, max_M, max_N, max_K):
        self._h = _c.c_void_p(None)
        _check(lib().fp8bs_host_ctx_create(_c.byref(self._h), max_M, max_N, max_K), "fp8bs_host_ctx_create")
        self.max = (max_M, max_N, max_K)

    def buffer(self, which, nbytes, dtype):
        """numpy view of pinned staging buffer `which` (0 A, 1 B, 2 a_scale, 3 b_scale, 4 C)."""
        ptr = lib().fp8bs_host_ctx_buffer(self._h, which)
        buf = (_c.c_uint8 * nbytes).from_address(ptr)
        return np.frombuffer(buf, dtype=dtype)

    def gemm(self, C, A, B, a_scale, b_scale, M, N, K, n0=0, n_total=None):
        """Host pointers (numpy arrays, ideally views of the pinned buffers) in and out; synchronous."""
        _check(lib().fp8bs_gemm_host(self._h, C.ctypes.data, A.ctypes.data, B.ctypes.data, a_scale.ctypes.data,
                                     b_scale.ctypes.data, M, N, K, n0, N if n_total is None else n_total),
               "fp8bs_gemm_host")
        return C

    def close(self):
        if self._h:
            lib().fp8bs_host_ctx_destroy(self._h)
            self._h = _c.c_void_p(None)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

/*
 * fp8bs.h -- C ABI of libfp8bs.so: the row-wise block-scaled FP8 GEMM for NVIDIA B200
 *
 *     C[M,N] (bf16, row-major) = sum_kb a_scale[m,kb] * b_scale[n/128,kb]
 *                                       * ( A[m, kb*128 .. kb*128+127] . B[n, kb*128 .. kb*128+127] )
 *
 * Operand layouts are those of the reference kernels' 8-argument signature
 * (mn_large.hip:11, mn_small.hip:10, check.cu:30-31):
 *     A        fp8 e4m3, M x K column-major      A[m + M*k]
 *     B        fp8 e4m3, N x K column-major      B[n + N*k]
 *     a_scale  fp32 [M, K/128]                   a_scale[m + M*kb]
 *     b_scale  fp32 [ceil(N/128), K/128]         b_scale[nb + ceil(N/128)*kb]
 *     C        bf16, M x N row-major             C[m*N + n]
 * fp8 bytes are OCP e4m3fn (the dialect B200 tensor cores read).  The reference stores
 * e4m3fnuz; every value v with 2^-6 <= |v| <= 240 (and 0) exists in both dialects,
 * with fn_byte = fnuz_byte - 8; fp8bs_fnuz_to_fn converts.
 *
 * All pointers passed to the fp8bs_gemm* functions are DEVICE pointers owned by the caller
 * (as in the reference, where gemmGPU owns every buffer: check.cu:66-81, 122-128).  The
 * library never allocates per call, launches asynchronously on the given stream and does
 * not synchronise.  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * There is no CPU fallback: without a B200-class device every call returns an error.
 *
 * Every function returns 0 on success or a negative FP8BS_ERR_* code; nothing throws or
 * aborts.  Requirements: M, N, K > 0; K % 128 == 0 (mn_large.hip:17); M % 16 == 0 and
 * N % 16 == 0 (16-byte strides of the column-major operands); A, B, C and a_scale
 * 16-byte aligned.
 */
#ifndef FP8BS_H
#define FP8BS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FP8BS_OK                  0
#define FP8BS_ERR_NULL           -1   /* a required pointer is NULL */
#define FP8BS_ERR_SHAPE          -2   /* M, N or K not positive, or K % 128 != 0 */
#define FP8BS_ERR_ALIGN          -3   /* M % 16, N % 16 or a pointer alignment rule broken */
#define FP8BS_ERR_WORKSPACE      -4   /* workspace missing or too small for the chosen path */
#define FP8BS_ERR_ARG            -5   /* bad path / splits / tile / n0 argument */
#define FP8BS_ERR_NO_DEVICE      -6   /* no usable sm_100 device or driver entry point */
#define FP8BS_ERR_CUDA           -7   /* a CUDA runtime call failed; see fp8bs_last_cuda_error */
#define FP8BS_ERR_DEVICE_TIMEOUT -8   /* a kernel gave up waiting on one of its barriers */
#define FP8BS_ERR_FP8_BYTE       -9   /* an fp8 byte has no equal value in the other dialect */

#define FP8BS_PATH_AUTO      0
#define FP8BS_PATH_MN_LARGE  1   /* persistent full-K kernel   (role of mn_large.hip) */
#define FP8BS_PATH_MN_SMALL  2   /* split-K kernel             (role of mn_small.hip) */

/* tile_n values: 0 = let the library choose; 128 or 256 = tile width with one CTA per 128-row tile;
 * 256 | FP8BS_TILE_PAIR = a 256 x 256 tile owned by a pair of CTAs (tcgen05 cta_group::2). */
#define FP8BS_TILE_PAIR      0x1000
/* Split-K partial sums are normally reduced inside a thread-block cluster through shared memory (2..8 splits, one
 * CTA per tile): no workspace is needed then.  OR this flag into tile_n to reduce through the workspace instead
 * (always used for more than 8 splits and for pair tiles). */
#define FP8BS_SPLIT_WORKSPACE 0x2000
/* Stream-K: the 128-K blocks of all tiles are dealt out evenly over the SMs, so the run time does not jump with the
 * tile count; a tile whose blocks fall to two or more CTAs is finished by the CTA that holds its first block, from
 * partial sums the others leave in the workspace (added in K order: results do not depend on timing).  Chosen by the
 * library when path and splits are left open and it is estimated fastest; OR this flag into tile_n (128 or 256, or 0)
 * to force it.  Needs the workspace (fp8bs_workspace_bytes_ex), splits must be 0 or 1. */
#define FP8BS_STREAM_K       0x4000
/* Short K (K <= 256): 256-wide tiles whose partial sums of both 128-K blocks stay in tensor memory and are handed to
 * the scaling warps once per tile instead of once per block.  Chosen by the library for such shapes when it is
 * estimated fastest; OR this flag into tile_n (256 or 0) to force it (path auto or mn_large, splits 0 or 1). */
#define FP8BS_SHORT_K        0x8000

/* ---- the operator ---------------------------------------------------------------- */

/* Run-time shape dispatch between the two kernels.  Replaces the reference's manual,
 * compile-time choice (which .hip file check.cu:13 / sgemm.cu:13 includes, plus OPTION,
 * mn_large.hip:9; policy in README.md:99, 161).  Falls back to the best full-K
 * configuration if the workspace is too small for split-K. */
int fp8bs_gemm(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C,
               int M, int N, int K, void* workspace, size_t workspace_bytes, void* stream);

/* Forced large-M.N path: replaces in_smem_kernel<<<grid, block>>> (mn_large.hip:11;
 * launch at check.cu:106-114).  Needs no workspace. */
int fp8bs_gemm_mn_large(const void* A, const void* B, const float* a_scale, const float* b_scale,
                        void* C, int M, int N, int K, void* stream);

/* Forced small-M.N / large-K path: replaces k_large_kernel<<<grid, block>>> (mn_small.hip:10;
 * launch at check.cu:92-101).  splits = 0 lets the library choose; 1 <= splits <= min(K/128, 32).
 * Partial sums are added in split order, so repeated calls give bit-identical C.  The workspace is only used
 * where fp8bs_workspace_bytes_ex reports a non-zero size for the configuration (may be NULL otherwise). */
int fp8bs_gemm_mn_small(const void* A, const void* B, const float* a_scale, const float* b_scale,
                        void* C, int M, int N, int K, int splits, void* workspace,
                        size_t workspace_bytes, void* stream);

/* Split-K GEMM that allocates nothing and needs no workspace from the caller.  No counterpart in the reference.
 * It is for callers that cannot hand over scratch memory at call time: code running where cudaMalloc is off limits
 * (a host process whose device memory is entirely owned by another allocator, a plug-in that is forbidden to
 * allocate, a latency-critical loop that cannot afford the device-wide synchronisation an allocation implies).
 * The partial sums go to a scratch array built into the library: FP8BS_STATIC_SCRATCH_BYTES (32 MiB + 64 KiB) of
 * device memory on every GPU that loads the library, held until the process exits.  A problem whose split-K
 * partial sums need more than that is refused with FP8BS_ERR_WORKSPACE (use fp8bs_gemm_mn_small with your own
 * workspace instead).  Arguments and results are those of fp8bs_gemm_mn_small; A, B, scales and C are still the
 * caller's device buffers.  The first call on a device performs one-time set-up (kernel attributes, the lookup of
 * the scratch array's device address), so make that first call before starting any stream capture.  All calls
 * share the one array, which still holds what the previous call wrote: the function zeroes the tile counters on
 * the stream before launching, and two calls that overlap on the GPU (different streams, no ordering) would
 * corrupt each other's partial sums -- keep calls to this function ordered. */
#define FP8BS_STATIC_SCRATCH_BYTES ((32u << 20) + 65536u)
int fp8bs_gemm_mn_small_static(const void* A, const void* B, const float* a_scale, const float* b_scale,
                               void* C, int M, int N, int K, int splits, void* stream);

/* Fused distribution of C for an N-sharded GEMM (no counterpart in the reference, which runs on one GPU).
 * Computes the columns [n0, n0 + N) of a C that is n_total columns wide, exactly as fp8bs_gemm_ex does (B holds only
 * those N columns, b_scale is the whole [ceil(n_total/128), K/128] array), and stores every finished tile into the
 * same window of each of the n_dest (1..8) row-major M x n_total bf16 buffers in C_dest: TMA stores straight out of the
 * epilogue, one per destination, instead of a separate all-gather and re-layout pass.  The pointers must be usable
 * from this device: the GPU's own buffer and peer-mapped buffers of other GPUs (cudaIpc / symmetric memory).  Runs the
 * full-K kernel.  The call returns when the launch is queued; a destination is complete when its owner has
 * synchronised with every writer (a barrier between the ranks after the stream has drained).  C_dest is a host array.
 * Needs 16-byte aligned buffers and n_total % 8 == 0, besides the rules of fp8bs_gemm_ex. */
int fp8bs_gemm_scatter(const void* A, const void* B, const float* a_scale, const float* b_scale,
                       void* const* C_dest, int n_dest, int M, int N, int K, int n0, int n_total, void* stream);

/* Everything explicit.  For an N-shard of a wider problem (multi-GPU partition by columns):
 * B and C hold columns [n0, n0+N) of an n_total-column problem, b_scale is the FULL
 * [ceil(n_total/128), K/128] array, n0 % 64 == 0.  The plain operator is n0 = 0,
 * n_total = N.  path: FP8BS_PATH_*; splits: 0 = choose; tile_n: see FP8BS_TILE_PAIR above.
 * No counterpart in the reference (it has no multi-GPU code); the arithmetic per element is
 * check.cu:38-48 with cy replaced by n0 + cy in the b_scale index. */
int fp8bs_gemm_ex(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C,
                  int M, int N, int K, int n0, int n_total, int path, int splits, int tile_n,
                  void* workspace, size_t workspace_bytes, void* stream);

/* One thread per C element, scalar fp32: the reference's ground-truth kernel restated in
 * CUDA (ref_kernel, check.cu:30-49; gemmGPU option 2, check.cu:87-90).  Slow; for the
 * on-device cross-check of the `check` program. */
int fp8bs_gemm_ref(const void* A, const void* B, const float* a_scale, const float* b_scale,
                   void* C, int M, int N, int K, void* stream);

/* Pure host functions (no GPU needed).  fp8bs_select_path returns FP8BS_PATH_MN_LARGE or
 * FP8BS_PATH_MN_SMALL (or a negative error) and stores the split count and tile width
 * (either pointer may be NULL).  Replaces the geometry switch of check.cu:86-117. */
int fp8bs_select_path(int M, int N, int K, int* splits, int* tile_n);
/* The same decision for a GPU with `sm_count` SMs (fp8bs_select_path plans for the current device once a call has
 * set it up, and for a full B200 -- 148 SMs -- before that or without a GPU).  *ctas (optional) receives the number
 * of CTAs the chosen configuration needs resident at the same time: the whole grid for stream-K, one cluster for the
 * cluster reduction, 0 otherwise; it never exceeds sm_count. */
int fp8bs_select_path_sms(int M, int N, int K, int sm_count, int* splits, int* tile_n, int* ctas);

/* Workspace the auto dispatch wants for this shape (0 if it would not split K), and the
 * same for an explicit configuration.  The workspace must be zeroed once with
 * fp8bs_workspace_init before its first use and after any FP8BS_ERR_DEVICE_TIMEOUT;
 * calls re-arm it themselves.  Concurrent calls need distinct workspaces. */
size_t fp8bs_workspace_bytes(int M, int N, int K);
size_t fp8bs_workspace_bytes_ex(int M, int N, int K, int path, int splits, int tile_n);
int fp8bs_workspace_init(void* workspace, size_t workspace_bytes, void* stream);

/* Synchronises `stream`, then returns FP8BS_OK or FP8BS_ERR_DEVICE_TIMEOUT if a kernel on
 * the current device recorded a barrier timeout since the last call (and clears the
 * record).  *detail (optional) receives the raw device status word. */
int fp8bs_last_device_status(void* stream, unsigned int* detail);

/* Failure-path self-test (no counterpart in the reference, which has no error handling): launches one warp that
 * waits, with a limit of 40 M cycles (about 20 ms), on a barrier nothing arrives on.  The wait gives up, the kernel ends normally,
 * and the next fp8bs_last_device_status returns FP8BS_ERR_DEVICE_TIMEOUT (detail & 0xFF == 9); the context stays usable. */
int fp8bs_selftest_wait_timeout(void* stream);

const char* fp8bs_status_string(int status);
/* cudaError_t of the most recent failing CUDA call made by this thread (0 if none). */
int fp8bs_last_cuda_error(void);
/* Number of this library's kernels launched by this process so far. */
unsigned long long fp8bs_launch_count(void);

/* ---- host harness helpers (mirror the reference's utils.h / gemmGPU) --------------- */

/* gemmGPU (check.cu:51-130): HOST buffers in, HOST bf16 C out; allocates device memory,
 * copies, converts fp32 -> fp8 on the device (convert_float_to_fp8, check.cu:17-22),
 * launches, copies back, frees.  A is fp32 M x K column-major, B fp32 N x K column-major.
 * option 0 = auto dispatch, 1 = forced mn_small, 2 = the ref kernel (the reference's own
 * option numbers, check.cu:86-117).  Synchronous. */
int fp8bs_gemmGPU(uint16_t* C, const float* A, const float* B, const float* a_scale,
                  const float* b_scale, size_t M, size_t N, size_t K, int option);

/* The same end-to-end call for operands that are already fp8 bytes, with the device
 * buffers and pinned staging owned by a reusable context (no allocation per call).
 * Used for end-to-end timing: H2D of A, B and both scales, the GEMM, D2H of C. */
typedef struct fp8bs_host_ctx fp8bs_host_ctx;
int fp8bs_host_ctx_create(fp8bs_host_ctx** ctx, size_t max_M, size_t max_N, size_t max_K);
int fp8bs_host_ctx_destroy(fp8bs_host_ctx* ctx);
/* Pinned staging buffers of the context (valid until destroy): fill these, then call. */
void* fp8bs_host_ctx_buffer(fp8bs_host_ctx* ctx, int which); /* 0 A, 1 B, 2 a_scale, 3 b_scale, 4 C */
int fp8bs_gemm_host(fp8bs_host_ctx* ctx, uint16_t* C, const void* A, const void* B,
                    const float* a_scale, const float* b_scale, int M, int N, int K, int n0,
                    int n_total);

/* Device-side quantisers that produce the GEMM's operands, following the reference's quantize.py.
 * fp8bs_quantize_rowwise = to_float8_rowwise_scale (quantize.py:43-67): X is row-major [M, K] on the device (fp32, or
 * bf16 when x_is_bf16 != 0, widened to fp32 first); one scale per (row, 128-K block): scale = fp8_max / max(|x|, 1e-12),
 * q = e4m3fn(clamp(x * scale)).  Writes A_out column-major (A[m + M*k]) and the INVERSE scales a_scale_out[m + M*kb],
 * i.e. the GEMM's A and a_scale.  fp8bs_quantize_block = to_float8_block_scale (quantize.py:16-41): W row-major [N, K],
 * one scale per 128 x 128 block; writes B_out column-major (B[n + N*k]) and b_scale_out[nb + ceil(N/128)*kb].  Unlike
 * the reference, N need not be a multiple of 128 (the last block is partial).  fp8_max is the largest magnitude to
 * produce: 448 for the full e4m3fn range, 240 to stay within the values e4m3fnuz (the reference's default dtype) also has.
 * M, N multiples of 16; K a multiple of 128; X/W and the outputs 16-byte aligned.  Asynchronous on `stream`. */
int fp8bs_quantize_rowwise(const void* X, int x_is_bf16, void* A_out, float* a_scale_out, int M, int K,
                           float fp8_max, void* stream);
int fp8bs_quantize_block(const void* W, int w_is_bf16, void* B_out, float* b_scale_out, int N, int K,
                         float fp8_max, void* stream);

/* Seeded synthetic inputs (role of genMat, utils.h:25-33, but counter-based so that any
 * slice can be generated independently).  Elements: N(0,1) rounded to nearest-even e4m3fn,
 * clamped to |x| <= 240, |x| < 2^-6 flushed to +0 -- every value exists in e4m3fnuz too.
 * Scales: uniform in [lo, hi). */
int fp8bs_gen_normal_e4m3(uint8_t* out, size_t n, uint64_t seed);
int fp8bs_gen_uniform_f32(float* out, size_t n, uint64_t seed, float lo, float hi);
/* fp32 -> e4m3fn, round to nearest even, saturating to +-448; NaN -> 0x7F. */
uint8_t fp8bs_float_to_e4m3fn(float x);
float fp8bs_e4m3fn_to_float(uint8_t b);
/* Re-encode e4m3fnuz bytes (the reference's element type, check.cu:17-21) as e4m3fn bytes
 * of equal value.  Returns FP8BS_ERR_FP8_BYTE at the first byte whose value e4m3fn cannot
 * hold (NaN 0x80, or an odd multiple of 2^-10 below 2^-6); *bad_index receives its index. */
int fp8bs_fnuz_to_fn(uint8_t* dst, const uint8_t* src, size_t n, size_t* bad_index);

/* The same re-encoding on the device, for operands that already live in GPU memory in the reference's format
 * (dst may equal src; both 16-byte aligned).  Bytes without an equal e4m3fn value do not stop it: NaN (0x80) becomes
 * the e4m3fn NaN, and the odd multiples of 2^-10 below 2^-6 are rounded to the nearest even multiple of 2^-9; their
 * number is stored in *inexact_count (a device pointer, may be NULL).  Asynchronous on `stream`. */
int fp8bs_fnuz_to_fn_device(void* dst, const void* src, size_t n, unsigned int* inexact_count, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FP8BS_H */

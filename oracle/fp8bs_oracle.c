/*
 * fp8bs_oracle.c -- CPU restatement of the reference's ground-truth kernel for the
 * row-wise block-scaled FP8 GEMM   C[M,N] = (A . a_scale) @ (B . b_scale)^T.
 *
 * THIS FILE IS TEST INFRASTRUCTURE.  It is the checker that the CUDA path is compared
 * against; nothing in the shipped library calls it and it is never the thing measured
 * (except as the labelled CPU baseline of the benchmark).
 *
 * Parity pin: the reference stores no expected outputs for this operator (its only test
 * is a GPU-vs-GPU self-comparison, check.cu:171-177).  What can be pinned is pinned by
 * tests/test_oracle.py: the e4m3 decode tables against torch's float8 views, the
 * reference's own CPU helpers genMat / gemmCPU (utils.h:25-33, 65-76) compiled from the
 * reference sources, and hand-derived known answers for every index formula below.
 *
 * Arithmetic followed, line by line (reference check.cu:30-49, `ref_kernel`):
 *     sn = ceil(N / 128)                                         check.cu:36
 *     result = 0                                                 check.cu:38
 *     for each 128-wide K block kb:                              check.cu:39
 *         block = 0; for kk in 0..127 (ascending):               check.cu:40-41
 *             block += float(A[m + (kb*128+kk)*M])
 *                    * float(B[n + (kb*128+kk)*N])               check.cu:42-44
 *         result += block * a_scale[m + kb*M] * b_scale[n/128 + kb*sn]   check.cu:46
 *     C[m*N + n] = bf16(result)   (round to nearest even)        check.cu:48
 * The product of two e4m3 values is exact in fp32 (4+4 significant bits), so a fused or
 * an unfused multiply-add give the same `block`; the scale line is evaluated unfused and
 * left to right, (block*as)*bs, then added (build with -ffp-contract=off).
 *
 * Loops are re-ordered for cache reuse only (rows and columns are independent); the
 * per-element order of floating-point operations is exactly the one above.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define KBLK 128

/* ---- fp8 decode ------------------------------------------------------------------ */

/* OCP e4m3fn: bias 7, no infinities, NaN = S.1111.111, subnormals m * 2^-9.
 * This is the dialect B200 tensor cores consume. */
float oracle_e4m3fn_to_float(uint8_t b)
{
    int s = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);
    else        v = ldexpf((float)(8 + m), e - 10);
    return s ? -v : v;
}

/* e4m3fnuz: bias 8, no negative zero, NaN = 0x80, subnormals m * 2^-10.
 * This is the dialect of the reference's element type (check.cu:17-21). */
float oracle_e4m3fnuz_to_float(uint8_t b)
{
    int s = b >> 7, e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (b == 0x80) return NAN;
    if (e == 0) v = ldexpf((float)m, -10);
    else        v = ldexpf((float)(8 + m), e - 11);
    return s ? -v : v;
}

/* fp32 -> bf16, round to nearest even; NaN -> quiet NaN. Matches the converting
 * constructor used at check.cu:48. */
uint16_t oracle_float_to_bf16(float f)
{
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fc0;
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

float oracle_bf16_to_float(uint16_t h)
{
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}

/* ---- the GEMM -------------------------------------------------------------------- */

#define ROWS_PER_PASS 8
#define NCHUNK 512

/*
 * Core routine.  Computes the listed rows of C (rows == NULL: rows 0..nrows-1).
 *   A        fp8 bytes, M x K column-major      A[m + M*k]                check.cu:42
 *   B        fp8 bytes, N x K column-major      B[n + N*k]                check.cu:43
 *   a_scale  fp32 [M, K/128], m contiguous      a_scale[m + M*kb]         check.cu:46
 *   b_scale  fp32 [sn, K/128], nb contiguous    b_scale[nb + sn*kb]       check.cu:46
 *   n0, sn   for an N-shard of a wider problem: column n of this B is global column
 *            n0+n, so nb = (n0+n)/128 and sn = ceil(N_total/128).  The plain operator
 *            is n0 = 0, sn = ceil(N/128) (check.cu:36).
 *   out      bf16 bits, nrows x N row-major (row i of out = row rows[i] of C)
 *   out_f32  optional fp32 copy of `result` before the bf16 cast (may be NULL)
 *   dialect  0 = e4m3fn bytes, 1 = e4m3fnuz bytes
 * Returns 0, or -1 on a bad argument / allocation failure.
 */
int oracle_gemm_rows_ex(const uint8_t* A, const uint8_t* B, const float* a_scale,
                        const float* b_scale, int M, int N, int K, int n0, int sn,
                        const int* rows, int nrows, uint16_t* out, float* out_f32,
                        int dialect, int threads)
{
    if (!A || !B || !a_scale || !b_scale || !out) return -1;
    if (M <= 0 || N <= 0 || K <= 0 || K % KBLK != 0 || nrows < 0 || sn <= 0 || n0 < 0) return -1;
    float lut[256];
    for (int i = 0; i < 256; ++i)
        lut[i] = dialect ? oracle_e4m3fnuz_to_float((uint8_t)i) : oracle_e4m3fn_to_float((uint8_t)i);

    /* B decoded once to fp32, same [k][n] order as the bytes. */
    float* Bf = (float*)malloc((size_t)K * N * sizeof(float));
    if (!Bf) return -1;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
#else
    threads = 1;
#endif
#pragma omp parallel for num_threads(threads) schedule(static)
    for (long long i = 0; i < (long long)K * N; ++i) Bf[i] = lut[B[i]];

    const int KB = K / KBLK;
    const int npass = (nrows + ROWS_PER_PASS - 1) / ROWS_PER_PASS;
    int fail = 0;

#pragma omp parallel num_threads(threads)
    {
        float* arow = (float*)malloc((size_t)ROWS_PER_PASS * K * sizeof(float));
        float* res  = (float*)malloc((size_t)ROWS_PER_PASS * NCHUNK * sizeof(float));
        float* blk  = (float*)malloc((size_t)ROWS_PER_PASS * NCHUNK * sizeof(float));
        if (!arow || !res || !blk) {
#pragma omp atomic write
            fail = 1;
        } else {
#pragma omp for schedule(dynamic, 1)
            for (int p = 0; p < npass; ++p) {
                const int r0 = p * ROWS_PER_PASS;
                const int nr = (nrows - r0 < ROWS_PER_PASS) ? nrows - r0 : ROWS_PER_PASS;
                int mrow[ROWS_PER_PASS];
                for (int r = 0; r < nr; ++r) {
                    mrow[r] = rows ? rows[r0 + r] : r0 + r;
                    const uint8_t* ap = A + mrow[r];
                    float* ar = arow + (size_t)r * K;
                    for (int k = 0; k < K; ++k) ar[k] = lut[ap[(size_t)k * M]];
                }
                for (int nc = 0; nc < N; nc += NCHUNK) {
                    const int nw = (N - nc < NCHUNK) ? N - nc : NCHUNK;
                    for (int i = 0; i < nr * NCHUNK; ++i) res[i] = 0.0f;
                    for (int kb = 0; kb < KB; ++kb) {
                        for (int i = 0; i < nr * NCHUNK; ++i) blk[i] = 0.0f;
                        for (int kk = 0; kk < KBLK; ++kk) {
                            const int k = kb * KBLK + kk;
                            const float* brow = Bf + (size_t)k * N + nc;
                            for (int r = 0; r < nr; ++r) {
                                const float av = arow[(size_t)r * K + k];
                                float* bl = blk + r * NCHUNK;
                                for (int n = 0; n < nw; ++n) bl[n] += av * brow[n];
                            }
                        }
                        for (int r = 0; r < nr; ++r) {
                            const float as = a_scale[mrow[r] + (size_t)kb * M];
                            float* bl = blk + r * NCHUNK;
                            float* rs = res + r * NCHUNK;
                            for (int n = 0; n < nw; ++n) {
                                const float bs = b_scale[(n0 + nc + n) / KBLK + (size_t)kb * sn];
                                rs[n] += bl[n] * as * bs;
                            }
                        }
                    }
                    for (int r = 0; r < nr; ++r) {
                        uint16_t* o = out + (size_t)(r0 + r) * N + nc;
                        const float* rs = res + r * NCHUNK;
                        for (int n = 0; n < nw; ++n) o[n] = oracle_float_to_bf16(rs[n]);
                        if (out_f32) {
                            float* of = out_f32 + (size_t)(r0 + r) * N + nc;
                            for (int n = 0; n < nw; ++n) of[n] = rs[n];
                        }
                    }
                }
            }
        }
        free(arow); free(res); free(blk);
    }
    free(Bf);
    return fail ? -1 : 0;
}

/* The plain operator: every row, n0 = 0, sn = ceil(N/128)  (check.cu:36). */
int oracle_gemm(const uint8_t* A, const uint8_t* B, const float* a_scale, const float* b_scale,
                uint16_t* C, int M, int N, int K, int dialect, int threads)
{
    return oracle_gemm_rows_ex(A, B, a_scale, b_scale, M, N, K, 0, (N + KBLK - 1) / KBLK,
                               NULL, M, C, NULL, dialect, threads);
}

/*
 * The arithmetic of ref_kernel written as the plain triple loop, one element at a time,
 * in the reference's own loop order (check.cu:38-48).  Slow; used by the tests to check
 * that the cache-blocked routine above is bit-identical to the naive statement.
 */
int oracle_gemm_naive(const uint8_t* A, const uint8_t* B, const float* a_scale,
                      const float* b_scale, uint16_t* C, int M, int N, int K, int dialect)
{
    if (K % KBLK != 0) return -1;
    const int sn = (N + KBLK - 1) / KBLK;
    for (int cx = 0; cx < M; ++cx)
        for (int cy = 0; cy < N; ++cy) {
            float result = 0;
            for (int i = 0; i < K; i += KBLK) {
                float block_result = 0;
                for (int ii = 0; ii < KBLK; ++ii) {
                    uint8_t ab = A[cx + (size_t)(i + ii) * M], bb = B[cy + (size_t)(i + ii) * N];
                    float av = dialect ? oracle_e4m3fnuz_to_float(ab) : oracle_e4m3fn_to_float(ab);
                    float bv = dialect ? oracle_e4m3fnuz_to_float(bb) : oracle_e4m3fn_to_float(bb);
                    block_result += av * bv;
                }
                result += block_result * a_scale[cx + (size_t)(i / KBLK) * M]
                                       * b_scale[cy / KBLK + (size_t)(i / KBLK) * sn];
            }
            C[(size_t)cx * N + cy] = oracle_float_to_bf16(result);
        }
    return 0;
}

/*
 * Tie-breaker: same sums in float64 (exact products, float64 block sums and float64
 * scaled accumulation), returned unrounded.  Used when a GPU value and the fp32 oracle
 * disagree near the tolerance edge, to see which is closer to the real-number result.
 */
int oracle_gemm_rows_f64(const uint8_t* A, const uint8_t* B, const float* a_scale,
                         const float* b_scale, int M, int N, int K, int n0, int sn,
                         const int* rows, int nrows, double* out, int dialect)
{
    if (K % KBLK != 0) return -1;
    float lut[256];
    for (int i = 0; i < 256; ++i)
        lut[i] = dialect ? oracle_e4m3fnuz_to_float((uint8_t)i) : oracle_e4m3fn_to_float((uint8_t)i);
#pragma omp parallel for schedule(dynamic, 1)
    for (int r = 0; r < nrows; ++r) {
        const int m = rows ? rows[r] : r;
        for (int n = 0; n < N; ++n) {
            double result = 0;
            for (int kb = 0; kb < K / KBLK; ++kb) {
                double blk = 0;
                for (int kk = 0; kk < KBLK; ++kk) {
                    size_t k = (size_t)kb * KBLK + kk;
                    blk += (double)lut[A[m + k * M]] * (double)lut[B[n + k * N]];
                }
                result += blk * (double)a_scale[m + (size_t)kb * M]
                              * (double)b_scale[(n0 + n) / KBLK + (size_t)kb * sn];
            }
            out[(size_t)r * N + n] = result;
        }
    }
    return 0;
}

/*
 * Tolerance check used by every parity test:  |got - ref| <= atol + rtol * |ref|,
 * a NaN on either side is a mismatch.  Returns the number of mismatches and stores the
 * index of the first one (or n when there is none).
 */
size_t oracle_allclose_bf16(const uint16_t* ref, const uint16_t* got, size_t n, float rtol,
                            float atol, size_t* first_bad, float* max_abs_err)
{
    size_t bad = 0, first = n;
    float maxerr = 0.0f;
    for (size_t i = 0; i < n; ++i) {
        float r = oracle_bf16_to_float(ref[i]), g = oracle_bf16_to_float(got[i]);
        float d = fabsf(g - r);
        int ok = (d <= atol + rtol * fabsf(r));   /* false when d is NaN */
        if (!ok) { if (first == n) first = i; ++bad; }
        if (d > maxerr) maxerr = d;
    }
    if (first_bad) *first_bad = first;
    if (max_abs_err) *max_abs_err = maxerr;
    return bad;
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// C-callable wrapper around the reference's own host helpers, compiled from the
// reference sources where they lie (utils.h is #included, never copied): genMat
// (utils.h:25-33), gemmCPU (utils.h:65-76), row_to_col_major (utils.h:49-55) and allClose
// (utils.h:35-47).  Built into oracle/_ref/libfp8bs_ref.so by oracle/Makefile.
// Test infrastructure: validates the CPU restatement and serves as the timed
// "reference CPU path" of the benchmark.  The shipped library never links it.
#include "utils.h"
#include <cstddef>
#include <cstring>
#include <thread>
#include <algorithm>

extern "C" {

// genMat(len): seed-7 U(-5,5) stream (utils.h:25-33).
int ref_genMat(float* out, size_t len)
{
    const std::vector<float> v = genMat(len);
    std::memcpy(out, v.data(), len * sizeof(float));
    return 0;
}

// gemmCPU on row-major A[M,K], B[K,N] -> C[M,N], all fp32 (utils.h:65-76), single thread.
int ref_gemmCPU(float* C, const float* A, const float* B, size_t M, size_t N, size_t K)
{
    std::vector<float> a(A, A + M * K), b(B, B + K * N), c(M * N);
    gemmCPU(c, a, b, M, N, K);
    std::memcpy(C, c.data(), M * N * sizeof(float));
    return 0;
}

// The same unmodified gemmCPU run on disjoint row slabs from `threads` host threads
// (each call sees its own M-slice of A and C and the whole of B).
int ref_gemmCPU_mt(float* C, const float* A, const float* B, size_t M, size_t N, size_t K, int threads)
{
    if (threads < 1) threads = 1;
    const std::vector<float> b(B, B + K * N);
    std::vector<std::thread> pool;
    const size_t per = (M + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        const size_t r0 = std::min(M, per * t), r1 = std::min(M, r0 + per);
        if (r1 <= r0) continue;
        pool.emplace_back([=, &b]() {
            std::vector<float> a(A + r0 * K, A + r1 * K), c((r1 - r0) * N);
            gemmCPU(c, a, b, r1 - r0, N, K);
            std::memcpy(C + r0 * N, c.data(), (r1 - r0) * N * sizeof(float));
        });
    }
    for (auto& th : pool) th.join();
    return 0;
}

int ref_row_to_col_major(const float* in, float* out, int M, int N)
{
    std::vector<float> a(in, in + (size_t)M * N), b((size_t)M * N);
    row_to_col_major(a, b, M, N);
    std::memcpy(out, b.data(), b.size() * sizeof(float));
    return 0;
}

// allClose on bf16 bit patterns with the reference's absolute tolerance (utils.h:35-47).
int ref_allClose(const uint16_t* a, const uint16_t* b, size_t n, float tol)
{
    std::vector<__hip_bfloat16> va(n), vb(n);
    for (size_t i = 0; i < n; ++i) { va[i].bits = a[i]; vb[i].bits = b[i]; }
    return allClose(va, vb, tol) ? 1 : 0;
}

}  // extern "C"

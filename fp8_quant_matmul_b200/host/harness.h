// Shared pieces of the two harness programs (role of the reference's utils.h): command-line
// parsing, seeded inputs through the library's generator, bf16 helpers and the tolerance check.
#pragma once
#include "fp8bs.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

struct Shape { int M, N, K; };

// The 18 shapes of the reference's results table (README.md:15-25).
inline std::vector<Shape> sweep_shapes()
{
    const int nk[9][2] = {{1536, 7168}, {3072, 1536}, {576, 7168}, {7168, 256}, {7168, 2048},
                          {4608, 7168}, {7168, 2304}, {512, 7168}, {4096, 512}};
    std::vector<Shape> v;
    for (int M : {1024, 6144})
        for (auto& p : nk) v.push_back({M, p[0], p[1]});
    return v;
}

inline bool parse_shape(const char* s, Shape* out) { return std::sscanf(s, "%d,%d,%d", &out->M, &out->N, &out->K) == 3; }

inline float bf16_to_float(uint16_t h)
{
    uint32_t u = static_cast<uint32_t>(h) << 16;
    float f;
    std::memcpy(&f, &u, 4);
    return f;
}

#define CUDA_OK(expr)                                                                        \
    do {                                                                                     \
        cudaError_t e__ = (expr);                                                            \
        if (e__ != cudaSuccess) {                                                            \
            std::fprintf(stderr, "%s:%d: %s -> %s\n", __FILE__, __LINE__, #expr, cudaGetErrorString(e__)); \
            std::exit(2);                                                                    \
        }                                                                                    \
    } while (0)

#define FP8BS_CHECK(expr)                                                                    \
    do {                                                                                     \
        int rc__ = (expr);                                                                   \
        if (rc__ != FP8BS_OK) {                                                              \
            std::fprintf(stderr, "%s:%d: %s -> %d (%s)\n", __FILE__, __LINE__, #expr, rc__, fp8bs_status_string(rc__)); \
            std::exit(2);                                                                    \
        }                                                                                    \
    } while (0)

// Host copies of one problem's operands (fp8 bytes and scales) with the benchmark's distributions.
struct HostProblem {
    Shape s;
    std::vector<uint8_t> A, B;
    std::vector<float> As, Bs;
    HostProblem(Shape shape, uint64_t seed, float scale_lo = 0.01f, float scale_hi = 1.0f) : s(shape)
    {
        const size_t KB = s.K / 128, sn = (s.N + 127) / 128;
        A.resize(static_cast<size_t>(s.M) * s.K);
        B.resize(static_cast<size_t>(s.N) * s.K);
        As.resize(s.M * KB);
        Bs.resize(sn * KB);
        fp8bs_gen_normal_e4m3(A.data(), A.size(), seed);
        fp8bs_gen_normal_e4m3(B.data(), B.size(), seed + 1);
        fp8bs_gen_uniform_f32(As.data(), As.size(), seed + 2, scale_lo, scale_hi);
        fp8bs_gen_uniform_f32(Bs.data(), Bs.size(), seed + 3, scale_lo, scale_hi);
    }
};

struct DeviceProblem {
    Shape s;
    uint8_t *A = nullptr, *B = nullptr;
    float *As = nullptr, *Bs = nullptr;
    uint16_t* C = nullptr;
    explicit DeviceProblem(const HostProblem& h) : s(h.s)
    {
        CUDA_OK(cudaMalloc(&A, h.A.size()));
        CUDA_OK(cudaMalloc(&B, h.B.size()));
        CUDA_OK(cudaMalloc(&As, h.As.size() * 4));
        CUDA_OK(cudaMalloc(&Bs, h.Bs.size() * 4));
        CUDA_OK(cudaMalloc(&C, static_cast<size_t>(s.M) * s.N * 2));
        CUDA_OK(cudaMemcpy(A, h.A.data(), h.A.size(), cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(B, h.B.data(), h.B.size(), cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(As, h.As.data(), h.As.size() * 4, cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemcpy(Bs, h.Bs.data(), h.Bs.size() * 4, cudaMemcpyHostToDevice));
    }
    DeviceProblem(const DeviceProblem&) = delete;
    ~DeviceProblem() { cudaFree(A); cudaFree(B); cudaFree(As); cudaFree(Bs); cudaFree(C); }
};

// |mine - ref| <= atol + rtol*|ref| for every element; prints the first mismatch in the
// reference's format "index---ref---mine" (utils.h:42) and returns the mismatch count.
inline size_t all_close(const std::vector<uint16_t>& ref, const std::vector<uint16_t>& mine, float rtol, float atol)
{
    size_t bad = 0;
    for (size_t i = 0; i < ref.size(); ++i) {
        const float r = bf16_to_float(ref[i]), m = bf16_to_float(mine[i]);
        if (!(std::fabs(m - r) <= atol + rtol * std::fabs(r))) {
            if (bad == 0) std::printf("%zu---%g---%g\n", i, r, m);
            ++bad;
        }
    }
    return bad;
}

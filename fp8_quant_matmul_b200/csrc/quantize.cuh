// Device-side FP8 quantisers that produce the GEMM's operands in the operator's own layouts.
// They follow the reference's quantize.py:
//   row-wise 1x128 scaling (to_float8_rowwise_scale, quantize.py:43-67) for the activation matrix A, and
//   128x128 block scaling  (to_float8_block_scale,  quantize.py:16-41) for the weight matrix B:
//       absmax = max(|x|) over the group, clamped to >= 1e-12
//       scale  = fp8_max / absmax (torch computes reciprocal(absmax) * fp8_max, and so does this kernel)
//       q = fp8(clamp(x * scale, -fp8_max, fp8_max));   returned scale = 1 / scale
// Input is row-major [rows, K] (fp32, or bf16 widened to fp32 first).  Output bytes are column-major
// (out[r + rows*k], the layout of mn_large.hip:13-14) and the inverse scales go to scale_out[r + rows*kb] (row-wise)
// or scale_out[rb + ceil(rows/128)*kb] (block) -- exactly what the GEMM reads (check.cu:42-46).
//
// One CTA handles a 128 x 128 tile: 64 KB read with float4 loads, each thread keeps its 64 values in registers,
// the fp8 bytes are transposed through shared memory so that global writes are 128-byte runs along the rows index.
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace fp8bs {

__host__ __device__ inline uint8_t float_to_e4m3fn_rne(float x);   // defined in fp8bs.cu

template <bool BLOCK_SCALE, typename InT>
__global__ void __launch_bounds__(256)
quantize_kernel(const InT* __restrict__ X, uint8_t* __restrict__ out, float* __restrict__ scale_out, int rows, int K,
                float fp8_max)
{
    // tile: rows [r0, r0+128), k [k0, k0+128)
    const int r0 = blockIdx.x * 128, kb = blockIdx.y, k0 = kb * 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __shared__ __align__(16) uint8_t tile[128][144];   // [k][row], pitch 144 = 128 + 16: 16-byte aligned rows, fewer conflicts
    __shared__ float warp_max[8];

    // each warp owns 16 rows; lane holds 4 consecutive k of every one of them
    float v[16][4];
    float amax[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int r = r0 + warp * 16 + i;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows) {
            const InT* src = X + static_cast<size_t>(r) * K + k0 + lane * 4;
            if constexpr (sizeof(InT) == 4) {
                x = *reinterpret_cast<const float4*>(src);
            } else {
                const uint2 raw = *reinterpret_cast<const uint2*>(src);
                const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                x = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
            }
        }
        v[i][0] = x.x; v[i][1] = x.y; v[i][2] = x.z; v[i][3] = x.w;
        float m = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        amax[i] = m;                                   // every lane: absmax of row i over the 128 k
    }
    if constexpr (BLOCK_SCALE) {
        float m = 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) m = fmaxf(m, amax[i]);
        if (lane == 0) warp_max[warp] = m;
        __syncthreads();
        m = warp_max[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
#pragma unroll
        for (int i = 0; i < 16; ++i) amax[i] = m;      // one scale for the whole 128 x 128 block
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float a = fmaxf(amax[i], 1e-12f);                       // .clamp(min=1e-12)   quantize.py:29, 57
        // finfo.max / absmax (quantize.py:30, 58): for a tensor divisor torch evaluates this as reciprocal(absmax) * max
        const float scale = __fmul_rn(__fdiv_rn(1.0f, a), fp8_max);
        const int rl = warp * 16 + i;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float q = __fmul_rn(v[i][j], scale);
            q = fminf(fmaxf(q, -fp8_max), fp8_max);                   // .clamp(min, max)    quantize.py:33, 61
            tile[lane * 4 + j][rl] = float_to_e4m3fn_rne(q);
        }
        if (!BLOCK_SCALE && lane == 0 && r0 + rl < rows)
            scale_out[static_cast<size_t>(kb) * rows + r0 + rl] = __fdiv_rn(1.0f, scale);      // reciprocal, quantize.py:65
    }
    if (BLOCK_SCALE && threadIdx.x == 0) {
        const float a = fmaxf(amax[0], 1e-12f);
        scale_out[static_cast<size_t>(kb) * gridDim.x + blockIdx.x] = __fdiv_rn(1.0f, __fmul_rn(__fdiv_rn(1.0f, a), fp8_max));
    }
    __syncthreads();
    // write out: k-row by k-row, 128 bytes (128 rows of the input) at a time; a thread moves 16 bytes
    for (int idx = threadIdx.x; idx < 128 * 8; idx += 256) {
        const int k = idx >> 3, c = (idx & 7) * 16;
        if (r0 + c < rows) {       // rows % 16 == 0 is required by the GEMM, so a 16-byte run is all in or all out
            const uint4 q = *reinterpret_cast<const uint4*>(&tile[k][c]);
            *reinterpret_cast<uint4*>(out + static_cast<size_t>(k0 + k) * rows + r0 + c) = q;
        }
    }
}

}  // namespace fp8bs

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
// One CTA handles a 128 x 128 tile: 64 KB read with float4 loads, each thread keeps its 64 values in registers (80
// registers per thread, three CTAs per SM: the scales are applied in place instead of being kept per row).  The
// fp8 bytes go through shared memory as 32-bit words that hold four consecutive rows at one k -- four bytes that are
// also neighbours in the column-major output -- laid out [row group][k] with a pitch of 132 words: a thread writes its
// four k of a row group as one 16-byte store (a warp: 512 contiguous bytes), and reads back 16 bytes with lane = row
// group, which is conflict-free per quarter warp; each word then leaves in a 128-byte coalesced run along the rows.
// The conversion is the hardware's cvt.rn.satfinite.e4m3x2.f32 (round to nearest even; the clamp before it keeps
// every value inside the format's range, where it equals torch's cast bit for bit).
#pragma once
#include <cuda_bf16.h>
#include <cstdint>

namespace fp8bs {

__host__ __device__ inline uint8_t float_to_e4m3fn_rne(float x);   // defined in fp8bs.cu

// Two fp32 -> two e4m3fn bytes (lo in bits 0-7, hi in bits 8-15), round to nearest even.
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi)
{
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

template <bool BLOCK_SCALE, typename InT>
__global__ void __launch_bounds__(256)
quantize_kernel(const InT* __restrict__ X, uint8_t* __restrict__ out, float* __restrict__ scale_out, int rows, int K,
                float fp8_max)
{
    // tile: rows [r0, r0+128), k [k0, k0+128)
    const int r0 = blockIdx.x * 128, kb = blockIdx.y, k0 = kb * 128;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int PITCH = 132;                                   // words per row group: 128 k + 4 (16-byte aligned rows)
    __shared__ __align__(16) uint32_t tile[32 * PITCH];          // [row group of 4][k]: one word = 4 rows at one k
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
                x = __ldcs(reinterpret_cast<const float4*>(src));            // streamed: read once
            } else {
                const uint2 raw = __ldcs(reinterpret_cast<const uint2*>(src));
                const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
                const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
                x = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
            }
        }
        v[i][0] = x.x; v[i][1] = x.y; v[i][2] = x.z; v[i][3] = x.w;
        amax[i] = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));   // this lane's 4 k of row i
    }
    // Row maxima over the 32 lanes by a halving butterfly: at offset 16 a lane keeps 8 of its 16 rows and hands the other
    // 8 to its partner, at offset 8 it keeps 4, ... : 8 + 4 + 2 + 1 + 1 = 16 shuffles instead of 5 per row (80).
    // Afterwards lanes 2r and 2r + 1 both hold the absmax of the warp's row r over the 128 k.
    float rowmax;
    {
        const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0, b2 = (lane & 4) != 0, b1 = (lane & 2) != 0;
        float h8[8], h4[4], h2[2];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float give = b4 ? amax[j] : amax[j + 8], keep = b4 ? amax[j + 8] : amax[j];
            h8[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 16));
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float give = b3 ? h8[j] : h8[j + 4], keep = b3 ? h8[j + 4] : h8[j];
            h4[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 8));
        }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float give = b2 ? h4[j] : h4[j + 2], keep = b2 ? h4[j + 2] : h4[j];
            h2[j] = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 4));
        }
        const float give = b1 ? h2[0] : h2[1], keep = b1 ? h2[1] : h2[0];
        rowmax = fmaxf(keep, __shfl_xor_sync(0xffffffffu, give, 2));
        rowmax = fmaxf(rowmax, __shfl_xor_sync(0xffffffffu, rowmax, 1));       // row (lane >> 1) & 15
    }
    if constexpr (BLOCK_SCALE) {
        float m = rowmax;                              // max over the warp's 16 rows: lanes 0, 2, .., 30 hold them
#pragma unroll
        for (int o = 16; o > 1; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) warp_max[warp] = m;
        __syncthreads();
        m = warp_max[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) m = fmaxf(m, warp_max[w]);
        rowmax = m;                                    // one scale for the whole 128 x 128 block
    }
    // The scale of a row (or of the block) is applied in place, so that no per-row scale stays live in the loops below.
    float sc;
    if constexpr (BLOCK_SCALE) {
        const float a = fmaxf(rowmax, 1e-12f);                        // .clamp(min=1e-12)   quantize.py:29
        // finfo.max / absmax (quantize.py:30): for a tensor divisor torch evaluates this as reciprocal(absmax) * max
        sc = __fmul_rn(__fdiv_rn(1.0f, a), fp8_max);
        if (threadIdx.x == 0) scale_out[static_cast<size_t>(kb) * gridDim.x + blockIdx.x] = __fdiv_rn(1.0f, sc);
    } else {
        // lanes 2r and 2r + 1 work out the scale of the warp's row r and its inverse (two exact divisions per lane);
        // the scales go round by shuffle below
        const float a = fmaxf(rowmax, 1e-12f);                        // .clamp(min=1e-12)   quantize.py:57
        sc = __fmul_rn(__fdiv_rn(1.0f, a), fp8_max);                  // reciprocal(absmax) * max, quantize.py:58
        // the even lanes store the inverse scales of the warp's 16 rows: one 64-byte run per warp
        const int rl = warp * 16 + (lane >> 1);
        if ((lane & 1) == 0 && r0 + rl < rows)
            scale_out[static_cast<size_t>(kb) * rows + r0 + rl] = __fdiv_rn(1.0f, sc);            // reciprocal, quantize.py:65
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const float s_i = BLOCK_SCALE ? sc : __shfl_sync(0xffffffffu, sc, 2 * i);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            v[i][j] = fminf(fmaxf(__fmul_rn(v[i][j], s_i), -fp8_max), fp8_max);    // .clamp(min, max)    quantize.py:33, 61
    }
    // quantise; rows 4g .. 4g+3 of this warp at k = 4*lane + j become one word
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
            w[j] = cvt_e4m3x2(v[4 * g][j], v[4 * g + 1][j]) | (cvt_e4m3x2(v[4 * g + 2][j], v[4 * g + 3][j]) << 16);
        *reinterpret_cast<uint4*>(&tile[(warp * 4 + g) * PITCH + lane * 4]) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    __syncthreads();
    // write out: lane = row group, a warp instruction stores 128 consecutive bytes of one k-row of the output
    // (rows % 16 == 0 is required by the GEMM, so a 4-row word is all in or all out)
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int kq = (warp + 8 * it) * 4;                            // this warp's four k in this round
        const uint4 q = *reinterpret_cast<const uint4*>(&tile[lane * PITCH + kq]);
        if (r0 + lane * 4 < rows) {
            uint8_t* dst = out + static_cast<size_t>(k0 + kq) * rows + r0 + lane * 4;
            *reinterpret_cast<uint32_t*>(dst) = q.x;
            *reinterpret_cast<uint32_t*>(dst + rows) = q.y;
            *reinterpret_cast<uint32_t*>(dst + 2 * static_cast<size_t>(rows)) = q.z;
            *reinterpret_cast<uint32_t*>(dst + 3 * static_cast<size_t>(rows)) = q.w;
        }
    }
}

}  // namespace fp8bs

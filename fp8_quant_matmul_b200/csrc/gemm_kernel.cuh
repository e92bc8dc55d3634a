// Row-wise block-scaled FP8 GEMM for sm_100a:
//     C[m,n] = sum_kb a_scale[m,kb] * b_scale[n/128,kb] * sum_{k in block kb} A[m,k] * B[n,k]
// A is M x K column-major fp8 e4m3, B is N x K column-major fp8 e4m3, C is bf16 row-major
// (the operand layouts of the reference kernels, mn_large.hip:11-15 and mn_small.hip:10-17).
//
// One kernel template serves both shape classes of the reference:
//   SPLITK = false  "mn_large": persistent CTAs walk 128 x BN output tiles over the whole K
//                   (replaces in_smem_kernel, mn_large.hip:11-128);
//   SPLITK = true   "mn_small": each 128 x BN tile is cut into `splits` K ranges, partial
//                   sums go to an fp32 workspace and the CTA that finishes a tile last adds
//                   them in split order 0..S-1, so the result does not depend on timing
//                   (replaces k_large_kernel, mn_small.hip:10-137, which instead shrinks
//                   the tile to get more blocks).
//
// Structure of a CTA (warp-specialised, no __syncthreads in the main loop):
//   warp 0     TMA producer.  Both operands are MN-major in global memory, so a box of
//              {128 m or n, 128 k} lands in shared memory as 128 rows (k) of 128 bytes,
//              128-byte swizzled: the MN-major operand layout tcgen05.mma reads directly.
//              The byte-wise transposing copy of the reference (mn_large.hip:40-48) has
//              no counterpart here.
//   warp 1     MMA issuer.  Per 128-K block: four tcgen05.mma kind::f8f6f4 (K = 32 each)
//              into a fresh TMEM buffer (first one overwrites), then two commits: one
//              frees the shared-memory stage, one publishes the TMEM buffer.
//   warps 2..  promotion + epilogue.  TMEM lane = C row, so a thread owns one row and
//              128 columns; per K block it reads the partial sums with tcgen05.ld and does
//              acc = fma(a_scale*b_scale, partial, acc)   (mn_large.hip:99-106).
//              The running sums stay in registers, so the MMA warp is already filling
//              TMEM buffers for the next tile while these warps convert and store C.
// All waits on mbarriers are bounded: on expiry the waiter raises a CTA-wide abort flag,
// writes a code to the device status word and every role falls through to the common
// exit, where TMEM is released.
#pragma once
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <cstdint>

namespace fp8bs {

// Device status codes (low byte); the reporting CTA index is stored in the upper bits.
enum : uint32_t {
    DS_OK = 0,
    DS_TIMEOUT_STAGE_EMPTY = 1,  // producer waited for the MMA warp to release a stage
    DS_TIMEOUT_STAGE_FULL = 2,   // MMA warp waited for TMA data
    DS_TIMEOUT_TMEM_EMPTY = 3,   // MMA warp waited for the promotion warps
    DS_TIMEOUT_TMEM_FULL = 4,    // promotion warps waited for the MMA warp
};

struct GemmParams {
    const float* a_scale;    // [M, K/128], m contiguous            (check.cu:46)
    const float* b_scale;    // [sn, K/128], nb contiguous          (check.cu:46)
    __nv_bfloat16* C;        // M x N row-major                     (check.cu:48)
    float4* partials;        // split-K only: [unit][BN/4][128] float4
    unsigned int* counters;  // split-K only: one arrival counter per tile, zero between calls
    unsigned int* status;    // device status word
    int M, N, K;
    int n_off;               // global column index of local column 0 (N-sharded calls), else 0
    int sn;                  // rows of b_scale = ceil(N_total / 128)  (check.cu:36)
    int m_tiles, n_tiles, splits;
    float elem_scale;        // folded into b_scale: 1 for e4m3fn bytes
};

template <int BN>
struct TileCfg {
    static_assert(BN == 128 || BN == 256, "tile width");
    static constexpr int BM = 128;
    static constexpr int BK = 128;                    // one scale block
    static constexpr int SLAB = 128 * 128;            // bytes of one {128 mn, 128 k} box
    static constexpr int NBOX_B = BN / 128;
    static constexpr int STAGE_BYTES = SLAB * (1 + NBOX_B);
    static constexpr int STAGES = (BN == 256) ? 4 : 6;
    static constexpr int TMEM_COLS = 512;
    static constexpr int NBUF = TMEM_COLS / BN;       // TMEM partial-sum buffers
    static constexpr int PROMO_WARPS = 4 * (BN / 128);
    static constexpr int PROMO_THREADS = 32 * PROMO_WARPS;
    static constexpr int THREADS = 64 + PROMO_THREADS;
    static constexpr int NUM_BARS = 2 * STAGES + 2 * NBUF;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + NUM_BARS * 8 + 64;
};

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about one second

// Spin on an mbarrier phase with a time limit.  Returns false if the CTA is aborting.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity,
                                             volatile uint32_t* abort_flag, unsigned int* status,
                                             uint32_t code)
{
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (ptx::mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
            *abort_flag = 1u;
            atomicMax(status, code | (static_cast<uint32_t>(blockIdx.x) << 8));
            return false;
        }
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), round to nearest even
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int BN, bool SPLITK>
__global__ void __launch_bounds__(TileCfg<BN>::THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const GemmParams p)
{
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int NBUF = Cfg::NBUF;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t stage_base = (raw + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
    uint8_t* aligned = smem_raw + (stage_base - raw);
    const uint32_t bar_base = stage_base + STAGES * Cfg::STAGE_BYTES;
    volatile uint32_t* ctrl =
        reinterpret_cast<volatile uint32_t*>(aligned + STAGES * Cfg::STAGE_BYTES + Cfg::NUM_BARS * 8);
    // ctrl[0] TMEM base address, ctrl[1] abort flag, ctrl[2] "this CTA reduces the tile"
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + NBUF + b); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), Cfg::PROMO_WARPS);
        }
        ctrl[1] = 0u;
        ctrl[2] = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(&ctrl[0])), Cfg::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = ctrl[0];
    volatile uint32_t* abort_flag = &ctrl[1];

    const int KB = p.K / Cfg::BK;
    const int units = p.m_tiles * p.n_tiles * p.splits;

    // unit -> (tile, split) -> (m0, n0, kb range).  Tiles are numbered m-fastest so CTAs that
    // run side by side share the (wider) B slab through L2.
    auto decode = [&](int u, int& tile, int& m0, int& n0, int& kb0, int& kb1) {
        const int split = SPLITK ? (u % p.splits) : 0;
        tile = SPLITK ? (u / p.splits) : u;
        m0 = (tile % p.m_tiles) * Cfg::BM;
        n0 = (tile / p.m_tiles) * BN;
        kb0 = SPLITK ? (split * KB) / p.splits : 0;
        kb1 = SPLITK ? ((split + 1) * KB) / p.splits : KB;
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int tile, m0, n0, kb0, kb1;
                decode(u, tile, m0, n0, kb0, kb1);
                int nbox = (p.N - n0 + 127) >> 7;          // B slabs that hold any real column
                nbox = nbox < Cfg::NBOX_B ? nbox : Cfg::NBOX_B;
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    ok = wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_STAGE_EMPTY);
                    if (!ok) break;
                    const uint32_t a_dst = stage_base + s * Cfg::STAGE_BYTES;
                    ptx::mbar_arrive_expect_tx(full_bar(s), Cfg::SLAB * (1 + nbox));
                    ptx::tma_load_2d(a_dst, &tmA, m0, kb * Cfg::BK, full_bar(s));
                    for (int j = 0; j < nbox; ++j)
                        ptx::tma_load_2d(a_dst + Cfg::SLAB * (1 + j), &tmB, n0 + 128 * j, kb * Cfg::BK,
                                         full_bar(s));
                }
            }
            if (!ok) {
                // Aborting with loads possibly in flight: give them a bounded time to land
                // before the shared memory can be handed to another CTA.
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) __nanosleep(1000);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer ------
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_e4m3_mnmajor(Cfg::BM, BN);
            uint32_t it = 0, ait = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
                int tile, m0, n0, kb0, kb1;
                decode(u, tile, m0, n0, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it, ++ait) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    const int b = ait % NBUF;
                    const uint32_t bph = (ait / NBUF) & 1u;
                    ok = wait_bounded(tempty_bar(b), bph ^ 1u, abort_flag, p.status, DS_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    ok = wait_bounded(full_bar(s), ph, abort_flag, p.status, DS_TIMEOUT_STAGE_FULL);
                    if (!ok) break;
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = stage_base + s * Cfg::STAGE_BYTES;
                    const uint64_t adesc = ptx::make_smem_desc_sw128(a_addr, Cfg::SLAB, 1024);
                    const uint64_t bdesc = ptx::make_smem_desc_sw128(a_addr + Cfg::SLAB, Cfg::SLAB, 1024);
                    const uint32_t d = tmem_base + static_cast<uint32_t>(b * BN);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // K = 32 per instruction = 4 swizzle atoms of 8 k-rows = 4096 bytes
                        ptx::mma_f8f6f4(d, adesc + static_cast<uint64_t>(j * (4096 >> 4)),
                                        bdesc + static_cast<uint64_t>(j * (4096 >> 4)), idesc, j > 0 ? 1u : 0u);
                    }
                    ptx::mma_commit(empty_bar(s));
                    ptx::mma_commit(tfull_bar(b));
                }
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ promotion -------
        const int pw = warp - 2;
        const int quarter = warp & 3;            // TMEM lanes this warp may read: 32*quarter ..
        const int grp = pw >> 2;                 // which 128 columns of the tile
        const int row_in_tile = quarter * 32 + lane;
        uint32_t ait = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < units; u += gridDim.x) {
            int tile, m0, n0, kb0, kb1;
            decode(u, tile, m0, n0, kb0, kb1);
            const int m = m0 + row_in_tile;
            const bool mvalid = m < p.M;
            const int ncol0 = n0 + grp * 128;                 // first local column of this thread
            const int gcol0 = p.n_off + ncol0;                // its global column (b_scale index)
            int nb_lo = gcol0 >> 7, nb_hi = (gcol0 + 127) >> 7;
            nb_lo = nb_lo < p.sn ? nb_lo : p.sn - 1;
            nb_hi = nb_hi < p.sn ? nb_hi : p.sn - 1;
            const int hi_from = 4 - ((gcol0 & 127) >> 5);     // first 32-col chunk that uses nb_hi

            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.0f;

            const float* as_ptr = p.a_scale + (mvalid ? m : 0);
            float as_n = mvalid ? __ldg(as_ptr + static_cast<size_t>(kb0) * p.M) : 0.0f;
            float bl_n = __ldg(p.b_scale + nb_lo + static_cast<size_t>(kb0) * p.sn);
            float bh_n = __ldg(p.b_scale + nb_hi + static_cast<size_t>(kb0) * p.sn);

            for (int kb = kb0; kb < kb1 && ok; ++kb, ++ait) {
                const float s_lo = as_n * (bl_n * p.elem_scale);
                const float s_hi = as_n * (bh_n * p.elem_scale);
                if (kb + 1 < kb1) {   // next block's scales, in flight while we wait for TMEM
                    as_n = mvalid ? __ldg(as_ptr + static_cast<size_t>(kb + 1) * p.M) : 0.0f;
                    bl_n = __ldg(p.b_scale + nb_lo + static_cast<size_t>(kb + 1) * p.sn);
                    bh_n = __ldg(p.b_scale + nb_hi + static_cast<size_t>(kb + 1) * p.sn);
                }
                const int b = ait % NBUF;
                const uint32_t bph = (ait / NBUF) & 1u;
                ok = wait_bounded(tfull_bar(b), bph, abort_flag, p.status, DS_TIMEOUT_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(b * BN + grp * 128);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    ptx::tmem_ld_x32(taddr + c * 32, v);
                    ptx::tmem_ld_wait();
                    const float sc = (c >= hi_from) ? s_hi : s_lo;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        acc[c * 32 + i] = fmaf(sc, __uint_as_float(v[i]), acc[c * 32 + i]);
                }
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(tempty_bar(b));
            }

            if constexpr (!SPLITK) {
                if (!ok) break;
                // ---- epilogue: fp32 -> bf16 (round to nearest even), 16-byte stores ----
                if (mvalid) {
                    __nv_bfloat16* crow = p.C + static_cast<size_t>(m) * p.N + ncol0;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if (ncol0 + j * 8 < p.N) {
                            uint4 q;
                            q.x = pack_bf16x2(acc[j * 8 + 0], acc[j * 8 + 1]);
                            q.y = pack_bf16x2(acc[j * 8 + 2], acc[j * 8 + 3]);
                            q.z = pack_bf16x2(acc[j * 8 + 4], acc[j * 8 + 5]);
                            q.w = pack_bf16x2(acc[j * 8 + 6], acc[j * 8 + 7]);
                            *reinterpret_cast<uint4*>(crow + j * 8) = q;
                        }
                    }
                }
            } else {
                // ---- split-K: publish this K range's partial sums ----
                // Layout [unit][column quad][row]: a warp's 32 rows of one column quad are
                // 512 contiguous bytes, for the writes here and the reads below alike.
                float4* part = p.partials + (static_cast<size_t>(u) * (BN / 4) + grp * 32) * 128 + row_in_tile;
                if (ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        part[static_cast<size_t>(j) * 128] =
                            make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
                    __threadfence();
                }
                // Every promotion thread reaches this barrier, aborting or not.
                int any_fail;
                {
                    uint32_t r;
                    asm volatile(
                        "{\n\t.reg .pred p, q;\n\t"
                        "setp.ne.b32 p, %1, 0;\n\t"
                        "barrier.cta.red.or.pred.aligned q, 1, %2, p;\n\t"
                        "selp.u32 %0, 1, 0, q;\n\t}"
                        : "=r"(r)
                        : "r"(ok ? 0u : 1u), "n"(Cfg::PROMO_THREADS)
                        : "memory");
                    any_fail = static_cast<int>(r);
                }
                if (any_fail) { ok = false; break; }
                if (pw == 0 && lane == 0) {
                    const unsigned int old = atomicAdd(&p.counters[tile], 1u);
                    const bool last = (old == static_cast<unsigned int>(p.splits - 1));
                    if (last) p.counters[tile] = 0u;     // every split has arrived: re-arm for the next call
                    ctrl[2] = last ? 1u : 0u;
                }
                asm volatile("barrier.cta.sync.aligned 1, %0;" ::"n"(Cfg::PROMO_THREADS) : "memory");
                if (ctrl[2]) {
                    __threadfence();
                    // ---- deterministic reduction: splits are added in the order 0, 1, .., S-1 ----
                    const float4* base = p.partials +
                        (static_cast<size_t>(tile) * p.splits * (BN / 4) + grp * 32) * 128 + row_in_tile;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float sum[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) sum[i] = 0.0f;
                        for (int s = 0; s < p.splits; ++s) {
                            const float4* ps = base + static_cast<size_t>(s) * (BN / 4) * 128;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float4 v = __ldcg(ps + static_cast<size_t>(c * 8 + j) * 128);
                                sum[4 * j + 0] += v.x;
                                sum[4 * j + 1] += v.y;
                                sum[4 * j + 2] += v.z;
                                sum[4 * j + 3] += v.w;
                            }
                        }
                        if (mvalid) {
                            __nv_bfloat16* crow = p.C + static_cast<size_t>(m) * p.N + ncol0 + c * 32;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (ncol0 + c * 32 + j * 8 < p.N) {
                                    uint4 q;
                                    q.x = pack_bf16x2(sum[j * 8 + 0], sum[j * 8 + 1]);
                                    q.y = pack_bf16x2(sum[j * 8 + 2], sum[j * 8 + 3]);
                                    q.z = pack_bf16x2(sum[j * 8 + 4], sum[j * 8 + 5]);
                                    q.w = pack_bf16x2(sum[j * 8 + 6], sum[j * 8 + 7]);
                                    *reinterpret_cast<uint4*>(crow + j * 8) = q;
                                }
                            }
                        }
                    }
                }
            }
        }
    }

    // ---------------------------------------------------------------- common exit -----
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace fp8bs

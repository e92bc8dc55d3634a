// Row-wise block-scaled FP8 GEMM for sm_100a:
//     C[m,n] = sum_kb a_scale[m,kb] * b_scale[n/128,kb] * sum_{k in block kb} A[m,k] * B[n,k]
// A is M x K column-major fp8 e4m3, B is N x K column-major fp8 e4m3, C is bf16 row-major
// (the operand layouts of the reference kernels, mn_large.hip:11-15 and mn_small.hip:10-17).
//
// One kernel template, three parameters:
//   BN      width of the output tile (128 or 256 columns)
//   CG      1: a CTA owns a 128 x BN tile.  2: two CTAs of a cluster own a 256 x BN tile; each
//           loads its own 128 rows of A and its own half of the B columns, the leader issues
//           tcgen05.mma.cta_group::2 (M = 256) that reads both CTAs' shared memory, and each
//           CTA's TMEM receives its own 128 rows.  Halves the B traffic per output element.
//   MODE    0 "mn_large": persistent CTAs walk tiles over the whole K
//                 (replaces in_smem_kernel, mn_large.hip:11-128);
//           1, 2 "mn_small": every tile is cut into `splits` K ranges and the partial sums are
//                 added in split order 0..S-1, so the result does not depend on timing (replaces
//                 k_large_kernel, mn_small.hip:10-137, which instead shrinks the tile to get more
//                 blocks).  MODE 2 (S <= 8): the S CTAs of a tile form a
//                 thread-block cluster, each leaves its fp32 partial tile in its own shared memory,
//                 and after a cluster barrier every CTA reduces 128/S rows straight out of its
//                 peers' shared memory (DSMEM): no workspace, no atomics.  MODE 1 (any S, also pair
//                 tiles): partial sums go to an fp32 workspace and whoever finishes a tile last adds
//                 them.
//           3 stream-K: the K blocks of all tiles are dealt out evenly over the CTAs; a tile that
//                 falls to several CTAs is finished by the one that holds its first K block, from
//                 partial tiles the others leave in the workspace (added in K order).
//           4 short K (K <= 256, 256-wide tiles): the partial sums of both K blocks of a tile stay in the two TMEM
//                 buffers and are handed over once per tile; a promotion thread reads both K blocks of 64 of its
//                 columns with two loads in flight, scales and adds them in registers and stages the result, then the
//                 other 64.  One barrier round trip per tile instead of one per K block, and no running sums.
// The epilogue stores a finished tile to one or several destinations (CMaps): the caller's C, and
// for the fused distribution of an N-sharded GEMM the peer-mapped C of the other GPUs.
//
// Warp roles (no __syncthreads in the main loop; registers are moved from the first warpgroup
// to the promotion warps with setmaxnreg: 168 at launch, then 64 for warps 0-3 and 216 for the
// rest, which the compiler fits without a single spill; 56/224 left a few spilled words in the
// promotion loop and cost 8-15 % on the long-K shapes):
//   warp 0     TMA producer for A and B.  Both operands are MN-major in global memory, so a box
//              of {128 m or n, 128 k} lands in shared memory as 128 rows (k) of 128 bytes,
//              128-byte swizzled: the MN-major operand layout tcgen05.mma reads directly.  The
//              byte-wise transposing copy of the reference (mn_large.hip:40-48) has no
//              counterpart here.
//   warp 1     MMA issuer.  Per 128-K block: four tcgen05.mma kind::f8f6f4 (K = 32 each) into a
//              fresh TMEM buffer (the first one overwrites), then a commit that publishes the TMEM
//              buffer and, in the three-stage kernels, a second one that frees the shared-memory stage
//              (with four or more stages a promotion warp frees it, see PROMO_RELEASE).
//   warp 2     TMA producer for a_scale: boxes of 128 rows x 8 K blocks into a small ring, so the
//              promotion warps never wait on a global load (mn_large.hip:50-55 stages the
//              pre-multiplied scales in LDS for the same reason) and pay one barrier round trip
//              per 8 K blocks.
//   warp 3     idle (completes the warpgroup that gives up its registers).
//   warps 4..  promotion + epilogue.  TMEM lane = C row, so a thread owns one row and 128
//              columns; per K block it reads the partial sums with tcgen05.ld, 64 columns at a
//              time, and does
//              acc = fma(a_scale*b_scale, partial, acc) two columns at a time (mn_large.hip:99-106);
//              the TMEM buffer goes back to the MMA warp as soon as its last columns are in registers.
//              The running sums stay in registers, so the MMA warp is already filling TMEM for
//              the next tile while these warps convert to bf16, stage through swizzled shared
//              memory and hand C to TMA stores.
// All waits on mbarriers are bounded: on expiry the waiter raises a CTA-wide abort flag, writes
// a code to the device status word and every role falls through to the common exit, where TMEM
// is released.
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
    DS_TIMEOUT_SCALE_EMPTY = 5,  // scale producer waited for the promotion warps
    DS_TIMEOUT_SCALE_FULL = 6,   // promotion warps waited for a_scale
};

// Where a finished C tile goes: the caller's C, and for the fused distribution (fp8bs_gemm_scatter) the same window
// of up to MAX_DEST - 1 further buffers, e.g. the peer-mapped C of the other GPUs of an N-sharded GEMM.
constexpr int MAX_DEST = 8;
struct CMaps {
    CUtensorMap m[MAX_DEST];
};

struct GemmParams {
    const float* b_scale;    // [sn, K/128], nb contiguous          (check.cu:46)
    __nv_bfloat16* C;        // M x N row-major                     (check.cu:48)
    float4* partials;        // split-K only: [half-tile][split][BN/4][128] float4
    unsigned int* counters;  // split-K only: one arrival counter per 128-row half-tile, zero between calls
    unsigned int* status;    // device status word
    int M, N, K;
    int n_off;               // global column index of local column 0 (N-sharded calls), else 0
    int sn;                  // rows of b_scale = ceil(N_total / 128)  (check.cu:36)
    int m_tiles, n_tiles, splits;
    float inv_m_tiles;       // 1 / m_tiles, for the tile -> (row block, column block) decode
    int n_dest;              // number of valid entries of the CMaps argument (1 = only the caller's C)
    float elem_scale;        // folded into b_scale: 1 for e4m3fn bytes
#ifdef FP8BS_PROFILE
    long long* prof;         // per CTA: 8 cycle counters (profiling builds only)
#endif
};

// a_scale reaches shared memory in boxes of 128 rows x SCALE_GROUP K blocks (the tensor map's box, see the host side):
// one barrier round trip per SCALE_GROUP K blocks instead of one per block.  Measured on B200 with the promotion loop
// otherwise unchanged: a per-block hand-off cost ~160 cycles per K block of a loop that has ~512 to spend.
constexpr int SCALE_GROUP = 8;

template <int BN, int CG>
struct TileCfg {
    static_assert(BN == 128 || BN == 256, "tile width");
    static_assert(CG == 1 || (CG == 2 && BN == 256), "pair tiles are 256 x 256");
    static constexpr int BM = 128;                    // rows per CTA
    static constexpr int TILE_M = BM * CG;            // rows per tile (pair of CTAs when CG == 2)
    static constexpr int BK = 128;                    // one scale block
    static constexpr int SLAB = 128 * 128;            // bytes of one {128 mn, 128 k} box
    static constexpr int B_COLS = BN / CG;            // B columns this CTA loads
    static constexpr int NBOX_B = B_COLS / 128;
    static constexpr int STAGE_BYTES = SLAB * (1 + NBOX_B);
    static constexpr int TMEM_COLS = 512;
    static constexpr int NBUF = TMEM_COLS / BN;       // TMEM partial-sum buffers
    static constexpr int COLS = BN / 2;               // columns of the tile row a promotion thread owns (64 or 128)
    static constexpr int NCH = COLS / 32;             // ... as 32-column chunks
    static constexpr int PROMO_WARPS = 8;             // 4 TMEM lane quarters x 2 column groups
    static constexpr int PROMO_THREADS = 32 * PROMO_WARPS;
    static constexpr int THREADS = 128 + PROMO_THREADS;
    // per warp: store boxes of 32 rows x 64 bf16 columns, one per 64-column half of a thread's columns, so the second half
    // need not wait for the first store to drain.  Pair tiles too: with two boxes and 4 stages they measured 1.5-3 % faster
    // than with one box and 5 stages at every K.
    static constexpr int NSTG = COLS / 64;
    static constexpr int STG_BYTES = PROMO_WARPS * 4096 * NSTG;
    static constexpr int SGRP = SCALE_GROUP;          // K blocks per a_scale ring entry (one TMA box {128 rows, SGRP})
    static constexpr int SRING = 4;                   // a_scale ring entries
    static constexpr int SRING_BYTES = SRING * SGRP * 512;
    static constexpr int SMEM_LIMIT = 232448;         // 227 KB per CTA
    static constexpr int FIXED = 1024 + STG_BYTES + SRING_BYTES + 512;
    static constexpr int STAGES = (SMEM_LIMIT - FIXED) / STAGE_BYTES;
    static_assert(STAGES >= 2, "pipeline depth");
    static constexpr int NUM_BARS = 2 * STAGES + 2 * NBUF + 2 * SRING;
    static_assert(NUM_BARS * 8 + 64 <= 512, "barrier area");
    static constexpr int SMEM_BYTES = FIXED + STAGES * STAGE_BYTES;
};

constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about one second

// Instrumentation, compiled in only by `python -m fp8_quant_matmul_b200.build --profile[=LEVEL]` (-DFP8BS_PROFILE=LEVEL,
// into a separate libfp8bs_prof.so).  Layout of the buffer GemmParams::prof points to, in 64-bit words:
//   [cta * 16 + slot]           slots 0-7 cycle counters (level >= 2): producer wait for a free stage, MMA wait for a
//                               free TMEM buffer, MMA wait for operands, MMA loop total, promotion wait for a_scale,
//                               promotion wait for partial sums, promotion loads + FMAs, epilogue;
//                               slots 8-14 %globaltimer stamps in ns: kernel start, set-up done, first operands
//                               there, MMA loop done, promotion loop done, all stores issued, exit; slot 15 the
//                               CTA's lifetime in cycles
//   [4096 + event * 128 + kb]   level 3, CTA 0, first 128 K blocks, clock64 at: 0 TMEM buffer free (MMA warp),
//                               1 operands there, 2 MMAs and commits issued, 3 a_scale there (promotion warp 4),
//                               4 partial sums there, 5 FMAs done, 6 stage free (producer), 7 / 8 = 4 / 5 for warp 5;
//                               [4096 + (9 or 10) * 128 + unit]: start / end of the epilogue of CTA 0's unit
#ifdef FP8BS_PROFILE
#define PROF_DECL(name) long long name = 0
#if FP8BS_PROFILE >= 2 && !defined(FP8BS_PROFILE_NOTIMERS)   // per-wait timers: they perturb the loops they measure
#define PROF_T0() const long long prof_t0__ = clock64()
#define PROF_ADD(name) name += clock64() - prof_t0__
#else
#define PROF_T0()
#define PROF_ADD(name)
#endif
#define PROF_OUT(slot, name) p.prof[blockIdx.x * 16 + (slot)] = (name)
__device__ __forceinline__ long long prof_now_ns() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return static_cast<long long>(t); }
#define PROF_STAMP(slot) p.prof[blockIdx.x * 16 + (slot)] = prof_now_ns()
#if FP8BS_PROFILE >= 3   // per-K-block time line of CTA 0
#define PROF_TRACE(ev, idx) do { if (blockIdx.x == 0 && (idx) < 128u) p.prof[4096 + (ev) * 128 + (idx)] = clock64(); } while (0)
#else
#define PROF_TRACE(ev, idx)
#endif
#define PROF_CLK0() const long long prof_c0__ = clock64()
#define PROF_CLK1(slot) p.prof[blockIdx.x * 16 + (slot)] = clock64() - prof_c0__
#else
#define PROF_CLK0()
#define PROF_CLK1(slot)
#define PROF_TRACE(ev, idx)
#define PROF_DECL(name)
#define PROF_T0()
#define PROF_ADD(name)
#define PROF_OUT(slot, name)
#define PROF_STAMP(slot)
#endif

// Spin on an mbarrier phase with a time limit.  Returns false if the CTA is aborting.
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                             unsigned int* status, uint32_t code,
                                             long long limit_cycles = WAIT_LIMIT_CYCLES)
{
    if (ptx::mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        // parked in hardware for up to 8 us per try: no issue slots are spent while waiting
        if (ptx::mbar_try_wait_parked(bar, parity, 8192u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit_cycles) {
            *abort_flag = 1u;
            atomicMax(status, code | (static_cast<uint32_t>(blockIdx.x) << 8));
            return false;
        }
    }
}

// Two fp32 values in one 64-bit register, the operand form of fma.rn.f32x2 (low word = first value).
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi)
{
    return static_cast<unsigned long long>(__float_as_uint(lo)) | (static_cast<unsigned long long>(__float_as_uint(hi)) << 32);
}
__device__ __forceinline__ float f32x2_lo(unsigned long long v) { return __uint_as_float(static_cast<uint32_t>(v)); }
__device__ __forceinline__ float f32x2_hi(unsigned long long v) { return __uint_as_float(static_cast<uint32_t>(v >> 32)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), round to nearest even
    return *reinterpret_cast<uint32_t*>(&h);
}

// Two views of "64 consecutive fp32 columns of this thread's row": the packed accumulators of two
// 32-column chunks, or a plain array.  pair(i) returns columns (2i, 2i+1).
struct PackedCols {
    const unsigned long long (&a)[16];
    const unsigned long long (&b)[16];
    __device__ __forceinline__ uint32_t bf16_pair(int i) const
    {
        const unsigned long long v = (i < 16) ? a[i & 15] : b[i & 15];
        return pack_bf16x2(f32x2_lo(v), f32x2_hi(v));
    }
};
struct FloatCols {
    const float (&v)[64];
    __device__ __forceinline__ uint32_t bf16_pair(int i) const { return pack_bf16x2(v[2 * i], v[2 * i + 1]); }
};

// Converts 64 columns of this thread's row to bf16 (round to nearest even) into a 32-row x 128-byte staging
// box laid out as the 128-byte-swizzled TMA store expects; then the warp's lane 0 issues the store.
// The box covers rows [row0, row0 + 32) and columns [col, col + 64); lane = row within the box.
// PENDING: how many of this thread's most recent stores may still be reading shared memory (1 when the warp
// alternates between two boxes: only the store before the last one used this box); negative: the caller has waited.
// Converts 64 columns of this thread's row to bf16 (round to nearest even) into row `lane` of a 32-row x 128-byte
// staging box, laid out as the 128-byte-swizzled TMA store expects.
template <class Cols>
__device__ __forceinline__ void stage_64(uint8_t* stg, int lane, const Cols cols)
{
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        uint4 q;
        q.x = cols.bf16_pair(4 * j + 0);
        q.y = cols.bf16_pair(4 * j + 1);
        q.z = cols.bf16_pair(4 * j + 2);
        q.w = cols.bf16_pair(4 * j + 3);
        // 16-byte chunk j, XOR-swizzled with the row index (bank-conflict free)
        *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = q;
    }
}

template <int PENDING, class Cols>
__device__ __forceinline__ void stage_and_store_64(const CUtensorMap* tmC, int n_dest, uint8_t* stg, uint32_t stg_addr,
                                                   int lane, const Cols cols, int col, int row0, int M, int N)
{
    if constexpr (PENDING >= 0) {
        if (lane == 0) ptx::tma_store_wait_read<PENDING>();  // the previous store out of this box has read it
        __syncwarp();
    }
    stage_64(stg, lane, cols);
    ptx::fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0 && col < N && row0 < M) {
        // rows >= M and columns >= N are clipped by the hardware; one bulk group covers every destination's copy
        for (int d = 0; d < n_dest; ++d) ptx::tma_store_2d(tmC + d, stg_addr, col, row0);
        ptx::tma_store_commit();
    }
}

// The two 64-column boxes of a warp's 32 x 128 piece at once: both are staged, then lanes 0 and 1 issue one store each
// in the same instruction, so the warp pays the issue latency of a TMA store once per tile instead of twice (1-3 % on
// the shapes with many tiles per CTA).  Bulk groups belong to the issuing thread: lane h issues, and waits for, the
// stores out of box h.  The caller has made sure that both boxes are free (wait_read<0> in lanes 0 and 1).
template <class Cols0, class Cols1>
__device__ __forceinline__ void stage_and_store_2x64(const CUtensorMap* tmC, int n_dest, uint8_t* stg, uint32_t stg_addr,
                                                     int lane, const Cols0 c0, const Cols1 c1, int col, int row0, int M, int N)
{
    stage_64(stg, lane, c0);
    stage_64(stg + 4096, lane, c1);
    ptx::fence_proxy_async_smem();
    __syncwarp();
    const int mycol = col + lane * 64;
    if (lane < 2 && mycol < N && row0 < M) {
        for (int d = 0; d < n_dest; ++d) ptx::tma_store_2d(tmC + d, stg_addr + lane * 4096, mycol, row0);
        ptx::tma_store_commit();
    }
}

// Self-test of the failure path: one warp waits, with a short limit, on a barrier that nothing ever arrives on.
// The wait must give up, record DS_TIMEOUT_SELFTEST in the status word and the kernel must end normally.
constexpr uint32_t DS_TIMEOUT_SELFTEST = 9;
constexpr uint32_t DS_TIMEOUT_PEER_PARTIAL = 10;   // stream-K: another CTA's partial sums never arrived
__global__ void wait_timeout_selftest_kernel(unsigned int* status, long long limit_cycles)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_word;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_word = 0u;
        ptx::fence_mbar_init();
    }
    __syncthreads();
    const bool ok = wait_bounded(ptx::smem_u32(&bar), 0u, &abort_word, status, DS_TIMEOUT_SELFTEST, limit_cycles);
    (void)ok;
}

template <int BN, int CG, int MODE>
__global__ void __launch_bounds__(TileCfg<BN, CG>::THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ CUtensorMap tmAs, const __grid_constant__ CMaps cmaps, const GemmParams p)
{
    using Cfg = TileCfg<BN, CG>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int NBUF = Cfg::NBUF;
    constexpr int SRING = Cfg::SRING;
    constexpr bool SPLITK = (MODE == 1 || MODE == 2);   // K cut into p.splits equal ranges per tile
    constexpr bool STREAMK = (MODE == 3);               // K blocks of all tiles dealt out evenly, see below
    static_assert(MODE != 2 || CG == 1, "the cluster reduction uses the cluster for the K splits");
    static_assert(MODE != 3 || CG == 1, "stream-K is built for single-CTA tiles");
    constexpr bool RESIDENT = (MODE == 4);              // both K blocks of a tile kept in TMEM (K <= 256)
    // Who frees a shared-memory stage.  Every tcgen05 instruction costs the issuing thread time, so with four or more
    // stages the MMA warp issues one commit per K block (TMEM buffer full) and a promotion warp, which learns from that
    // barrier that the MMAs are done, arrives on the stage's barrier: 1.5-4 % faster on the pair and the 128-wide
    // kernels.  With three stages (256-wide single-CTA tiles) the later release starves the loads (3-7 % slower),
    // so there the MMA warp frees the stage with a second commit.
    constexpr bool PROMO_RELEASE = (STAGES >= 4) && !RESIDENT;
    static_assert(!RESIDENT || (CG == 1 && BN == 256), "the short-K mode uses 256-wide single-CTA tiles");
    // MODE 2: fp32 partial tile of this CTA, rows padded by 16 bytes so that a warp's 32 rows hit distinct banks
    constexpr int PART_PITCH = BN * 4 + 16;
    static_assert(MODE != 2 || 128 * PART_PITCH <= STAGES * Cfg::STAGE_BYTES, "partial tile must fit in the stage area");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t stage_base = (raw + 1023u) & ~1023u;   // swizzle atoms need 1024-byte alignment
    uint8_t* aligned = smem_raw + (stage_base - raw);
    // layout: [stages][epilogue staging][a_scale ring][barriers + control words]
    const uint32_t stg_base = stage_base + STAGES * Cfg::STAGE_BYTES;
    uint8_t* stg_ptr = aligned + STAGES * Cfg::STAGE_BYTES;
    const uint32_t sring_base = stg_base + Cfg::STG_BYTES;
    const float* sring_ptr = reinterpret_cast<const float*>(stg_ptr + Cfg::STG_BYTES);
    const uint32_t bar_base = sring_base + Cfg::SRING_BYTES;
    volatile uint32_t* ctrl = reinterpret_cast<volatile uint32_t*>(stg_ptr + Cfg::STG_BYTES + Cfg::SRING_BYTES +
                                                                    Cfg::NUM_BARS * 8);
    // ctrl[0] TMEM base address, ctrl[1] abort flag, ctrl[2] "this CTA reduces the tile"
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
    auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + NBUF + b); };
    auto sfull_bar = [&](int i) { return bar_base + 8u * (2 * STAGES + 2 * NBUF + i); };
    auto sempty_bar = [&](int i) { return bar_base + 8u * (2 * STAGES + 2 * NBUF + SRING + i); };

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    PROF_CLK0();
    if (threadIdx.x == 0) { PROF_STAMP(8); }
    const uint32_t rank = (CG == 2) ? ptx::cluster_ctarank() : 0u;     // 0 = leader of the pair (MODE 2: not used)
    const int group_id = blockIdx.x / CG;                               // which tile walker this CTA belongs to
    const int num_groups = gridDim.x / CG;

    if (threadIdx.x == 0) {
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
        ptx::prefetch_tensormap(&tmAs);
        for (int d = 0; d < p.n_dest; ++d) ptx::prefetch_tensormap(&cmaps.m[d]);
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(full_bar(s), 1);
            ptx::mbar_init(empty_bar(s), 1);
        }
        for (int b = 0; b < NBUF; ++b) {
            ptx::mbar_init(tfull_bar(b), 1);
            ptx::mbar_init(tempty_bar(b), Cfg::PROMO_WARPS * CG);   // the leader also hears from the peer's warps
        }
        for (int i = 0; i < SRING; ++i) {
            ptx::mbar_init(sfull_bar(i), 1);
            ptx::mbar_init(sempty_bar(i), Cfg::PROMO_WARPS);
        }
        ctrl[1] = 0u;
        ctrl[2] = 0u;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        if constexpr (CG == 2) {
            ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(&ctrl[0])), Cfg::TMEM_COLS);
            ptx::tmem_relinquish_pair();
        } else {
            ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(&ctrl[0])), Cfg::TMEM_COLS);
            ptx::tmem_relinquish();
        }
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2) ptx::cluster_sync();      // the peer's barriers exist before anything remote touches them
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = ctrl[0];
    volatile uint32_t* abort_flag = &ctrl[1];
    // Everything above (barriers, TMEM, descriptor prefetch) touched no global data, so it may overlap the tail of
    // the previous kernel in the stream; from here on operands are read and C is written.
    ptx::grid_dependency_wait();
    ptx::grid_launch_dependents();
    if (threadIdx.x == 0) { PROF_STAMP(9); }

    const int KB = p.K / Cfg::BK;
    // MODE 3 (stream-K): the K blocks of all tiles form one line, tile after tile, and CTA c owns the piece
    // [c * T / G, (c + 1) * T / G) of it, so every CTA does the same number of K blocks (+-1) whatever the tile count.
    // A piece covers the end of one tile, whole tiles, and the beginning of one more.  A segment that starts inside
    // a tile (only a CTA's first can) leaves its partial sums in workspace slot c and raises flag c; the segment
    // that holds the tile's first K block adds the partials of the CTAs after it, in CTA (= K) order, and finishes
    // the tile.  Those CTAs work on that tile first, so their flags are up long before they are looked at; nobody
    // waits on a CTA that can itself be waiting (a first segment never waits).
    long long sk_lo = 0, sk_hi = 0;
    int sk_first = 0, sk_last = -1;
    if constexpr (STREAMK) {
        const long long T = static_cast<long long>(p.m_tiles) * p.n_tiles * KB;
        sk_lo = blockIdx.x * T / gridDim.x;
        sk_hi = (blockIdx.x + 1) * T / gridDim.x;
        if (sk_hi > sk_lo) {
            sk_first = static_cast<int>(sk_lo / KB);
            sk_last = static_cast<int>((sk_hi - 1) / KB);
        }
    }
    const int units = STREAMK ? (sk_last - sk_first + 1) : p.m_tiles * p.n_tiles * p.splits;
    const int unit0 = STREAMK ? 0 : group_id;          // a CTA's (pair's) first work unit and its stride
    const int unit_step = STREAMK ? 1 : num_groups;

    // unit -> (tile, split) -> (row of this CTA, first column, K-block range).  Tiles are numbered
    // m-fastest so CTAs that run side by side share the B slab through L2.
    auto decode = [&](int u, int& tile, int& m0, int& n0, int& kb0, int& kb1) {
        if constexpr (STREAMK) {
            tile = sk_first + u;
            kb0 = (u == 0) ? static_cast<int>(sk_lo - static_cast<long long>(sk_first) * KB) : 0;
            kb1 = (tile == sk_last) ? static_cast<int>(sk_hi - static_cast<long long>(sk_last) * KB) : KB;
        } else {
            const int split = SPLITK ? (u % p.splits) : 0;
            tile = SPLITK ? (u / p.splits) : u;
            kb0 = SPLITK ? (split * KB) / p.splits : 0;
            kb1 = SPLITK ? ((split + 1) * KB) / p.splits : KB;
        }
        // tile = ni * m_tiles + mi without an integer division (some 100 cycles, twice per tile in every role): the
        // float quotient is off by at most one for tile counts below 2^22, and the remainder says which way
        int ni = __float2int_rz(__int2float_rn(tile) * p.inv_m_tiles);
        int mi = tile - ni * p.m_tiles;
        if (mi < 0) { --ni; mi += p.m_tiles; }
        else if (mi >= p.m_tiles) { ++ni; mi -= p.m_tiles; }
        m0 = mi * Cfg::TILE_M + static_cast<int>(rank) * Cfg::BM;
        n0 = ni * BN;
    };

    if (warp < 4) {
        ptx::setmaxnreg_dec<64>();
        if (warp == 0 && lane == 0) {
            // ---------------------------------------------------- TMA producer: A and B ----
            uint32_t it = 0;
            bool ok = true;
            PROF_DECL(w_empty);
            for (int u = unit0; u < units && ok; u += unit_step) {
                int tile, m0, n0, kb0, kb1;
                decode(u, tile, m0, n0, kb0, kb1);
                const int nb0 = n0 + static_cast<int>(rank) * Cfg::B_COLS;    // first B column this CTA loads
                int nbox = (p.N - nb0 + 127) >> 7;                            // B slabs that hold any real column
                nbox = nbox < 0 ? 0 : (nbox < Cfg::NBOX_B ? nbox : Cfg::NBOX_B);
                if (CG == 2) nbox = Cfg::NBOX_B;                              // pairs: fixed byte count (zero fill)
                for (int kb = kb0; kb < kb1; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    { PROF_T0();
                    ok = wait_bounded(empty_bar(s), ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_STAGE_EMPTY);
                    PROF_ADD(w_empty); }
                    if (!ok) break;
                    PROF_TRACE(6, it);
                    const uint32_t a_dst = stage_base + s * Cfg::STAGE_BYTES;
                    if constexpr (CG == 2) {
                        // both CTAs' bytes are counted on the leader's barrier, which the MMA warp waits on
                        const uint32_t lead_full = ptx::mapa(full_bar(s), 0);
                        if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * Cfg::STAGE_BYTES);
                        ptx::tma_load_2d_pair(a_dst, &tmA, m0, kb * Cfg::BK, lead_full);
                        for (int j = 0; j < Cfg::NBOX_B; ++j)
                            ptx::tma_load_2d_pair(a_dst + Cfg::SLAB * (1 + j), &tmB, nb0 + 128 * j, kb * Cfg::BK, lead_full);
                    } else {
                        ptx::mbar_arrive_expect_tx(full_bar(s), Cfg::SLAB * (1 + nbox));
                        ptx::tma_load_2d(a_dst, &tmA, m0, kb * Cfg::BK, full_bar(s));
                        for (int j = 0; j < nbox; ++j)
                            ptx::tma_load_2d(a_dst + Cfg::SLAB * (1 + j), &tmB, nb0 + 128 * j, kb * Cfg::BK, full_bar(s));
                    }
                }
            }
            PROF_OUT(0, w_empty);
            if (!ok) {
                // Aborting with loads possibly in flight: give them a bounded time to land before the
                // shared memory can be handed to another CTA.
                const long long t0 = clock64();
                while (clock64() - t0 < 2000000LL) __nanosleep(1000);
            }
        } else if (warp == 1 && lane == 0 && rank == 0) {
            // ---------------------------------------------------- MMA issuer ----------------
            constexpr uint32_t idesc = ptx::make_idesc_e4m3_mnmajor(Cfg::TILE_M, BN);
            uint32_t it = 0, ait = 0, tcount = 0;
            bool ok = true;
            PROF_DECL(w_tempty); PROF_DECL(w_full); PROF_DECL(t_mma_total);
#ifdef FP8BS_PROFILE
            const long long mma_start = clock64();
#endif
            for (int u = unit0; u < units && ok; u += unit_step) {
                int tile, m0, n0, kb0, kb1;
                decode(u, tile, m0, n0, kb0, kb1);
                for (int kb = kb0; kb < kb1; ++kb, ++it, ++ait) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1u;
                    // MODE 4: K block j of a tile goes to buffer j; the pair is handed over and taken back once per tile
                    // (barriers tfull / tempty number 0, phase = tile count)
                    const int b = RESIDENT ? (kb - kb0) : static_cast<int>(ait % NBUF);
                    const uint32_t bph = RESIDENT ? (tcount & 1u) : ((ait / NBUF) & 1u);
                    const int eb = RESIDENT ? 0 : b;                       // the barrier pair that guards this buffer
                    // operands first (they are usually there already), then the TMEM buffer: nothing but the MMA
                    // issue stands between the promotion warps' release of the buffer and its reuse
                    { PROF_T0();
                    ok = wait_bounded(full_bar(s), ph, abort_flag, p.status, DS_TIMEOUT_STAGE_FULL);
                    PROF_ADD(w_full); }
                    if (!ok) break;
                    PROF_TRACE(1, it);
                    if (!RESIDENT || kb == kb0) {
                        PROF_T0();
                        ok = wait_bounded(tempty_bar(eb), bph ^ 1u, abort_flag, p.status, DS_TIMEOUT_TMEM_EMPTY);
                        PROF_ADD(w_tempty);
                    }
                    if (!ok) break;
                    PROF_TRACE(0, it);
#ifdef FP8BS_PROFILE
                    if (it == 0) { PROF_STAMP(10); }
#endif
                    ptx::tc_fence_after_sync();
                    const uint32_t a_addr = stage_base + s * Cfg::STAGE_BYTES;
                    const uint64_t adesc = ptx::make_smem_desc_sw128(a_addr, Cfg::SLAB, 1024);
                    const uint64_t bdesc = ptx::make_smem_desc_sw128(a_addr + Cfg::SLAB, Cfg::SLAB, 1024);
                    const uint32_t d = tmem_base + static_cast<uint32_t>(b * BN);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        // K = 32 per instruction = 4 swizzle atoms of 8 k-rows = 4096 bytes
                        const uint64_t step = static_cast<uint64_t>(j * (4096 >> 4));
                        if constexpr (CG == 2) ptx::mma_f8f6f4_pair(d, adesc + step, bdesc + step, idesc, j > 0 ? 1u : 0u);
                        else ptx::mma_f8f6f4(d, adesc + step, bdesc + step, idesc, j > 0 ? 1u : 0u);
                    }
                    // the promotion warps wait on this one; the producer is several stages ahead
                    if constexpr (CG == 2) {
                        // one commit per barrier reaches both CTAs of the pair (with plain commits, two per barrier, the
                        // fourth one of a K block cost ~100 cycles of tensor-pipe time)
                        ptx::mma_commit_pair_all(tfull_bar(b), 3);
                        if constexpr (!PROMO_RELEASE) ptx::mma_commit_pair_all(empty_bar(s), 3);
                    } else {
                        if (!RESIDENT || kb == kb1 - 1) ptx::mma_commit(tfull_bar(eb));
                        if constexpr (!PROMO_RELEASE) ptx::mma_commit(empty_bar(s));
                    }
                    PROF_TRACE(2, it);
                }
                ++tcount;
            }
#ifdef FP8BS_PROFILE
            t_mma_total = clock64() - mma_start;
#endif
            PROF_OUT(1, w_tempty); PROF_OUT(2, w_full); PROF_OUT(3, t_mma_total); PROF_STAMP(11);
        } else if (warp == 2 && lane == 0) {
            // ---------------------------------------------------- TMA producer: a_scale ----
            uint32_t sit = 0;
            bool ok = true;
            for (int u = unit0; u < units && ok; u += unit_step) {
                int tile, m0, n0, kb0, kb1;
                decode(u, tile, m0, n0, kb0, kb1);
                for (int kb = kb0; kb < kb1; kb += Cfg::SGRP, ++sit) {
                    const int i = sit % SRING;
                    const uint32_t ph = (sit / SRING) & 1u;
                    ok = wait_bounded(sempty_bar(i), ph ^ 1u, abort_flag, p.status, DS_TIMEOUT_SCALE_EMPTY);
                    if (!ok) break;
                    // a whole box is always written and counted: rows >= M and K blocks past the end read as 0
                    ptx::mbar_arrive_expect_tx(sfull_bar(i), Cfg::SGRP * 512);
                    ptx::tma_load_2d(sring_base + i * (Cfg::SGRP * 512), &tmAs, m0, kb, sfull_bar(i));
                }
            }
        }
        __syncwarp();
    } else {
        // -------------------------------------------------------- promotion + epilogue ------
        ptx::setmaxnreg_inc<216>();
        const int pw = warp - 4;
        const int quarter = warp & 3;            // TMEM lanes this warp may read: 32*quarter ..
        const int grp = pw >> 2;                 // which half of the tile's columns
        const int row_in_tile = quarter * 32 + lane;
        uint8_t* my_stg = stg_ptr + pw * 4096 * Cfg::NSTG;
        const uint32_t my_stg_addr = stg_base + pw * 4096 * Cfg::NSTG;
        uint32_t lead_tempty = tempty_bar(0);
        if constexpr (CG == 2) lead_tempty = ptx::mapa(tempty_bar(0), 0);
        uint32_t ait = 0;
        uint32_t sgit = 0;                       // a_scale ring entries consumed so far
        uint32_t tcount = 0;                     // MODE 4: tiles done by this CTA
        bool ok = true;
        PROF_DECL(w_sfull); PROF_DECL(w_tfull); PROF_DECL(t_fma); PROF_DECL(t_epi);
        // b_scale lane vectors of unit u: K blocks kb0 + lane and kb0 + 32 + lane of the one or two 128-column blocks
        // this thread's columns fall into (same index arithmetic as at the top of the unit loop)
        float pf_bl = 0.0f, pf_bh = 0.0f, pf_bln = 0.0f, pf_bhn = 0.0f;
        auto fetch_bscale = [&](int u) {
            int tile, m0, n0, kb0, kb1;
            decode(u, tile, m0, n0, kb0, kb1);
            const int g0 = p.n_off + n0 + grp * Cfg::COLS;
            int lo = g0 >> 7, hi = (g0 >> 7) + 1;
            lo = lo < p.sn ? lo : p.sn - 1;
            hi = hi < p.sn ? hi : p.sn - 1;
            auto ld = [&](int nb, int kbase) {
                const int k = kbase + lane;
                return (k < kb1) ? __ldg(p.b_scale + nb + static_cast<size_t>(k) * p.sn) : 0.0f;
            };
            pf_bl = ld(lo, kb0);
            pf_bh = ld(hi, kb0);
            pf_bln = ld(lo, kb0 + 32);
            pf_bhn = ld(hi, kb0 + 32);
        };
        if (unit0 < units) fetch_bscale(unit0);
        for (int u = unit0; u < units; u += unit_step) {
            int tile, m0, n0, kb0, kb1;
            decode(u, tile, m0, n0, kb0, kb1);
            const int ncol0 = n0 + grp * Cfg::COLS;           // first local column of this thread
            const int gcol0 = p.n_off + ncol0;                // its global column (b_scale index)
            int nb_lo = gcol0 >> 7, nb_hi = (gcol0 >> 7) + 1;  // a thread's columns touch at most two 128-blocks
            nb_lo = nb_lo < p.sn ? nb_lo : p.sn - 1;
            nb_hi = nb_hi < p.sn ? nb_hi : p.sn - 1;
            const int hi_from = 4 - ((gcol0 & 127) >> 5);     // first 32-col chunk that uses nb_hi

            // running sums of this thread's row: 4 chunks of 32 columns, two fp32 per 64-bit register
            unsigned long long acc[Cfg::NCH][16];
#pragma unroll
            for (int c = 0; c < Cfg::NCH; ++c)
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[c][i] = 0ull;

            // b_scale is tiny and warp-uniform.  Lane l holds the values of K block (base + l); every 32 blocks
            // the vector loaded one round earlier takes over, so no iteration waits on a global load.  The first two
            // vectors of a unit were fetched before the previous unit's epilogue (pf_*), so a tile switch does not
            // wait on global memory either (measured: 3 % on 1024 x 7168 x 256, neutral elsewhere).
            const float* bl_ptr = p.b_scale + nb_lo;
            const float* bh_ptr = p.b_scale + nb_hi;
            auto load_bvec = [&](const float* ptr, int kbase) {
                const int k = kbase + lane;
                return (k < kb1) ? __ldg(ptr + static_cast<size_t>(k) * p.sn) : 0.0f;
            };
            float bl_vec = pf_bl, bh_vec = pf_bh, bl_nxt = pf_bln, bh_nxt = pf_bhn;

            if constexpr (RESIDENT) {
                // ---- short K: both K blocks of the tile are in TMEM when the MMA warp hands it over ----
                const bool two = (kb1 - kb0) > 1;
                const float bl0 = __shfl_sync(0xffffffffu, bl_vec, 0) * p.elem_scale;
                const float bh0 = __shfl_sync(0xffffffffu, bh_vec, 0) * p.elem_scale;
                const float bl1 = __shfl_sync(0xffffffffu, bl_vec, 1) * p.elem_scale;
                const float bh1 = __shfl_sync(0xffffffffu, bh_vec, 1) * p.elem_scale;
                if (u + unit_step < units) fetch_bscale(u + unit_step);      // in flight during everything below
                const int si = sgit % SRING;
                ok = wait_bounded(sfull_bar(si), (sgit / SRING) & 1u, abort_flag, p.status, DS_TIMEOUT_SCALE_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const float as0 = sring_ptr[(si * Cfg::SGRP + 0) * 128 + row_in_tile];   // entry released below
                const float as1 = sring_ptr[(si * Cfg::SGRP + 1) * 128 + row_in_tile];   // 0 when K = 128 (zero fill)
                // same arithmetic as the K loop of the other modes: acc = fma(p0, s0, 0), then acc = fma(p1, s1, acc)
                const float s0l = as0 * bl0, s0h = as0 * bh0, s1l = as1 * bl1, s1h = as1 * bh1;
                const unsigned long long s0l2 = pack_f32x2(s0l, s0l), s0h2 = pack_f32x2(s0h, s0h);
                const unsigned long long s1l2 = pack_f32x2(s1l, s1l), s1h2 = pack_f32x2(s1h, s1h);
                // box h belongs to lane h: its previous store has read the box before anything is staged into it
                if (lane < 2) ptx::tma_store_wait_read<0>();
                ok = wait_bounded(tfull_bar(0), tcount & 1u, abort_flag, p.status, DS_TIMEOUT_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                ptx::tc_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(grp * Cfg::COLS);
                const bool last_unit = !(u + unit_step < units);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t v0[64], v1[64];
                    if (two) ptx::tmem_ld_2x64_sync(taddr + h * 64, taddr + BN + h * 64, v0, v1);
                    else ptx::tmem_ld_x64_sync(taddr + h * 64, v0);
                    if (h == 1) {
                        // the whole tile is in registers or staged: the MMA warp may fill TMEM for the next tile
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(tempty_bar(0));
                    }
#pragma unroll
                    for (int i = 0; i < 16; ++i) { acc[0][i] = 0ull; acc[1][i] = 0ull; }
                    ptx::fma32_from64<0>(acc[0], v0, (2 * h >= hi_from) ? s0h2 : s0l2);
                    ptx::fma32_from64<32>(acc[1], v0, (2 * h + 1 >= hi_from) ? s0h2 : s0l2);
                    if (two) {
                        ptx::fma32_from64<0>(acc[0], v1, (2 * h >= hi_from) ? s1h2 : s1l2);
                        ptx::fma32_from64<32>(acc[1], v1, (2 * h + 1 >= hi_from) ? s1h2 : s1l2);
                    }
                    if (last_unit) {
                        // the CTA's last tile: each store leaves as soon as its box is staged (shorter tail)
                        stage_and_store_64<-1>(cmaps.m, p.n_dest, my_stg + h * 4096, my_stg_addr + h * 4096, lane,
                                               PackedCols{acc[0], acc[1]}, ncol0 + h * 64, m0 + quarter * 32, p.M, p.N);
                    } else {
                        stage_64(my_stg + h * 4096, lane, PackedCols{acc[0], acc[1]});
                    }
                }
                if (!last_unit) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    const int mycol = ncol0 + lane * 64;
                    if (lane < 2 && mycol < p.N && m0 + quarter * 32 < p.M) {
                        for (int d = 0; d < p.n_dest; ++d)
                            ptx::tma_store_2d(cmaps.m + d, my_stg_addr + lane * 4096, mycol, m0 + quarter * 32);
                        ptx::tma_store_commit();
                    }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(sempty_bar(si));
                ++sgit;
                ++tcount;
                continue;                                                     // next tile
            }
            if constexpr (!RESIDENT)
            for (int kb = kb0; kb < kb1 && ok; ++kb, ++ait) {
                const int kj = (kb - kb0) & 31;
                if (kj == 0 && kb != kb0) {
                    bl_vec = bl_nxt;
                    bh_vec = bh_nxt;
                    bl_nxt = load_bvec(bl_ptr, kb + 32);
                    bh_nxt = load_bvec(bh_ptr, kb + 32);
                }
                const float bl = __shfl_sync(0xffffffffu, bl_vec, kj) * p.elem_scale;
                const float bh = __shfl_sync(0xffffffffu, bh_vec, kj) * p.elem_scale;
                // a_scale of this row and block, from the ring: one entry holds SGRP consecutive K blocks
                const int kr = (kb - kb0) % Cfg::SGRP;
                const int si = sgit % SRING;
                if (kr == 0) {
                    PROF_T0();
                    ok = wait_bounded(sfull_bar(si), (sgit / SRING) & 1u, abort_flag, p.status, DS_TIMEOUT_SCALE_FULL);
                    PROF_ADD(w_sfull);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                }
                if (pw == 0 && lane == 0) PROF_TRACE(3, ait);
                const float as = sring_ptr[(si * Cfg::SGRP + kr) * 128 + row_in_tile];   // entry released below
                const float s_lo = as * bl, s_hi = as * bh;

                const int b = ait % NBUF;
                { PROF_T0();
                ok = wait_bounded(tfull_bar(b), (ait / NBUF) & 1u, abort_flag, p.status, DS_TIMEOUT_TMEM_FULL);
                PROF_ADD(w_tfull); }
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                // the MMAs of this K block are done: its operands' stage may be refilled
                if constexpr (PROMO_RELEASE)
                    if (pw == 0 && lane == 0) ptx::mbar_arrive(empty_bar(ait % STAGES));
                if (pw == 0 && lane == 0) PROF_TRACE(4, ait);
                if (pw == 1 && lane == 0) PROF_TRACE(7, ait);
                PROF_T0();
                ptx::tc_fence_after_sync();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                                       static_cast<uint32_t>(b * BN + grp * Cfg::COLS);
                // partial sums -> registers, 64 columns per load.  Each load and its wait are one asm statement:
                // the destination registers of a tcgen05.ld are written asynchronously, and code the compiler
                // places between a load and its wait (a spill, a move) would read them too early.
                const unsigned long long s_lo2 = pack_f32x2(s_lo, s_lo), s_hi2 = pack_f32x2(s_hi, s_hi);
                uint32_t v[64];
#pragma unroll
                for (int q = 0; q < Cfg::COLS / 64; ++q) {
                    ptx::tmem_ld_x64_sync(taddr + q * 64, v);
                    if (q == Cfg::COLS / 64 - 1) {
                        // The last columns of the buffer are in registers: hand the TMEM buffer back now, so that
                        // the hand-off to the MMA warp overlaps the FMAs below instead of following them.
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) {
                            if constexpr (CG == 2) ptx::mbar_arrive_cluster(lead_tempty + 8u * b);
                            else ptx::mbar_arrive(tempty_bar(b));
                        }
                    }
                    ptx::fma32_from64<0>(acc[2 * q], v, (2 * q >= hi_from) ? s_hi2 : s_lo2);
                    ptx::fma32_from64<32>(acc[2 * q + 1], v, (2 * q + 1 >= hi_from) ? s_hi2 : s_lo2);
                }
                // Release the a_scale ring entry after its last K block, and only after the FMAs that consumed the
                // value.  An arrive placed straight after the shared-memory read of a_scale (its value not yet
                // used) let the producer refill the entry before a slow warp's read had completed: rare 32-row
                // blocks scaled with the a_scale of a later work unit.
                if (pw == 0 && lane == 0) PROF_TRACE(5, ait);
                if (pw == 1 && lane == 0) PROF_TRACE(8, ait);
                const bool entry_done = (kr == Cfg::SGRP - 1) || (kb == kb1 - 1);
                if (entry_done) {
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(sempty_bar(si));
                    ++sgit;
                }
                PROF_ADD(t_fma);
            }
            if (u + unit_step < units) fetch_bscale(u + unit_step);      // in flight during the epilogue below
#ifdef FP8BS_PROFILE
            const long long epi_start = clock64();
            if (pw == 0 && lane == 0) PROF_TRACE(9, static_cast<uint32_t>((u - unit0) / unit_step));
            if (pw == 0 && lane == 0) { PROF_STAMP(12); }
#endif

            // ---- epilogue of a finished tile: fp32 -> bf16 (round to nearest even), staged, TMA store ----
            auto store_tile = [&]() {
                if constexpr (Cfg::NSTG == 2) {
                    // box h belongs to lane h: its previous store has read the box before anything is staged into it
                    if (lane < 2) ptx::tma_store_wait_read<0>();
                    __syncwarp();
                    if (u + unit_step < units) {
                        stage_and_store_2x64(cmaps.m, p.n_dest, my_stg, my_stg_addr, lane, PackedCols{acc[0], acc[1]},
                                             PackedCols{acc[2], acc[3]}, ncol0, m0 + quarter * 32, p.M, p.N);
                    } else {
                        // the CTA's last tile: the first store leaves while the second box is being staged (shorter tail)
                        stage_and_store_64<-1>(cmaps.m, p.n_dest, my_stg, my_stg_addr, lane, PackedCols{acc[0], acc[1]},
                                               ncol0, m0 + quarter * 32, p.M, p.N);
                        stage_and_store_64<-1>(cmaps.m, p.n_dest, my_stg + 4096, my_stg_addr + 4096, lane,
                                               PackedCols{acc[2], acc[3]}, ncol0 + 64, m0 + quarter * 32, p.M, p.N);
                    }
                } else {
                    stage_and_store_64<0>(cmaps.m, p.n_dest, my_stg, my_stg_addr, lane, PackedCols{acc[0], acc[1]}, ncol0,
                                          m0 + quarter * 32, p.M, p.N);
                }
            };
            if constexpr (MODE == 0) {
                if (!ok) break;
                store_tile();
            } else if constexpr (MODE == 3) {
                if (!ok) break;
                // slot c of the workspace: [BN/4 column quads][128 rows] float4, a warp's 32 rows of one quad contiguous
                auto slot_of = [&](int c) {
                    return p.partials + (static_cast<size_t>(c) * (BN / 4) + grp * (Cfg::COLS / 4)) * 128 + row_in_tile;
                };
                if (kb0 > 0) {
                    // ---- this segment starts inside the tile: publish its partial sums, raise the flag ----
                    float4* part = slot_of(static_cast<int>(blockIdx.x));
#pragma unroll
                    for (int j = 0; j < Cfg::COLS / 4; ++j)
                        part[static_cast<size_t>(j) * 128] =
                            make_float4(f32x2_lo(acc[j / 8][(2 * j) % 16]), f32x2_hi(acc[j / 8][(2 * j) % 16]),
                                        f32x2_lo(acc[j / 8][(2 * j + 1) % 16]), f32x2_hi(acc[j / 8][(2 * j + 1) % 16]));
                    __threadfence();
                    asm volatile("barrier.cta.sync.aligned 1, %0;" ::"n"(Cfg::PROMO_THREADS) : "memory");
                    if (pw == 0 && lane == 0) {
                        __threadfence();      // the whole CTA's partial sums (seen through the barrier) before the flag
                        atomicExch(&p.counters[blockIdx.x], 1u);
                    }
                } else {
                    if (kb1 < KB) {
                        // ---- the tile's first K blocks are here, the rest was (or is being) done by the next CTAs ----
                        int c_end = static_cast<int>(blockIdx.x) + 1;       // CTAs [blockIdx.x + 1, c_end) start inside this tile
                        {
                            const long long tile_end = static_cast<long long>(tile + 1) * KB;
                            const long long T = static_cast<long long>(p.m_tiles) * p.n_tiles * KB;
                            while (c_end < static_cast<int>(gridDim.x) && c_end * T / gridDim.x < tile_end) ++c_end;
                        }
                        for (int c = static_cast<int>(blockIdx.x) + 1; c < c_end; ++c) {
                            if (pw == 0 && lane == 0) {
                                // bounded wait for CTA c's flag
                                const long long t0 = clock64();
                                bool seen = false;
                                while (!seen) {
                                    unsigned int f;
                                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(f) : "l"(p.counters + c) : "memory");
                                    seen = (f != 0u);
                                    if (!seen) {
                                        if (*abort_flag) break;
                                        if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                                            *abort_flag = 1u;
                                            atomicMax(p.status, DS_TIMEOUT_PEER_PARTIAL | (static_cast<uint32_t>(blockIdx.x) << 8));
                                            break;
                                        }
                                        __nanosleep(100);
                                    }
                                }
                                ctrl[2] = seen ? 1u : 0u;
                            }
                            asm volatile("barrier.cta.sync.aligned 1, %0;" ::"n"(Cfg::PROMO_THREADS) : "memory");
                            if (!ctrl[2]) { ok = false; break; }
                            const float4* ps = slot_of(c);
#pragma unroll
                            for (int h = 0; h < Cfg::COLS / 32; ++h) {      // 32 columns = one accumulator chunk per round
                                float4 v[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) v[j] = __ldcg(ps + static_cast<size_t>(h * 8 + j) * 128);
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    // columns 32h + 4j .. +3 are the pairs 2j and 2j + 1 of chunk h
                                    unsigned long long& a0 = acc[h][2 * j];
                                    unsigned long long& a1 = acc[h][2 * j + 1];
                                    a0 = pack_f32x2(f32x2_lo(a0) + v[j].x, f32x2_hi(a0) + v[j].y);
                                    a1 = pack_f32x2(f32x2_lo(a1) + v[j].z, f32x2_hi(a1) + v[j].w);
                                }
                            }
                            // every thread has read slot c: re-arm its flag for the next call
                            asm volatile("barrier.cta.sync.aligned 1, %0;" ::"n"(Cfg::PROMO_THREADS) : "memory");
                            if (pw == 0 && lane == 0) p.counters[c] = 0u;
                        }
                        if (!ok) break;
                    }
                    store_tile();
                }
            } else if constexpr (MODE == 2) {
                // ---- split-K through the cluster: leave this K range's partial tile in shared memory ----
                // The stage buffers are free: every MMA of this CTA has completed (the last TMEM buffer was full)
                // and every load that was issued has been consumed.
                if (ok) {
                    float4* dst = reinterpret_cast<float4*>(aligned + row_in_tile * PART_PITCH + grp * Cfg::COLS * 4);
#pragma unroll
                    for (int j = 0; j < Cfg::COLS / 4; ++j)
                        dst[j] = make_float4(f32x2_lo(acc[j / 8][(2 * j) % 16]), f32x2_hi(acc[j / 8][(2 * j) % 16]),
                                             f32x2_lo(acc[j / 8][(2 * j + 1) % 16]), f32x2_hi(acc[j / 8][(2 * j + 1) % 16]));
                }
            } else {
                // ---- split-K: publish this K range's partial sums ----
                // One 128-row half-tile per CTA.  Layout [half-tile][split][column quad][row]: a warp's
                // 32 rows of one column quad are 512 contiguous bytes, for the writes here and the reads below.
                const int split = u % p.splits;
                const int half_tile = tile * CG + static_cast<int>(rank);
                float4* part = p.partials +
                               ((static_cast<size_t>(half_tile) * p.splits + split) * (BN / 4) + grp * (Cfg::COLS / 4)) * 128 + row_in_tile;
                if (ok) {
#pragma unroll
                    for (int j = 0; j < Cfg::COLS / 4; ++j)
                        part[static_cast<size_t>(j) * 128] =
                            make_float4(f32x2_lo(acc[j / 8][(2 * j) % 16]), f32x2_hi(acc[j / 8][(2 * j) % 16]),
                                        f32x2_lo(acc[j / 8][(2 * j + 1) % 16]), f32x2_hi(acc[j / 8][(2 * j + 1) % 16]));
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
                    __threadfence();      // the partial sums of the whole CTA (seen through the barrier) before the ticket
                    const unsigned int old = atomicAdd(&p.counters[half_tile], 1u);
                    const bool last = (old == static_cast<unsigned int>(p.splits - 1));
                    if (last) p.counters[half_tile] = 0u;     // every split has arrived: re-arm for the next call
                    ctrl[2] = last ? 1u : 0u;
                }
                asm volatile("barrier.cta.sync.aligned 1, %0;" ::"n"(Cfg::PROMO_THREADS) : "memory");
                if (ctrl[2]) {
                    __threadfence();
                    // ---- deterministic reduction: splits are added in the order 0, 1, .., S-1 ----
                    const float4* base = p.partials +
                        (static_cast<size_t>(half_tile) * p.splits * (BN / 4) + grp * (Cfg::COLS / 4)) * 128 + row_in_tile;
#pragma unroll
                    for (int h = 0; h < Cfg::COLS / 64; ++h) {
                        float sum[64];
#pragma unroll
                        for (int i = 0; i < 64; ++i) sum[i] = 0.0f;
                        for (int s = 0; s < p.splits; ++s) {
                            const float4* ps = base + static_cast<size_t>(s) * (BN / 4) * 128;
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const float4 v = __ldcg(ps + static_cast<size_t>(h * 16 + j) * 128);
                                sum[4 * j + 0] += v.x;
                                sum[4 * j + 1] += v.y;
                                sum[4 * j + 2] += v.z;
                                sum[4 * j + 3] += v.w;
                            }
                        }
                        stage_and_store_64<0>(cmaps.m, p.n_dest, my_stg, my_stg_addr, lane, FloatCols{sum}, ncol0 + h * 64, m0 + quarter * 32, p.M, p.N);
                    }
                }
            }
#ifdef FP8BS_PROFILE
            t_epi += clock64() - epi_start;
            if (pw == 0 && lane == 0) PROF_TRACE(10, static_cast<uint32_t>((u - unit0) / unit_step));
#endif
        }
#ifdef FP8BS_PROFILE
        t_epi += 0;
        if (pw == 0 && lane == 0) { PROF_OUT(4, w_sfull); PROF_OUT(5, w_tfull); PROF_OUT(6, t_fma); PROF_OUT(7, t_epi); PROF_STAMP(13); }
#endif
        // C must have been read out of shared memory before the CTA goes away
        if (lane < 2) ptx::tma_store_wait_read<0>();
        __syncwarp();
    }

    if constexpr (MODE == 2) {
        // ------------------------------------------------------------ cluster reduction ---
        __syncthreads();                 // this CTA's partial tile is complete ...
        ptx::cluster_sync();             // ... and so are those of the other K ranges of the tile
        if (warp >= 4 && *abort_flag == 0u) {
            const int S = p.splits;
            const int my = static_cast<int>(ptx::cluster_ctarank());     // = this CTA's split index
            int tile, m0, n0, kb0, kb1;
            decode(static_cast<int>(blockIdx.x), tile, m0, n0, kb0, kb1);
            const int r0 = (128 * my) / S, r1 = (128 * (my + 1)) / S;     // the rows this CTA finishes
            uint32_t peer[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) peer[s] = ptx::mapa(stage_base, static_cast<uint32_t>(s < S ? s : 0));
            const int items = (r1 - r0) * (BN / 4);
            for (int idx = static_cast<int>(threadIdx.x) - 128; idx < items; idx += Cfg::PROMO_THREADS) {
                const int row = r0 + idx / (BN / 4), c4 = idx % (BN / 4);
                const uint32_t off = static_cast<uint32_t>(row * PART_PITCH + c4 * 16);
                float4 v[8];
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < S) v[s] = ptx::ld_shared_cluster_v4(peer[s] + off);
                float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int s = 0; s < 8; ++s)              // fixed order 0, 1, .., S-1: bit-deterministic
                    if (s < S) { sum.x += v[s].x; sum.y += v[s].y; sum.z += v[s].z; sum.w += v[s].w; }
                const int m = m0 + row, n = n0 + c4 * 4;
                if (m < p.M && n < p.N) {
                    uint2 q;
                    q.x = pack_bf16x2(sum.x, sum.y);
                    q.y = pack_bf16x2(sum.z, sum.w);
                    *reinterpret_cast<uint2*>(p.C + static_cast<size_t>(m) * p.N + n) = q;
                }
            }
        }
    }

    // ---------------------------------------------------------------- common exit -----
    ptx::tc_fence_before_sync();
    __syncthreads();
    if constexpr (CG == 2 || MODE == 2) ptx::cluster_sync();   // nothing remote may touch this CTA after it has left
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        if constexpr (CG == 2) ptx::tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
        else ptx::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
    if (threadIdx.x == 0) { PROF_STAMP(14); PROF_CLK1(15); }
}

}  // namespace fp8bs

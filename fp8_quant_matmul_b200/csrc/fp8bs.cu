// libfp8bs.so: the C ABI declared in include/fp8bs.h -- argument checking, run-time shape
// dispatch, TMA descriptor construction and kernel launches.  Host-side role of the
// reference's gemmGPU wrapper and its geometry switch (check.cu:51-130).
#include "../../include/fp8bs.h"
#include "gemm_kernel.cuh"

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <cstdlib>
#include <mutex>
#include <new>

namespace fp8bs {

// ---------------------------------------------------------------------------------------
// per-thread / per-process state
// ---------------------------------------------------------------------------------------
static thread_local int tl_last_cuda_error = 0;
static std::atomic<unsigned long long> g_launches{0};

// Device status word written by kernels whose bounded waits expire.
__device__ unsigned int g_device_status[4];

// Built-in split-K scratch for fp8bs_gemm_mn_small_static: tile counters (first 64 KiB) followed by the fp32
// partial sums.  It lives in the library's device image, so every GPU that loads the library holds these
// bytes until the process exits; that is why the size is kept modest.
constexpr size_t STATIC_SCRATCH_BYTES = FP8BS_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

#define CUDA_TRY(expr)                                     \
    do {                                                   \
        cudaError_t e__ = (expr);                          \
        if (e__ != cudaSuccess) {                          \
            tl_last_cuda_error = static_cast<int>(e__);    \
            (void)cudaGetLastError();                      \
            return FP8BS_ERR_CUDA;                         \
        }                                                  \
    } while (0)

constexpr int MAX_DEVICES = 64;
constexpr size_t COUNTER_BYTES = 65536;            // head of the workspace: 16384 tile counters
constexpr int MAX_SPLITS = 32;
constexpr size_t BSCALE_MAX_BYTES = 4u << 20;     // b_scale staging of the end-to-end context

// What the dispatch needs to know about a GPU: how many SMs, and how many thread-block clusters of each size
// (one CTA per SM, this library's shared-memory footprint) can be resident at once.
struct DeviceModel {
    int sm_count;
    int max_clusters[9];
};
// A full B200: 148 SMs; cudaOccupancyMaxActiveClusters for the split-K kernel gives 148/74/45/33/26/22/15/15 for
// cluster sizes 1..8.  Used when no device has been set up (the pure host functions on a machine without a GPU).
static const DeviceModel kB200Model = {148, {0, 148, 74, 45, 33, 26, 22, 15, 15}};

// The model of a GPU with `sm_count` SMs when it cannot be asked: the B200 table scaled by the SM count.
static DeviceModel scaled_model(int sm_count)
{
    DeviceModel m = kB200Model;
    if (sm_count > 0 && sm_count != kB200Model.sm_count) {
        m.sm_count = sm_count;
        for (int s = 1; s <= 8; ++s) {
            m.max_clusters[s] = kB200Model.max_clusters[s] * sm_count / kB200Model.sm_count;
            if (m.max_clusters[s] < 1 && s <= sm_count) m.max_clusters[s] = 1;
        }
    }
    return m;
}

struct DeviceInfo {
    bool ready = false;
    int status = FP8BS_OK;
    int sm_count = 0;
    DeviceModel model = kB200Model;
    unsigned int* status_ptr = nullptr;            // device address of g_device_status
    void* static_scratch = nullptr;                // device address of g_static_scratch (looked up on first use)
};
static DeviceInfo g_dev[MAX_DEVICES];
static std::mutex g_dev_mutex;

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn g_encode_tiled = nullptr;
static const bool g_use_pdl = []() { const char* e = std::getenv("FP8BS_PDL"); return !(e && e[0] == '0'); }();
#ifdef FP8BS_PROFILE
static long long* g_prof_buf = nullptr;
#endif

template <int BN, int CG, int MODE>
static int prepare_kernel()
{
    CUDA_TRY(cudaFuncSetAttribute(gemm_kernel<BN, CG, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  TileCfg<BN, CG>::SMEM_BYTES));
    return FP8BS_OK;
}

// One-time set-up for the current device: capability check, kernel attributes, driver
// entry point for tensor-map encoding (looked up at run time so that the library has no
// link-time dependency on libcuda and loads on a machine without a driver).
static int device_setup(DeviceInfo** out)
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        (void)cudaGetLastError();
        return FP8BS_ERR_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceInfo& d = g_dev[dev];
    if (!d.ready) {
        d.ready = true;
        d.status = FP8BS_ERR_NO_DEVICE;
        int major = 0;
        if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess || major != 10) {
            (void)cudaGetLastError();
            return d.status;
        }
        if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return d.status;
        if (!g_encode_tiled) {
            void* fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
                qres != cudaDriverEntryPointSuccess || !fn) {
                (void)cudaGetLastError();
                return d.status;
            }
            g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
        }
        int rc;
        if ((rc = prepare_kernel<128, 1, 0>()) || (rc = prepare_kernel<256, 1, 0>()) ||
            (rc = prepare_kernel<256, 2, 0>()) || (rc = prepare_kernel<128, 1, 1>()) ||
            (rc = prepare_kernel<256, 1, 1>()) || (rc = prepare_kernel<256, 2, 1>()) ||
            (rc = prepare_kernel<128, 1, 2>()) || (rc = prepare_kernel<256, 1, 2>()) ||
            (rc = prepare_kernel<128, 1, 3>()) || (rc = prepare_kernel<256, 1, 3>()) ||
            (rc = prepare_kernel<256, 1, 4>())) {
            d.status = rc;
            return rc;
        }
        void* sp = nullptr;
        if (cudaGetSymbolAddress(&sp, g_device_status) != cudaSuccess) {
            (void)cudaGetLastError();
            d.status = FP8BS_ERR_CUDA;
            return d.status;
        }
        d.status_ptr = static_cast<unsigned int*>(sp);
        // cluster occupancy of the split-K kernel on this device (both tile widths have the same footprint)
        d.model = scaled_model(d.sm_count);
        for (int cs = 1; cs <= 8; ++cs) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(static_cast<unsigned>(cs * 64), 1, 1);
            cfg.blockDim = dim3(TileCfg<128, 1>::THREADS, 1, 1);
            cfg.dynamicSmemBytes = TileCfg<128, 1>::SMEM_BYTES;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = static_cast<unsigned>(cs);
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_kernel<128, 1, 2>, &cfg) == cudaSuccess && n > 0) d.model.max_clusters[cs] = n;
            else (void)cudaGetLastError();
        }
        if (cudaMemset(sp, 0, sizeof(unsigned int) * 4) != cudaSuccess) {
            (void)cudaGetLastError();
            d.status = FP8BS_ERR_CUDA;
            return d.status;
        }
        d.status = FP8BS_OK;
    }
    if (out) *out = &d;
    return d.status;
}

// The model the pure host functions plan with: that of the current device once a call has set it up, else a full
// B200.  Never touches a device that has not been set up, so it works on a machine without a GPU.
static DeviceModel host_model()
{
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
        (void)cudaGetLastError();
        return kB200Model;
    }
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    return (g_dev[dev].ready && g_dev[dev].status == FP8BS_OK) ? g_dev[dev].model : kB200Model;
}

// ---------------------------------------------------------------------------------------
// dispatch
// ---------------------------------------------------------------------------------------
struct Config {
    int path;     // FP8BS_PATH_MN_LARGE / FP8BS_PATH_MN_SMALL
    int tile_n;   // 128 or 256
    int splits;   // 1 for mn_large
    int cg;       // 1: a CTA owns 128 rows of a tile; 2: a pair of CTAs owns 256 rows
    int mode;     // 0 full K; 1 split-K reduced through a workspace; 2 split-K reduced inside a cluster;
                  // 3 stream-K: the K blocks of all tiles dealt out evenly over `ctas` CTAs; 4 short K (K <= 256):
                  // full K with both K blocks of a tile resident in TMEM
    int ctas;     // mode 3 only
};

constexpr int MAX_CLUSTER_SPLITS = 8;   // portable cluster size limit; 7 and 8 fit only 15 at a time on a B200

static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Stream-K grid: every SM, but at least 4 K blocks per CTA.  Never more CTAs than SMs: a CTA waits (bounded) for
// partial tiles of CTAs that must therefore be running at the same time.
static int stream_k_ctas(int tiles, int KB, int sm_count)
{
    const long long total = static_cast<long long>(tiles) * KB;
    long long g = total / 4;
    if (g > sm_count) g = sm_count;
    if (g < 1) g = 1;
    return static_cast<int>(g);
}


// Estimated run time of a configuration in microseconds.  The constants come from a measured sweep of
// every configuration over the 18 benchmark shapes on a B200 (power-capped, cold L2):
//   per 128-K block of one work unit: 0.44 us (128-wide tile), 0.53 us (256-wide), 0.505 us (256 x 256 pair, with
//   one multicast commit per K block and the stages freed by a promotion warp: the pair wins from K = 1536 on,
//   2 % at K = 1536 and M = 6144 (equal at M = 1024), 3-5 % from K = 2048 on; at K = 512 it is 2-8 % slower);
//   per work unit (tile switch, epilogue): 0.35 / 1.2 / 1.40 us;  per launch: 3.5 us;
//   split-K through a workspace: 3.5 us + 1 us per split and 128 columns for the partial-sum round trip, doubled
//   when a CTA has to walk more than one unit (the last-arriver reduction then delays the next unit);
//   split-K inside a cluster: one CTA per (tile, K range); the number of clusters that fit on the GPU at once is
//   cudaOccupancyMaxActiveClusters for this kernel's footprint (one CTA per SM), tabulated below for a B200;
//   overhead 2 us (3 us for 256-wide tiles) + 0.5 us per split and 128 columns (shared-memory round trip, two
//   cluster barriers), paid again with 3 us of prologue by every further wave of clusters.
// Stream-K hand-over per 128 columns of tile width: a CTA first leaves a partial tile in the workspace (its promotion
// warps are busy with that while its MMA warp runs dry) and at the end reads its neighbours'; CTAs that run side by side
// are also on tiles far apart and share less through L2.  Measured 6-11 us in total on the benchmark shapes, which
// is why the estimate keeps stream-K for shapes with very few, very long tiles only.
constexpr double STREAM_K_FIXUP_US = 6.0;
// Mode 4 (K <= 256, partial sums resident in TMEM) is chosen by rule, see choose_config.
constexpr int SHORT_K_MAX_WAVES = 3;
static double config_cost(const DeviceModel& dm, int M, int N, int K, int tile_n, int splits, int cg, int mode)
{
    const int KB = K / 128;
    const int tiles = ceil_div(M, 128 * cg) * ceil_div(N, tile_n);
    if (mode == 3) {
        // every CTA: ceil(T / G) K blocks, its share of the tile switches, one partial-sum hand-over each way
        const int g = stream_k_ctas(tiles, KB, dm.sm_count);
        const long long total = static_cast<long long>(tiles) * KB;
        const double kb_each = static_cast<double>((total + g - 1) / g);
        const double per_kb3 = (tile_n == 256 ? 0.53 : 0.44), per_unit3 = (tile_n == 256 ? 1.2 : 0.35);
        // the CTA that finishes a tile reads the partial tile of every other CTA that worked on it, one after the other
        const double sharers = (kb_each < KB) ? (KB / kb_each + 1.0) : 2.0;
        return 3.5 + kb_each * per_kb3 + (static_cast<double>(tiles) / g + 1.0) * per_unit3 +
               STREAM_K_FIXUP_US * (tile_n / 128) * (sharers / 2.0);
    }
    const int units = tiles * splits;
    if (dm.sm_count < cg || (mode == 2 && dm.max_clusters[splits] < 1)) return 1e300;   // cannot run on this device
    const int waves = (mode == 2) ? ceil_div(tiles, dm.max_clusters[splits]) : ceil_div(units, dm.sm_count / cg);
    const double per_kb = (cg == 2) ? 0.505 : (tile_n == 256 ? 0.53 : 0.44);
    const double per_unit = (cg == 2) ? 1.40 : (tile_n == 256 ? 1.2 : 0.35);
    double cost = 3.5 + waves * (ceil_div(KB, splits) * per_kb + per_unit);
    if (splits > 1 && mode == 2) {
        // One CTA per (tile, K range), not persistent: a second wave of clusters pays the prologue and the
        // reduction again, and nothing of it overlaps the wave before (measured on M = 16384 shapes).
        const double overhead = (tile_n == 256 ? 3.0 : 2.0) + 0.5 * splits * (tile_n / 128);
        cost += overhead + (waves - 1) * (overhead + 3.0);
    } else if (splits > 1) {
        // (pair tiles through the workspace measured 1.5 % slower than single-CTA tiles on 1024 x 1536 x 7168: + 1 us)
        const double overhead = 3.5 + 1.0 * splits * (tile_n / 128) + (cg == 2 ? 1.0 : 0.0);
        cost += (waves > 1) ? 2.0 * overhead : overhead;
    }
    return cost;
}

// tile_n argument of the API: 0 = choose; 128 or 256 = tile width, one CTA per tile;
// 256 | FP8BS_TILE_PAIR = 256 x 256 tile owned by a pair of CTAs; | FP8BS_SPLIT_WORKSPACE = reduce split-K partial
// sums through the workspace even where the cluster reduction could be used.
static Config choose_config(const DeviceModel& dm, int M, int N, int K, int path, int splits, int tile_n)
{
    const int KB = K / 128;
    const bool force_ws = (tile_n & FP8BS_SPLIT_WORKSPACE) != 0;
    const bool force_sk = (tile_n & FP8BS_STREAM_K) != 0;
    const int want_tile = tile_n & ~(FP8BS_SPLIT_WORKSPACE | FP8BS_STREAM_K | FP8BS_SHORT_K);
    Config best{FP8BS_PATH_MN_LARGE, 128, 1, 1, 0, 0};
    double best_cost = 1e300;
    // short K: the tile's partial sums stay in TMEM (mode 4), a member of the mn_large family (K is not cut)
    if (tile_n & FP8BS_SHORT_K) return Config{FP8BS_PATH_MN_LARGE, 256, 1, 1, 4, 0};
    if (KB <= 2 && path != FP8BS_PATH_MN_SMALL && splits <= 1 && !force_ws && !force_sk && want_tile == 0) {
        // Measured on a B200: 5-6 % faster than the full-K kernel at K = 128 and, at K = 256, up to about three tiles
        // per SM (1024 x 7168 x 256, 1.5 per SM: 7.20 against 7.64 us; 2048 x 7168 x 256, 3.0: 11.1 against 11.4);
        // with more tiles the store path of the SMs sets the pace and the full-K kernel, which overlaps the MMAs of
        // a tile with the scaling of the one before, is ahead (3072 x 7168 x 256, 4.5 per SM: 14.1 against 14.9 us;
        // 6144 x 7168 x 256, 9.1: 23.7 against 24.4).
        const int tiles = ceil_div(M, 128) * ceil_div(N, 256);
        if (KB == 1 || tiles <= SHORT_K_MAX_WAVES * dm.sm_count) return Config{FP8BS_PATH_MN_LARGE, 256, 1, 1, 4, 0};
    }
    // stream-K: a member of the mn_small family (it cuts K), chosen when it is asked for or when the caller left
    // both path and splits open
    if (force_sk || (path != FP8BS_PATH_MN_LARGE && splits == 0 && !force_ws)) {
        for (int tn = 128; tn <= 256; tn += 128) {
            if (want_tile && want_tile != tn) continue;
            const int tiles = ceil_div(M, 128) * ceil_div(N, tn);
            // With more tiles than SMs the CTAs that run side by side are on tiles far apart and share little
            // through L2 (measured: 369 us against 186 us on 16384 x 1536 x 7168): only on request there.
            if (!force_sk && tiles > dm.sm_count) continue;
            const double c = config_cost(dm, M, N, K, tn, 1, 1, 3);
            if (c < best_cost) {
                best_cost = c;
                best = Config{FP8BS_PATH_MN_SMALL, tn, 1, 1, 3, stream_k_ctas(tiles, KB, dm.sm_count)};
            }
        }
        if (force_sk) return best;
    }
    for (int cg = 1; cg <= 2; ++cg)
        for (int tn = 128; tn <= 256; tn += 128) {
            if (cg == 2 && tn != 256) continue;
            if (want_tile && want_tile != (tn | (cg == 2 ? FP8BS_TILE_PAIR : 0))) continue;
            const int smax = (path == FP8BS_PATH_MN_LARGE) ? 1 : (KB < MAX_SPLITS ? KB : MAX_SPLITS);
            for (int s = 1; s <= smax; ++s) {
                if (splits && s != splits) continue;
                const bool small = (s > 1 || path == FP8BS_PATH_MN_SMALL);
                const bool cluster_ok = small && cg == 1 && s >= 2 && s <= MAX_CLUSTER_SPLITS && !force_ws &&
                                        dm.max_clusters[s] > 0;
                for (int mode = small ? 1 : 0; mode <= (cluster_ok ? 2 : (small ? 1 : 0)); ++mode) {
                    const double c = config_cost(dm, M, N, K, tn, s, cg, mode);
                    if (c < best_cost) {
                        best_cost = c;
                        best = Config{small ? FP8BS_PATH_MN_SMALL : FP8BS_PATH_MN_LARGE, tn, s, cg, mode, 0};
                    }
                }
            }
        }
    return best;
}

static size_t config_workspace(int M, int N, const Config& c)
{
    if (c.mode == 3)                                                 // flags + one partial tile per CTA
        return COUNTER_BYTES + static_cast<size_t>(c.ctas) * (static_cast<size_t>(c.tile_n) * 128 * sizeof(float));
    if (c.path != FP8BS_PATH_MN_SMALL || c.mode != 1) return 0;      // only the workspace reduction needs scratch
    const size_t half_tiles = static_cast<size_t>(ceil_div(M, 128 * c.cg)) * c.cg * ceil_div(N, c.tile_n);
    return COUNTER_BYTES + half_tiles * c.splits * (static_cast<size_t>(c.tile_n) * 128 * sizeof(float));
}

static int check_shape(int M, int N, int K)
{
    if (M <= 0 || N <= 0 || K <= 0 || K % 128 != 0) return FP8BS_ERR_SHAPE;
    if (M % 16 != 0 || N % 16 != 0) return FP8BS_ERR_ALIGN;
    return FP8BS_OK;
}

static int check_args(int M, int N, int K, int n0, int n_total, int path, int splits, int tile_n)
{
    int rc = check_shape(M, N, K);
    if (rc) return rc;
    if (path < FP8BS_PATH_AUTO || path > FP8BS_PATH_MN_SMALL) return FP8BS_ERR_ARG;
    if (splits < 0 || splits > K / 128 || splits > MAX_SPLITS) return FP8BS_ERR_ARG;
    if (path == FP8BS_PATH_MN_LARGE && splits > 1) return FP8BS_ERR_ARG;
    {
        const int t = tile_n & ~(FP8BS_SPLIT_WORKSPACE | FP8BS_STREAM_K | FP8BS_SHORT_K);
        if (t != 0 && t != 128 && t != 256 && t != (256 | FP8BS_TILE_PAIR)) return FP8BS_ERR_ARG;
        if ((tile_n & FP8BS_SHORT_K) && ((t != 0 && t != 256) || (tile_n & (FP8BS_SPLIT_WORKSPACE | FP8BS_STREAM_K)) ||
                                         splits > 1 || path == FP8BS_PATH_MN_SMALL || K > 256))
            return FP8BS_ERR_ARG;
        if ((tile_n & FP8BS_STREAM_K) && ((tile_n & (FP8BS_TILE_PAIR | FP8BS_SPLIT_WORKSPACE)) || splits > 1 ||
                                          path == FP8BS_PATH_MN_LARGE))
            return FP8BS_ERR_ARG;
    }
    if (n0 < 0 || n0 % 64 != 0 || n_total < n0 + N) return FP8BS_ERR_ARG;
    return FP8BS_OK;
}

// ---------------------------------------------------------------------------------------
// launch
// ---------------------------------------------------------------------------------------
static int encode_operand_map(CUtensorMap* tm, const void* base, int mn, int K)
{
    // Global view: 8-bit elements, dimension 0 = M (or N), contiguous; dimension 1 = K with
    // a stride of M (or N) bytes.  Box = 128 x 128, 128-byte swizzle, zero fill outside.
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(mn), static_cast<cuuint64_t>(K)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(mn)};
    const cuuint32_t box[2] = {128u, 128u};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = g_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_last_cuda_error = static_cast<int>(r);
        return FP8BS_ERR_CUDA;
    }
    return FP8BS_OK;
}

// a_scale as a 2-D fp32 tensor {M, K/128}; one box = the scales of a tile's 128 rows for SCALE_GROUP K blocks.
static int encode_scale_map(CUtensorMap* tm, const float* base, int M, int KB)
{
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(M), static_cast<cuuint64_t>(KB)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(M) * 4};
    const cuuint32_t box[2] = {128u, static_cast<cuuint32_t>(SCALE_GROUP)};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = g_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides,
                                      box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_last_cuda_error = static_cast<int>(r);
        return FP8BS_ERR_CUDA;
    }
    return FP8BS_OK;
}

// C as a 2-D bf16 tensor {N, M} (row-major M x N); a store box is 64 columns x 32 rows, 128-byte swizzled.
static int encode_c_map(CUtensorMap* tm, void* base, int M, int N, int ld)
{
    // `base` is the first element of the M x N window this call writes; `ld` is the row pitch of the buffer in elements
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(M)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
    const cuuint32_t box[2] = {64u, 32u};
    const cuuint32_t estr[2] = {1u, 1u};
    const CUresult r = g_encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        tl_last_cuda_error = static_cast<int>(r);
        return FP8BS_ERR_CUDA;
    }
    return FP8BS_OK;
}

struct TensorMaps {
    CUtensorMap A, B, As;
    CMaps C;
};

template <int BN, int CG, int MODE>
static int launch(const TensorMaps& tm, const GemmParams& p, int sm_count, cudaStream_t stream)
{
    using Cfg = TileCfg<BN, CG>;
    const int units = p.m_tiles * p.n_tiles * p.splits;
    int groups = units < sm_count / CG ? units : sm_count / CG;    // tile walkers: CTAs or CTA pairs
    if (MODE == 2) groups = units;                                  // one CTA per (tile, K range); a cluster per tile
    if (MODE == 3) groups = stream_k_ctas(p.m_tiles * p.n_tiles, p.K / 128, sm_count);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(groups * CG), 1, 1);
    cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (MODE == 2) ? static_cast<unsigned>(p.splits) : CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // The kernel does its set-up, then waits for the previous kernel of the stream (griddepcontrol.wait) before it
    // touches global memory: letting it start early hides launch latency and set-up behind that kernel's tail.
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_use_pdl ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_kernel<BN, CG, MODE>, tm.A, tm.B, tm.As, tm.C, p);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    CUDA_TRY(e);
    return FP8BS_OK;
}

static int launch_config(const Config& c, const TensorMaps& tm, const GemmParams& p, int sm_count, cudaStream_t st)
{
    if (c.mode == 3)
        return c.tile_n == 256 ? launch<256, 1, 3>(tm, p, sm_count, st) : launch<128, 1, 3>(tm, p, sm_count, st);
    if (c.mode == 2)
        return c.tile_n == 256 ? launch<256, 1, 2>(tm, p, sm_count, st) : launch<128, 1, 2>(tm, p, sm_count, st);
    if (c.mode == 1) {
        if (c.cg == 2) return launch<256, 2, 1>(tm, p, sm_count, st);
        return c.tile_n == 256 ? launch<256, 1, 1>(tm, p, sm_count, st) : launch<128, 1, 1>(tm, p, sm_count, st);
    }
    if (c.mode == 4) return launch<256, 1, 4>(tm, p, sm_count, st);
    if (c.cg == 2) return launch<256, 2, 0>(tm, p, sm_count, st);
    return c.tile_n == 256 ? launch<256, 1, 0>(tm, p, sm_count, st) : launch<128, 1, 0>(tm, p, sm_count, st);
}

// `dests` / `n_dest`: null / 0 for the ordinary call (C is an M x N buffer of its own); otherwise n_dest buffers of
// n_total columns each, all of which receive this call's columns [n0, n0 + N) (C is ignored).
static int gemm_impl(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M,
                     int N, int K, int n0, int n_total, int path, int splits, int tile_n, void* workspace,
                     size_t workspace_bytes, void* stream, void* const* dests = nullptr, int n_dest = 0)
{
    if (dests) {
        if (n_dest < 1 || n_dest > MAX_DEST) return FP8BS_ERR_ARG;
        for (int d = 0; d < n_dest; ++d) {
            if (!dests[d]) return FP8BS_ERR_NULL;
            if (reinterpret_cast<uintptr_t>(dests[d]) & 15u) return FP8BS_ERR_ALIGN;
        }
        if (n_total % 8 != 0) return FP8BS_ERR_ALIGN;       // row pitch of the destinations: a multiple of 16 bytes
        C = dests[0];
    }
    if (!A || !B || !a_scale || !b_scale || !C) return FP8BS_ERR_NULL;
    int rc = check_args(M, N, K, n0, n_total, path, splits, tile_n);
    if (rc) return rc;
    if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15u)
        return FP8BS_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(a_scale) & 15u) || (reinterpret_cast<uintptr_t>(b_scale) & 3u)) return FP8BS_ERR_ALIGN;

    // The device is set up before the dispatch decides (its SM count and cluster occupancy go into the decision),
    // but a failure here is only reported once the remaining argument and workspace checks have passed.
    DeviceInfo* dev = nullptr;
    const int dev_rc = device_setup(&dev);
    const DeviceModel dm = (dev_rc == FP8BS_OK) ? dev->model : kB200Model;
    Config cfg = choose_config(dm, M, N, K, path, splits, tile_n);
    if (dests && cfg.mode == 2) return FP8BS_ERR_ARG;       // the cluster reduction stores C itself, to one buffer
    if (cfg.mode == 1 || cfg.mode == 3) {
        const size_t need = config_workspace(M, N, cfg);
        const size_t half_tiles = (cfg.mode == 3) ? static_cast<size_t>(cfg.ctas)
            : static_cast<size_t>(ceil_div(M, 128 * cfg.cg)) * cfg.cg * ceil_div(N, cfg.tile_n);
        const bool fits = workspace && workspace_bytes >= need && half_tiles <= COUNTER_BYTES / sizeof(unsigned int) &&
                          (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0;
        if (!fits) {
            if (path != FP8BS_PATH_AUTO || (tile_n & (FP8BS_STREAM_K | FP8BS_SPLIT_WORKSPACE))) return FP8BS_ERR_WORKSPACE;
            cfg = choose_config(dm, M, N, K, FP8BS_PATH_MN_LARGE, 1, tile_n);   // best full-K configuration
        }
    }
    if (dev_rc) return dev_rc;

    TensorMaps tm{};
    if ((rc = encode_operand_map(&tm.A, A, M, K))) return rc;
    if ((rc = encode_operand_map(&tm.B, B, N, K))) return rc;
    if ((rc = encode_scale_map(&tm.As, a_scale, M, K / 128))) return rc;
    if (dests) {
        for (int d = 0; d < n_dest; ++d)
            if ((rc = encode_c_map(&tm.C.m[d], static_cast<__nv_bfloat16*>(dests[d]) + n0, M, N, n_total))) return rc;
    } else if ((rc = encode_c_map(&tm.C.m[0], C, M, N, N))) return rc;

    GemmParams p;
    p.b_scale = b_scale;
    p.C = static_cast<__nv_bfloat16*>(C);
    p.partials = nullptr;
    p.counters = nullptr;
    p.status = dev->status_ptr;
    p.M = M; p.N = N; p.K = K;
    p.n_off = n0;
    p.sn = ceil_div(n_total, 128);
    p.m_tiles = ceil_div(M, 128 * cfg.cg);
    p.n_tiles = ceil_div(N, cfg.tile_n);
    p.inv_m_tiles = 1.0f / static_cast<float>(p.m_tiles);
    p.splits = cfg.splits;
    p.n_dest = dests ? n_dest : 1;
    p.elem_scale = 1.0f;
#ifdef FP8BS_PROFILE
    {
        static long long* prof_buf = nullptr;       // profiling builds only: 8 counters per CTA, read by fp8bs_debug_prof
        if (!prof_buf) cudaMalloc(&prof_buf, 16 * 1024 * sizeof(long long));
        cudaMemsetAsync(prof_buf, 0, 16 * 1024 * sizeof(long long), static_cast<cudaStream_t>(stream));
        p.prof = prof_buf;
        g_prof_buf = prof_buf;
    }
#endif
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    if (cfg.mode == 1 || cfg.mode == 3) {
        p.counters = static_cast<unsigned int*>(workspace);
        p.partials = reinterpret_cast<float4*>(static_cast<char*>(workspace) + COUNTER_BYTES);
    }
    return launch_config(cfg, tm, p, dev->sm_count, st);
}

// ---------------------------------------------------------------------------------------
// scalar kernels: ground truth restated (check.cu:30-49) and fp32 -> fp8 (check.cu:17-22)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float e4m3fn_decode(uint8_t b)
{
    const uint32_t e = (b >> 3) & 0xFu, m = b & 7u;
    float v;
    if (e == 0xFu && m == 7u) v = __int_as_float(0x7fc00000);
    else if (e == 0u) v = static_cast<float>(m) * 0.001953125f;                    // m * 2^-9
    else v = __int_as_float(((e + 120u) << 23) | (m << 20));                         // (1 + m/8) * 2^(e-7)
    return (b & 0x80u) ? -v : v;
}

// Thread (n, m): n across the warp so the B reads coalesce; per 128-K block a sequential
// fp32 sum, then result += block * as * bs, then a round-to-nearest-even bf16 cast.
__global__ void ref_gemm_kernel(const uint8_t* __restrict__ A, const uint8_t* __restrict__ B,
                                const float* __restrict__ as, const float* __restrict__ bs,
                                __nv_bfloat16* __restrict__ C, int M, int N, int K)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y * blockDim.y + threadIdx.y;
    if (m >= M || n >= N) return;
    const int sn = (N + 127) / 128;
    float result = 0.0f;
    for (int kb = 0; kb < K / 128; ++kb) {
        float block = 0.0f;
        for (int kk = 0; kk < 128; ++kk) {
            const size_t k = static_cast<size_t>(kb) * 128 + kk;
            block = __fmaf_rn(e4m3fn_decode(A[m + k * M]), e4m3fn_decode(B[n + k * N]), block);
        }
        result = __fadd_rn(result, __fmul_rn(__fmul_rn(block, as[m + static_cast<size_t>(kb) * M]),
                                             bs[n / 128 + static_cast<size_t>(kb) * sn]));
    }
    C[static_cast<size_t>(m) * N + n] = __float2bfloat16_rn(result);
}

__host__ __device__ inline uint8_t float_to_e4m3fn_rne(float x)
{
    uint32_t u;
#ifdef __CUDA_ARCH__
    u = __float_as_uint(x);
#else
    std::memcpy(&u, &x, 4);
#endif
    const uint8_t sign = static_cast<uint8_t>((u >> 24) & 0x80u);
    const uint32_t a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return 0x7F;                         // NaN
    if (a >= 0x43e80000u) return sign | 0x7E;                 // >= 464 (and inf): saturate to 448
    if (a < 0x3a800000u) {                                    // < 2^-10: rounds to 0 or the first subnormal
        // 2^-10 itself is the midpoint between 0 and 2^-9 and ties to even (0)
        return sign;
    }
    const int e = static_cast<int>(a >> 23) - 127;            // unbiased exponent
    if (e < -6) {
        // subnormal target: value = q * 2^-9, q in 0..8 (8 promotes to the first normal)
        const uint32_t mant = (a & 0x7fffffu) | 0x800000u;    // 1.m as a 24-bit integer, value mant * 2^(e-23)
        const int shift = (-9) - (e - 23);                    // q = mant >> shift, shift = 14 - e in 21..24
        uint32_t q = mant >> shift;
        const uint32_t rem = mant & ((1u << shift) - 1u), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (q & 1u))) ++q;
        return sign | static_cast<uint8_t>(q);                // q == 8 is exactly the encoding of 2^-6
    }
    uint32_t q = (a >> 20) & 7u;                              // top three mantissa bits
    const uint32_t rem = a & 0xfffffu, half = 0x80000u;
    uint32_t be = static_cast<uint32_t>(e + 7);
    if (rem > half || (rem == half && (q & 1u))) {
        if (++q == 8u) { q = 0u; ++be; }
    }
    if (be > 15u || (be == 15u && q == 7u)) return sign | 0x7E;
    return sign | static_cast<uint8_t>((be << 3) | q);
}

}  // namespace fp8bs
#include "quantize.cuh"
namespace fp8bs {

__global__ void convert_float_to_e4m3fn_kernel(const float* __restrict__ in, uint8_t* __restrict__ out, size_t n)
{
    const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i < n) out[i] = float_to_e4m3fn_rne(in[i]);
}

// ---------------------------------------------------------------------------------------
// host generator helpers
// ---------------------------------------------------------------------------------------
static inline uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static inline float u01(uint64_t bits) { return static_cast<float>((bits >> 40) + 1) * (1.0f / 16777217.0f); }  // (0,1)

static float host_e4m3fn_to_float(uint8_t b)
{
    const int e = (b >> 3) & 0xF, m = b & 7;
    float v;
    if (e == 0xF && m == 7) return NAN;
    if (e == 0) v = std::ldexp(static_cast<float>(m), -9);
    else v = std::ldexp(static_cast<float>(8 + m), e - 10);
    return (b & 0x80) ? -v : v;
}

constexpr int HOST_CHUNKS = 4;   // column chunks fp8bs_gemm_host pipelines (copy in, GEMM, copy out)

struct fp8bs_host_ctx_impl {
    size_t max_M, max_N, max_K;
    void *dA, *dB, *dAs, *dBs, *dC, *dW;
    void *hA, *hB, *hAs, *hBs, *hC;
    size_t w_bytes;
    cudaStream_t stream;                 // GEMM launches
    cudaStream_t s_in, s_out;            // host-to-device and device-to-host copies: one DMA engine each way
    cudaEvent_t e_a, e_b[HOST_CHUNKS], e_g[HOST_CHUNKS];
};

}  // namespace fp8bs

using namespace fp8bs;

// =======================================================================================
// exported C ABI
// =======================================================================================
extern "C" {

int fp8bs_gemm(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M, int N,
               int K, void* workspace, size_t workspace_bytes, void* stream)
{
    return gemm_impl(A, B, a_scale, b_scale, C, M, N, K, 0, N, FP8BS_PATH_AUTO, 0, 0, workspace, workspace_bytes,
                     stream);
}

int fp8bs_gemm_mn_large(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M,
                        int N, int K, void* stream)
{
    return gemm_impl(A, B, a_scale, b_scale, C, M, N, K, 0, N, FP8BS_PATH_MN_LARGE, 1, 0, nullptr, 0, stream);
}

int fp8bs_gemm_mn_small(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M,
                        int N, int K, int splits, void* workspace, size_t workspace_bytes, void* stream)
{
    return gemm_impl(A, B, a_scale, b_scale, C, M, N, K, 0, N, FP8BS_PATH_MN_SMALL, splits, 0, workspace,
                     workspace_bytes, stream);
}

int fp8bs_gemm_ex(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M, int N,
                  int K, int n0, int n_total, int path, int splits, int tile_n, void* workspace,
                  size_t workspace_bytes, void* stream)
{
    return gemm_impl(A, B, a_scale, b_scale, C, M, N, K, n0, n_total, path, splits, tile_n, workspace,
                     workspace_bytes, stream);
}

int fp8bs_gemm_scatter(const void* A, const void* B, const float* a_scale, const float* b_scale, void* const* C_dest,
                       int n_dest, int M, int N, int K, int n0, int n_total, void* stream)
{
    if (!C_dest) return FP8BS_ERR_NULL;
    return gemm_impl(A, B, a_scale, b_scale, nullptr, M, N, K, n0, n_total, FP8BS_PATH_MN_LARGE, 1, 0, nullptr, 0,
                     stream, C_dest, n_dest);
}

// Split-K GEMM for callers that must not allocate.  The scratch is the file-scope device array above: in host code
// its name is only a handle, so the real device address is fetched once per device with cudaGetSymbolAddress
// (with that device current) and handed to the kernel like any caller-provided workspace.
int fp8bs_gemm_mn_small_static(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C,
                               int M, int N, int K, int splits, void* stream)
{
    if (!A || !B || !a_scale || !b_scale || !C) return FP8BS_ERR_NULL;
    int rc = check_args(M, N, K, 0, N, FP8BS_PATH_MN_SMALL, splits, 0);
    if (rc) return rc;
    // refuse anything the built-in scratch cannot hold, before touching the device
    const Config cfg = choose_config(host_model(), M, N, K, FP8BS_PATH_MN_SMALL, splits, FP8BS_SPLIT_WORKSPACE);
    if (config_workspace(M, N, cfg) > STATIC_SCRATCH_BYTES) return FP8BS_ERR_WORKSPACE;
    DeviceInfo* dev = nullptr;
    rc = device_setup(&dev);                       // first call on a device: attribute set-up, no allocation
    if (rc) return rc;
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!dev->static_scratch) {
            void* ptr = nullptr;
            const cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr) {
                tl_last_cuda_error = static_cast<int>(e);
                (void)cudaGetLastError();
                return FP8BS_ERR_CUDA;
            }
            dev->static_scratch = ptr;
        }
    }
    // The array keeps whatever the previous call left: the tile counters must start at zero.
    CUDA_TRY(cudaMemsetAsync(dev->static_scratch, 0, COUNTER_BYTES, static_cast<cudaStream_t>(stream)));
    return gemm_impl(A, B, a_scale, b_scale, C, M, N, K, 0, N, FP8BS_PATH_MN_SMALL, splits, FP8BS_SPLIT_WORKSPACE,
                     dev->static_scratch, STATIC_SCRATCH_BYTES, stream);
}

int fp8bs_gemm_ref(const void* A, const void* B, const float* a_scale, const float* b_scale, void* C, int M, int N,
                   int K, void* stream)
{
    if (!A || !B || !a_scale || !b_scale || !C) return FP8BS_ERR_NULL;
    if (M <= 0 || N <= 0 || K <= 0 || K % 128 != 0) return FP8BS_ERR_SHAPE;
    const dim3 block(32, 8), grid(ceil_div(N, 32), ceil_div(M, 8));
    ref_gemm_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(A), static_cast<const uint8_t*>(B), a_scale, b_scale,
        static_cast<__nv_bfloat16*>(C), M, N, K);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    CUDA_TRY(cudaGetLastError());
    return FP8BS_OK;
}

int fp8bs_select_path(int M, int N, int K, int* splits, int* tile_n)
{
    const int rc = check_shape(M, N, K);
    if (rc) return rc;
    const Config c = choose_config(host_model(), M, N, K, FP8BS_PATH_AUTO, 0, 0);
    if (splits) *splits = c.splits;
    if (tile_n) *tile_n = c.tile_n | (c.cg == 2 ? FP8BS_TILE_PAIR : 0) | (c.mode == 1 ? FP8BS_SPLIT_WORKSPACE : 0) | (c.mode == 4 ? FP8BS_SHORT_K : 0) |
                          (c.mode == 3 ? FP8BS_STREAM_K : 0);
    return c.path;
}

int fp8bs_select_path_sms(int M, int N, int K, int sm_count, int* splits, int* tile_n, int* ctas)
{
    const int rc = check_shape(M, N, K);
    if (rc) return rc;
    if (sm_count < 1) return FP8BS_ERR_ARG;
    const Config c = choose_config(scaled_model(sm_count), M, N, K, FP8BS_PATH_AUTO, 0, 0);
    if (splits) *splits = c.splits;
    if (tile_n) *tile_n = c.tile_n | (c.cg == 2 ? FP8BS_TILE_PAIR : 0) | (c.mode == 1 ? FP8BS_SPLIT_WORKSPACE : 0) | (c.mode == 4 ? FP8BS_SHORT_K : 0) |
                          (c.mode == 3 ? FP8BS_STREAM_K : 0);
    if (ctas) {
        // CTAs that have to be resident together: stream-K's whole grid, one cluster for the cluster reduction,
        // otherwise none (the tile walkers never wait on one another)
        *ctas = (c.mode == 3) ? c.ctas : (c.mode == 2 ? c.splits : 0);
    }
    return c.path;
}

size_t fp8bs_workspace_bytes(int M, int N, int K)
{
    if (check_shape(M, N, K)) return 0;
    return config_workspace(M, N, choose_config(host_model(), M, N, K, FP8BS_PATH_AUTO, 0, 0));
}

size_t fp8bs_workspace_bytes_ex(int M, int N, int K, int path, int splits, int tile_n)
{
    if (check_args(M, N, K, 0, N, path, splits, tile_n)) return 0;
    return config_workspace(M, N, choose_config(host_model(), M, N, K, path, splits, tile_n));
}

int fp8bs_workspace_init(void* workspace, size_t workspace_bytes, void* stream)
{
    if (!workspace) return FP8BS_ERR_NULL;
    if (workspace_bytes < COUNTER_BYTES) return FP8BS_ERR_WORKSPACE;
    CUDA_TRY(cudaMemsetAsync(workspace, 0, COUNTER_BYTES, static_cast<cudaStream_t>(stream)));
    return FP8BS_OK;
}

int fp8bs_last_device_status(void* stream, unsigned int* detail)
{
    DeviceInfo* dev = nullptr;
    const int rc = device_setup(&dev);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // read, and if needed clear, on the caller's stream: nothing here orders or blocks other streams
    unsigned int word = 0;
    CUDA_TRY(cudaMemcpyAsync(&word, dev->status_ptr, sizeof(word), cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    if (detail) *detail = word;
    if (word != 0) {
        CUDA_TRY(cudaMemsetAsync(dev->status_ptr, 0, sizeof(word), st));
        return FP8BS_ERR_DEVICE_TIMEOUT;
    }
    return FP8BS_OK;
}

int fp8bs_selftest_wait_timeout(void* stream)
{
    DeviceInfo* dev = nullptr;
    const int rc = device_setup(&dev);
    if (rc) return rc;
    // about 20 ms at 2 GHz: long enough to be a real wait, short enough for a test
    wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(dev->status_ptr, 40000000LL);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    CUDA_TRY(cudaGetLastError());
    return FP8BS_OK;
}

const char* fp8bs_status_string(int status)
{
    switch (status) {
        case FP8BS_OK: return "ok";
        case FP8BS_ERR_NULL: return "a required pointer is NULL";
        case FP8BS_ERR_SHAPE: return "bad shape: M, N, K must be positive and K a multiple of 128";
        case FP8BS_ERR_ALIGN: return "alignment: M and N must be multiples of 16; A, B, C 16-byte aligned";
        case FP8BS_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case FP8BS_ERR_ARG: return "bad path, splits, tile_n, n0 or n_total argument";
        case FP8BS_ERR_NO_DEVICE: return "no usable sm_100 device (this library has no CPU fallback)";
        case FP8BS_ERR_CUDA: return "a CUDA call failed (see fp8bs_last_cuda_error)";
        case FP8BS_ERR_DEVICE_TIMEOUT: return "a kernel gave up waiting on a barrier";
        case FP8BS_ERR_FP8_BYTE: return "fp8 byte has no equal value in the other dialect";
        default: return "unknown status";
    }
}

#ifdef FP8BS_PROFILE
int fp8bs_debug_prof(long long* out, int n)
{
    cudaDeviceSynchronize();
    return cudaMemcpy(out, g_prof_buf, sizeof(long long) * n, cudaMemcpyDeviceToHost);
}
#endif
int fp8bs_last_cuda_error(void) { return tl_last_cuda_error; }
unsigned long long fp8bs_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

// ---- gemmGPU mirror -------------------------------------------------------------------
int fp8bs_gemmGPU(uint16_t* C, const float* A, const float* B, const float* a_scale, const float* b_scale, size_t M,
                  size_t N, size_t K, int option)
{
    if (!C || !A || !B || !a_scale || !b_scale) return FP8BS_ERR_NULL;
    if (option < 0 || option > 2) return FP8BS_ERR_ARG;
    if (M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return FP8BS_ERR_SHAPE;
    int rc = check_shape(static_cast<int>(M), static_cast<int>(N), static_cast<int>(K));
    if (rc) return rc;
    const size_t sn = (N + 127) / 128, KB = K / 128;
    float *dA = nullptr, *dB = nullptr, *dAs = nullptr, *dBs = nullptr;
    uint8_t *dA8 = nullptr, *dB8 = nullptr;
    void *dC = nullptr, *dW = nullptr;
    size_t wbytes = 0;
    auto cleanup = [&]() {
        cudaFree(dA); cudaFree(dB); cudaFree(dAs); cudaFree(dBs); cudaFree(dA8); cudaFree(dB8); cudaFree(dC); cudaFree(dW);
    };
#define GG_TRY(expr)                                                        \
    do {                                                                    \
        cudaError_t e__ = (expr);                                           \
        if (e__ != cudaSuccess) {                                           \
            tl_last_cuda_error = static_cast<int>(e__);                     \
            (void)cudaGetLastError();                                       \
            cleanup();                                                      \
            return FP8BS_ERR_CUDA;                                          \
        }                                                                   \
    } while (0)
    GG_TRY(cudaMalloc(&dA, sizeof(float) * M * K));
    GG_TRY(cudaMalloc(&dB, sizeof(float) * N * K));
    GG_TRY(cudaMalloc(&dC, sizeof(uint16_t) * M * N));
    GG_TRY(cudaMalloc(&dAs, sizeof(float) * M * KB));
    GG_TRY(cudaMalloc(&dBs, sizeof(float) * sn * KB));
    GG_TRY(cudaMemcpy(dA, A, sizeof(float) * M * K, cudaMemcpyHostToDevice));
    GG_TRY(cudaMemcpy(dB, B, sizeof(float) * N * K, cudaMemcpyHostToDevice));
    GG_TRY(cudaMemcpy(dAs, a_scale, sizeof(float) * M * KB, cudaMemcpyHostToDevice));
    GG_TRY(cudaMemcpy(dBs, b_scale, sizeof(float) * sn * KB, cudaMemcpyHostToDevice));
    GG_TRY(cudaMalloc(&dA8, M * K));
    GG_TRY(cudaMalloc(&dB8, N * K));
    convert_float_to_e4m3fn_kernel<<<static_cast<unsigned>((M * K + 255) / 256), 256>>>(dA, dA8, M * K);
    convert_float_to_e4m3fn_kernel<<<static_cast<unsigned>((N * K + 255) / 256), 256>>>(dB, dB8, N * K);
    g_launches.fetch_add(2, std::memory_order_relaxed);
    GG_TRY(cudaGetLastError());
    const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
    if (option == 2) {
        rc = fp8bs_gemm_ref(dA8, dB8, dAs, dBs, dC, m, n, k, nullptr);
    } else {
        const int path = option == 1 ? FP8BS_PATH_MN_SMALL : FP8BS_PATH_AUTO;
        wbytes = fp8bs_workspace_bytes_ex(m, n, k, path, 0, 0);
        if (wbytes) {
            GG_TRY(cudaMalloc(&dW, wbytes));
            GG_TRY(cudaMemset(dW, 0, COUNTER_BYTES));
        }
        rc = gemm_impl(dA8, dB8, dAs, dBs, dC, m, n, k, 0, n, path, 0, 0, dW, wbytes, nullptr);
    }
    if (rc == FP8BS_OK) {
        GG_TRY(cudaMemcpy(C, dC, sizeof(uint16_t) * M * N, cudaMemcpyDeviceToHost));
        rc = fp8bs_last_device_status(nullptr, nullptr);
    }
    cleanup();
#undef GG_TRY
    return rc;
}

// ---- reusable end-to-end context ------------------------------------------------------
int fp8bs_host_ctx_create(fp8bs_host_ctx** out, size_t max_M, size_t max_N, size_t max_K)
{
    if (!out) return FP8BS_ERR_NULL;
    *out = nullptr;
    if (max_M == 0 || max_N == 0 || max_K == 0 || max_K % 128 != 0) return FP8BS_ERR_SHAPE;
    DeviceInfo* dev = nullptr;
    int rc = device_setup(&dev);
    if (rc) return rc;
    fp8bs_host_ctx_impl* c = new (std::nothrow) fp8bs_host_ctx_impl();
    if (!c) return FP8BS_ERR_CUDA;
    std::memset(c, 0, sizeof(*c));
    c->max_M = max_M; c->max_N = max_N; c->max_K = max_K;
    const size_t KB = max_K / 128;
    // split-K is only ever chosen for small M*N; 64 MiB covers every such configuration
    c->w_bytes = static_cast<size_t>(64) << 20;
    bool ok = cudaMalloc(&c->dA, max_M * max_K) == cudaSuccess && cudaMalloc(&c->dB, max_N * max_K) == cudaSuccess &&
              cudaMalloc(&c->dAs, max_M * KB * 4) == cudaSuccess && cudaMalloc(&c->dBs, BSCALE_MAX_BYTES) == cudaSuccess &&
              cudaMalloc(&c->dC, max_M * max_N * 2) == cudaSuccess && cudaMalloc(&c->dW, c->w_bytes) == cudaSuccess &&
              cudaMallocHost(&c->hA, max_M * max_K) == cudaSuccess && cudaMallocHost(&c->hB, max_N * max_K) == cudaSuccess &&
              cudaMallocHost(&c->hAs, max_M * KB * 4) == cudaSuccess && cudaMallocHost(&c->hBs, BSCALE_MAX_BYTES) == cudaSuccess &&
              cudaMallocHost(&c->hC, max_M * max_N * 2) == cudaSuccess &&
              cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking) == cudaSuccess &&
              cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking) == cudaSuccess &&
              cudaEventCreateWithFlags(&c->e_a, cudaEventDisableTiming) == cudaSuccess &&
              cudaMemset(c->dW, 0, COUNTER_BYTES) == cudaSuccess;
    for (int j = 0; ok && j < HOST_CHUNKS; ++j)
        ok = cudaEventCreateWithFlags(&c->e_b[j], cudaEventDisableTiming) == cudaSuccess &&
             cudaEventCreateWithFlags(&c->e_g[j], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) {
        tl_last_cuda_error = static_cast<int>(cudaGetLastError());
        fp8bs_host_ctx_destroy(reinterpret_cast<fp8bs_host_ctx*>(c));
        return FP8BS_ERR_CUDA;
    }
    *out = reinterpret_cast<fp8bs_host_ctx*>(c);
    return FP8BS_OK;
}

int fp8bs_host_ctx_destroy(fp8bs_host_ctx* ctx)
{
    if (!ctx) return FP8BS_OK;
    fp8bs_host_ctx_impl* c = reinterpret_cast<fp8bs_host_ctx_impl*>(ctx);
    if (c->stream) cudaStreamDestroy(c->stream);
    if (c->s_in) cudaStreamDestroy(c->s_in);
    if (c->s_out) cudaStreamDestroy(c->s_out);
    if (c->e_a) cudaEventDestroy(c->e_a);
    for (int j = 0; j < HOST_CHUNKS; ++j) {
        if (c->e_b[j]) cudaEventDestroy(c->e_b[j]);
        if (c->e_g[j]) cudaEventDestroy(c->e_g[j]);
    }
    cudaFree(c->dA); cudaFree(c->dB); cudaFree(c->dAs); cudaFree(c->dBs); cudaFree(c->dC); cudaFree(c->dW);
    cudaFreeHost(c->hA); cudaFreeHost(c->hB); cudaFreeHost(c->hAs); cudaFreeHost(c->hBs); cudaFreeHost(c->hC);
    (void)cudaGetLastError();
    delete c;
    return FP8BS_OK;
}

void* fp8bs_host_ctx_buffer(fp8bs_host_ctx* ctx, int which)
{
    if (!ctx) return nullptr;
    fp8bs_host_ctx_impl* c = reinterpret_cast<fp8bs_host_ctx_impl*>(ctx);
    switch (which) {
        case 0: return c->hA;
        case 1: return c->hB;
        case 2: return c->hAs;
        case 3: return c->hBs;
        case 4: return c->hC;
        default: return nullptr;
    }
}

int fp8bs_gemm_host(fp8bs_host_ctx* ctx, uint16_t* C, const void* A, const void* B, const float* a_scale,
                    const float* b_scale, int M, int N, int K, int n0, int n_total)
{
    if (!ctx || !C || !A || !B || !a_scale || !b_scale) return FP8BS_ERR_NULL;
    fp8bs_host_ctx_impl* c = reinterpret_cast<fp8bs_host_ctx_impl*>(ctx);
    int rc = check_args(M, N, K, n0, n_total, FP8BS_PATH_AUTO, 0, 0);
    if (rc) return rc;
    if (static_cast<size_t>(M) > c->max_M || static_cast<size_t>(N) > c->max_N || static_cast<size_t>(K) > c->max_K)
        return FP8BS_ERR_SHAPE;
    const size_t KB = K / 128, sn = (static_cast<size_t>(n_total) + 127) / 128;
    if (sn * KB * 4 > BSCALE_MAX_BYTES) return FP8BS_ERR_SHAPE;
    // Pipeline over column chunks: while chunk j is multiplied, the columns of B for chunk j + 1 come in on one copy
    // engine and the columns of C of chunk j - 1 go out on the other.  A chunk is a run of whole 128-column blocks;
    // on the device its B columns ([K][Nc], contiguous) and its C ([M][Nc]) sit at the chunk's offset in dB / dC.
    const int nblk = (N + 127) / 128;
    int chunks = (static_cast<size_t>(N) * K + static_cast<size_t>(M) * N * 2 >= (static_cast<size_t>(4) << 20)) ? HOST_CHUNKS : 1;
    if (chunks > nblk / 4) chunks = nblk / 4 > 0 ? nblk / 4 : 1;      // at least 512 columns per chunk
    const uint8_t* hB = static_cast<const uint8_t*>(B);
    const size_t a_bytes = static_cast<size_t>(M) * K, b_bytes = static_cast<size_t>(N) * K, c_bytes = static_cast<size_t>(M) * N * 2;
    if (a_bytes > b_bytes + c_bytes && a_bytes >= (static_cast<size_t>(8) << 20) && M >= 4 * 256) {
        // A is the bulk of the traffic: pipeline over row chunks instead.  B and b_scale go in first; then, chunk by
        // chunk, the rows of A and a_scale (as [K][Mc] and [K/128][Mc], contiguous on the device), the GEMM on those
        // rows, and the copy-out of the finished rows of C, which are contiguous in the caller's buffer.
        const uint8_t* hA = static_cast<const uint8_t*>(A);
        const int mblk = (M + 127) / 128;
        const int mchunks = mblk / 2 < HOST_CHUNKS ? (mblk / 2 > 0 ? mblk / 2 : 1) : HOST_CHUNKS;
        CUDA_TRY(cudaMemcpyAsync(c->dB, hB, b_bytes, cudaMemcpyHostToDevice, c->s_in));
        CUDA_TRY(cudaMemcpyAsync(c->dBs, b_scale, sn * KB * 4, cudaMemcpyHostToDevice, c->s_in));
        for (int j = 0; j < mchunks; ++j) {
            const int r0 = (mblk * j / mchunks) * 128;
            int r1 = (mblk * (j + 1) / mchunks) * 128;
            if (r1 > M) r1 = M;
            const int mc = r1 - r0;
            uint8_t* dAj = static_cast<uint8_t*>(c->dA) + static_cast<size_t>(r0) * K;
            float* dAsj = static_cast<float*>(c->dAs) + static_cast<size_t>(r0) * KB;
            __nv_bfloat16* dCj = static_cast<__nv_bfloat16*>(c->dC) + static_cast<size_t>(r0) * N;
            CUDA_TRY(cudaMemcpy2DAsync(dAj, mc, hA + r0, M, mc, K, cudaMemcpyHostToDevice, c->s_in));
            CUDA_TRY(cudaMemcpy2DAsync(dAsj, static_cast<size_t>(mc) * 4, a_scale + r0, static_cast<size_t>(M) * 4,
                                       static_cast<size_t>(mc) * 4, KB, cudaMemcpyHostToDevice, c->s_in));
            CUDA_TRY(cudaEventRecord(c->e_b[j], c->s_in));
            CUDA_TRY(cudaStreamWaitEvent(c->stream, c->e_b[j], 0));
            rc = gemm_impl(dAj, c->dB, dAsj, static_cast<const float*>(c->dBs), dCj, mc, N, K, n0, n_total,
                           FP8BS_PATH_AUTO, 0, 0, c->dW, c->w_bytes, c->stream);
            if (rc) {
                (void)cudaStreamSynchronize(c->s_in);
                (void)cudaStreamSynchronize(c->stream);
                (void)cudaStreamSynchronize(c->s_out);
                return rc;
            }
            CUDA_TRY(cudaEventRecord(c->e_g[j], c->stream));
            CUDA_TRY(cudaStreamWaitEvent(c->s_out, c->e_g[j], 0));
            CUDA_TRY(cudaMemcpyAsync(C + static_cast<size_t>(r0) * N, dCj, static_cast<size_t>(mc) * N * 2,
                                     cudaMemcpyDeviceToHost, c->s_out));
        }
        CUDA_TRY(cudaStreamSynchronize(c->s_out));
        CUDA_TRY(cudaStreamSynchronize(c->stream));
        CUDA_TRY(cudaStreamSynchronize(c->s_in));
        return FP8BS_OK;
    }
    CUDA_TRY(cudaMemcpyAsync(c->dA, A, static_cast<size_t>(M) * K, cudaMemcpyHostToDevice, c->s_in));
    CUDA_TRY(cudaMemcpyAsync(c->dAs, a_scale, static_cast<size_t>(M) * KB * 4, cudaMemcpyHostToDevice, c->s_in));
    CUDA_TRY(cudaMemcpyAsync(c->dBs, b_scale, sn * KB * 4, cudaMemcpyHostToDevice, c->s_in));
    CUDA_TRY(cudaEventRecord(c->e_a, c->s_in));
    CUDA_TRY(cudaStreamWaitEvent(c->stream, c->e_a, 0));
    for (int j = 0; j < chunks; ++j) {
        const int c0 = (nblk * j / chunks) * 128;
        int c1 = (nblk * (j + 1) / chunks) * 128;
        if (c1 > N) c1 = N;
        const int nc = c1 - c0;
        uint8_t* dBj = static_cast<uint8_t*>(c->dB) + static_cast<size_t>(c0) * K;
        __nv_bfloat16* dCj = static_cast<__nv_bfloat16*>(c->dC) + static_cast<size_t>(c0) * M;
        if (chunks == 1) CUDA_TRY(cudaMemcpyAsync(dBj, hB, static_cast<size_t>(N) * K, cudaMemcpyHostToDevice, c->s_in));
        else CUDA_TRY(cudaMemcpy2DAsync(dBj, nc, hB + c0, N, nc, K, cudaMemcpyHostToDevice, c->s_in));
        CUDA_TRY(cudaEventRecord(c->e_b[j], c->s_in));
        CUDA_TRY(cudaStreamWaitEvent(c->stream, c->e_b[j], 0));
        rc = gemm_impl(c->dA, dBj, static_cast<const float*>(c->dAs), static_cast<const float*>(c->dBs), dCj, M, nc, K,
                       n0 + c0, n_total, FP8BS_PATH_AUTO, 0, 0, c->dW, c->w_bytes, c->stream);
        if (rc) {
            (void)cudaStreamSynchronize(c->s_in);
            (void)cudaStreamSynchronize(c->stream);
            (void)cudaStreamSynchronize(c->s_out);
            return rc;
        }
        CUDA_TRY(cudaEventRecord(c->e_g[j], c->stream));
        CUDA_TRY(cudaStreamWaitEvent(c->s_out, c->e_g[j], 0));
        if (chunks == 1) CUDA_TRY(cudaMemcpyAsync(C, dCj, static_cast<size_t>(M) * N * 2, cudaMemcpyDeviceToHost, c->s_out));
        else CUDA_TRY(cudaMemcpy2DAsync(C + c0, static_cast<size_t>(N) * 2, dCj, static_cast<size_t>(nc) * 2,
                                        static_cast<size_t>(nc) * 2, M, cudaMemcpyDeviceToHost, c->s_out));
    }
    CUDA_TRY(cudaStreamSynchronize(c->s_out));
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    CUDA_TRY(cudaStreamSynchronize(c->s_in));
    return FP8BS_OK;
}

// ---- e4m3fnuz -> e4m3fn on the device -----------------------------------------------------------
// One byte in, one byte out, 16 bytes per thread.  Same mapping as fp8bs_fnuz_to_fn; the eight magnitudes e4m3fn
// cannot hold (odd multiples of 2^-10 below 2^-6) are rounded to the nearest even multiple of 2^-9 and counted.
__device__ __forceinline__ uint32_t fnuz_to_fn_byte(uint32_t b, unsigned int& inexact)
{
    const uint32_t e = (b >> 3) & 0xFu, m = b & 7u, sign = b & 0x80u;
    if (b == 0x80u) return 0x7Fu;                       // NaN stays NaN
    if ((b & 0x7Fu) == 0u) return 0u;
    if (e >= 2u) return b - 8u;                         // same mantissa, exponent field one lower
    const uint32_t q = (e == 0u) ? m : 8u + m;          // value = q * 2^-10
    uint32_t h = q >> 1;                                // -> h * 2^-9
    if (q & 1u) { ++inexact; h += (h & 1u); }           // tie: round half to even
    return sign | h;                                    // h <= 8; 8 is the encoding of 2^-6
}

// Four bytes at a time, without a branch on the data (in real data one word in twenty holds a small magnitude, so a
// branch would send nearly every warp down the slow path).  Per byte, with low7 = b & 0x7F:
//   low7 >= 0x10 (exponent field >= 2): a normal number of both dialects, the byte only loses 8;
//   low7 <  0x10: the value is low7 * 2^-10, i.e. (low7 / 2) * 2^-9 rounded half to even, counted when low7 is odd;
//   0x80 (the NaN of e4m3fnuz) becomes 0x7F.
__device__ __forceinline__ uint32_t fnuz_to_fn_word(uint32_t w, unsigned int& inexact)
{
    const uint32_t low7 = w & 0x7F7F7F7Fu, sign = w & 0x80808080u;
    const uint32_t big = (low7 + 0x70707070u) & 0x80808080u;            // 0x80 in every byte with low7 >= 0x10
    if (big == 0x80808080u) return w - 0x08080808u;                      // warp-uniform for most words of real data
    const uint32_t big_ff = (big >> 7) * 0xFFu;                          // ... as a byte mask
    // setting bit 7 first keeps the borrow of a small byte out of its neighbour
    const uint32_t cand_big = (((low7 | 0x80808080u) - 0x08080808u) & 0x7F7F7F7Fu) | sign;
    uint32_t h = (low7 >> 1) & 0x7F7F7F7Fu;                             // per byte: low7 / 2
    const uint32_t odd = low7 & 0x01010101u;
    h += odd & h;                                                        // tie: round half to even (h <= 7, no carry)
    const uint32_t cand_small = sign | h;
    inexact += __popc(odd & ~(big >> 7));
    uint32_t r = (cand_big & big_ff) | (cand_small & ~big_ff);
    const uint32_t zero7 = ~(low7 + 0x7F7F7F7Fu) & 0x80808080u;         // 0x80 in every byte with low7 == 0
    const uint32_t nan_ff = ((zero7 & sign) >> 7) * 0xFFu;              // bytes equal to 0x80
    return (r & ~nan_ff) | (0x7F7F7F7Fu & nan_ff);
}

__global__ void __launch_bounds__(256)
fnuz_to_fn_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n16,
                  const uint8_t* __restrict__ src_tail, uint8_t* __restrict__ dst_tail, int tail,
                  unsigned int* __restrict__ inexact_count)
{
    unsigned int inexact = 0;
    const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
    size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    // two independent 16-byte loads in flight per thread and round
    for (; i + stride < n16; i += 2 * stride) {
        const uint4 a = __ldcs(src + i), b = __ldcs(src + i + stride);
        dst[i] = make_uint4(fnuz_to_fn_word(a.x, inexact), fnuz_to_fn_word(a.y, inexact), fnuz_to_fn_word(a.z, inexact),
                            fnuz_to_fn_word(a.w, inexact));
        dst[i + stride] = make_uint4(fnuz_to_fn_word(b.x, inexact), fnuz_to_fn_word(b.y, inexact),
                                     fnuz_to_fn_word(b.z, inexact), fnuz_to_fn_word(b.w, inexact));
    }
    if (i < n16) {
        const uint4 a = __ldcs(src + i);
        dst[i] = make_uint4(fnuz_to_fn_word(a.x, inexact), fnuz_to_fn_word(a.y, inexact), fnuz_to_fn_word(a.z, inexact),
                            fnuz_to_fn_word(a.w, inexact));
    }
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < tail)
        dst_tail[threadIdx.x] = static_cast<uint8_t>(fnuz_to_fn_byte(src_tail[threadIdx.x], inexact));
    if (inexact && inexact_count) atomicAdd(inexact_count, inexact);
}

int fp8bs_fnuz_to_fn_device(void* dst, const void* src, size_t n, unsigned int* inexact_count, void* stream)
{
    if (!dst || !src) return FP8BS_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15u) return FP8BS_ERR_ALIGN;
    DeviceInfo* dev = nullptr;
    const int rc = device_setup(&dev);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (inexact_count) CUDA_TRY(cudaMemsetAsync(inexact_count, 0, sizeof(unsigned int), st));
    const size_t n16 = n / 16;
    const int tail = static_cast<int>(n % 16);
    size_t blocks = (n16 + 255) / 256;
    const size_t cap = static_cast<size_t>(dev->sm_count) * 8;      // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    fnuz_to_fn_kernel<<<static_cast<unsigned>(blocks), 256, 0, st>>>(
        static_cast<const uint4*>(src), static_cast<uint4*>(dst), n16, static_cast<const uint8_t*>(src) + n16 * 16,
        static_cast<uint8_t*>(dst) + n16 * 16, tail, inexact_count);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    CUDA_TRY(cudaGetLastError());
    return FP8BS_OK;
}

// ---- device-side quantisers (quantize.py) ------------------------------------------------------
static int quantize_impl(bool block, const void* X, int x_is_bf16, void* out, float* scale_out, int rows, int K,
                         float fp8_max, void* stream)
{
    if (!X || !out || !scale_out) return FP8BS_ERR_NULL;
    if (rows <= 0 || K <= 0 || K % 128 != 0) return FP8BS_ERR_SHAPE;
    if (rows % 16 != 0) return FP8BS_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(out)) & 15u) return FP8BS_ERR_ALIGN;
    if (!(fp8_max > 0.0f) || fp8_max > 448.0f) return FP8BS_ERR_ARG;
    DeviceInfo* dev = nullptr;
    const int rc = device_setup(&dev);
    if (rc) return rc;
    const dim3 grid(ceil_div(rows, 128), K / 128), blk(256);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* o = static_cast<uint8_t*>(out);
    if (x_is_bf16) {
        const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);
        if (block) quantize_kernel<true, __nv_bfloat16><<<grid, blk, 0, st>>>(x, o, scale_out, rows, K, fp8_max);
        else quantize_kernel<false, __nv_bfloat16><<<grid, blk, 0, st>>>(x, o, scale_out, rows, K, fp8_max);
    } else {
        const float* x = static_cast<const float*>(X);
        if (block) quantize_kernel<true, float><<<grid, blk, 0, st>>>(x, o, scale_out, rows, K, fp8_max);
        else quantize_kernel<false, float><<<grid, blk, 0, st>>>(x, o, scale_out, rows, K, fp8_max);
    }
    g_launches.fetch_add(1, std::memory_order_relaxed);
    CUDA_TRY(cudaGetLastError());
    return FP8BS_OK;
}

int fp8bs_quantize_rowwise(const void* X, int x_is_bf16, void* A_out, float* a_scale_out, int M, int K, float fp8_max,
                           void* stream)
{
    return quantize_impl(false, X, x_is_bf16, A_out, a_scale_out, M, K, fp8_max, stream);
}

int fp8bs_quantize_block(const void* W, int w_is_bf16, void* B_out, float* b_scale_out, int N, int K, float fp8_max,
                         void* stream)
{
    return quantize_impl(true, W, w_is_bf16, B_out, b_scale_out, N, K, fp8_max, stream);
}

// ---- generators / conversions (host only) -------------------------------------------------
uint8_t fp8bs_float_to_e4m3fn(float x) { return float_to_e4m3fn_rne(x); }
float fp8bs_e4m3fn_to_float(uint8_t b) { return host_e4m3fn_to_float(b); }

int fp8bs_gen_normal_e4m3(uint8_t* out, size_t n, uint64_t seed)
{
    if (!out) return FP8BS_ERR_NULL;
    const uint64_t key = mix64(seed ^ 0xA5A5A5A5DEADBEEFull);
    for (size_t i = 0; i < n; i += 2) {
        // Box-Muller on two counter-based uniforms; element i and i+1 share one pair
        const float u1 = u01(mix64(key + 2 * (i / 2))), u2 = u01(mix64(key + 2 * (i / 2) + 1));
        const float r = std::sqrt(-2.0f * std::log(u1)), t = 6.28318530717958647692f * u2;
        const float z[2] = {r * std::cos(t), r * std::sin(t)};
        for (size_t j = 0; j < 2 && i + j < n; ++j) {
            float v = z[j];
            if (v > 240.0f) v = 240.0f;
            if (v < -240.0f) v = -240.0f;
            uint8_t b = float_to_e4m3fn_rne(v);
            if ((b & 0x7F) < 0x08) b = 0;     // |x| < 2^-6 (all e4m3fn subnormals) -> +0
            out[i + j] = b;
        }
    }
    return FP8BS_OK;
}

int fp8bs_gen_uniform_f32(float* out, size_t n, uint64_t seed, float lo, float hi)
{
    if (!out) return FP8BS_ERR_NULL;
    const uint64_t key = mix64(seed ^ 0x5C5C5C5C12345678ull);
    for (size_t i = 0; i < n; ++i) {
        const float u = static_cast<float>(mix64(key + i) >> 40) * (1.0f / 16777216.0f);   // [0,1)
        float v = lo + (hi - lo) * u;
        if (v >= hi) v = lo;
        out[i] = v;
    }
    return FP8BS_OK;
}

int fp8bs_fnuz_to_fn(uint8_t* dst, const uint8_t* src, size_t n, size_t* bad_index)
{
    if (!dst || !src) return FP8BS_ERR_NULL;
    for (size_t i = 0; i < n; ++i) {
        const uint8_t b = src[i];
        const int e = (b >> 3) & 0xF, m = b & 7;
        uint8_t o;
        if (b == 0x80) { if (bad_index) *bad_index = i; return FP8BS_ERR_FP8_BYTE; }   // NaN
        if ((b & 0x7F) == 0) o = 0;
        else if (e >= 2) o = static_cast<uint8_t>(b - 8);         // same mantissa, exponent field one lower
        else {
            // value = q * 2^-10 with q = m (e == 0) or 8 + m (e == 1); e4m3fn holds q/2 * 2^-9
            const int q = (e == 0) ? m : 8 + m;
            if (q & 1) { if (bad_index) *bad_index = i; return FP8BS_ERR_FP8_BYTE; }
            o = static_cast<uint8_t>((b & 0x80) | (q / 2));       // q/2 in 1..7: an e4m3fn subnormal
        }
        dst[i] = o;
    }
    return FP8BS_OK;
}

}  // extern "C"

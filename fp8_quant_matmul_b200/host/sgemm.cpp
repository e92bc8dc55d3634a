// sgemm -- benchmark harness (role of the reference's sgemm.cu:193-245 and its timing loops,
// sgemm.cu:96-131).  For every shape it reports
//   * "event" timing as the reference does it: 10 launches, each between two events, the first
//     dropped, mean of the other 9 (but over the WHOLE grid: the reference's loop halves it, sgemm.cu:106);
//   * "graph" timing: a CUDA graph of back-to-back launches rotating over enough buffer sets to
//     exceed twice the L2, so every launch reads its operands from HBM; min and median per launch;
// with TFLOP/s, % of the nominal dense FP8 peak (4500 TFLOP/s), GB/s of algorithmic bytes and % of 8 TB/s.
//
//   sgemm [--shape M,N,K | --sweep] [--path auto|large|small] [--splits S] [--tile 128|256] [--json FILE]
#include "harness.h"

#include <algorithm>
#include <memory>

static double algorithmic_bytes(const Shape& s)
{
    const double KB = s.K / 128, sn = (s.N + 127) / 128;
    return 1.0 * s.M * s.K + 1.0 * s.N * s.K + 4.0 * s.M * KB + 4.0 * sn * KB + 2.0 * s.M * s.N;
}

int main(int argc, char** argv)
{
    std::vector<Shape> shapes = {{1024, 7168, 2304}};   // the reference's active shape (sgemm.cu:223)
    int path = FP8BS_PATH_AUTO, splits = 0, tile = 0;
    const char* json_path = nullptr;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        Shape s;
        if (a == "--shape" && i + 1 < argc && parse_shape(argv[i + 1], &s)) { shapes = {s}; ++i; }
        else if (a == "--sweep") shapes = sweep_shapes();
        else if (a == "--path" && i + 1 < argc) {
            const std::string p = argv[++i];
            path = p == "large" ? FP8BS_PATH_MN_LARGE : p == "small" ? FP8BS_PATH_MN_SMALL : FP8BS_PATH_AUTO;
        }
        else if (a == "--splits" && i + 1 < argc) splits = std::atoi(argv[++i]);
        else if (a == "--tile" && i + 1 < argc) tile = std::atoi(argv[++i]);
        else if (a == "--json" && i + 1 < argc) json_path = argv[++i];
        else { std::fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
    }
    FILE* jf = json_path ? std::fopen(json_path, "w") : nullptr;
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
    cudaEvent_t e0, e1;
    CUDA_OK(cudaEventCreate(&e0));
    CUDA_OK(cudaEventCreate(&e1));
    std::printf("%6s %6s %6s %-9s %2s %4s | %9s | %9s %9s | %8s %7s %8s %6s\n", "M", "N", "K", "path", "S", "tile",
                "event us", "graph min", "graph med", "TFLOP/s", "%FP8", "GB/s", "%HBM");
    double log_sum = 0;
    for (size_t si = 0; si < shapes.size(); ++si) {
        const Shape s = shapes[si];
        HostProblem hp(s, 7 + 100 * si);
        const double bytes = algorithmic_bytes(s), flops = 2.0 * s.M * s.N * s.K;
        const int nsets = std::max(3, std::min(24, static_cast<int>((2.0 * 126 * 1048576 + 8e6) / bytes) + 1));
        std::vector<std::unique_ptr<DeviceProblem>> sets;
        for (int i = 0; i < nsets; ++i) sets.emplace_back(new DeviceProblem(hp));
        void* ws = nullptr;
        const size_t wbytes = fp8bs_workspace_bytes_ex(s.M, s.N, s.K, path, splits, tile);
        if (wbytes) {
            CUDA_OK(cudaMalloc(&ws, wbytes));
            FP8BS_CHECK(fp8bs_workspace_init(ws, wbytes, stream));
        }
        auto launch = [&](DeviceProblem& d) {
            FP8BS_CHECK(fp8bs_gemm_ex(d.A, d.B, d.As, d.Bs, d.C, s.M, s.N, s.K, 0, s.N, path, splits, tile, ws, wbytes, stream));
        };
        // reference-style loop (sgemm.cu:96-126)
        float total = 0;
        for (int i = 0; i < 10; ++i) {
            CUDA_OK(cudaEventRecord(e0, stream));
            launch(*sets[i % nsets]);
            CUDA_OK(cudaEventRecord(e1, stream));
            CUDA_OK(cudaEventSynchronize(e1));
            float ms = 0;
            CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
            if (i > 0) total += ms;
        }
        const double event_us = 1000.0 * total / 9.0;
        // graph of nsets back-to-back launches
        cudaGraph_t graph;
        cudaGraphExec_t exec;
        CUDA_OK(cudaStreamBeginCapture(stream, cudaStreamCaptureModeThreadLocal));
        for (int i = 0; i < nsets; ++i) launch(*sets[i]);
        CUDA_OK(cudaStreamEndCapture(stream, &graph));
        CUDA_OK(cudaGraphInstantiate(&exec, graph, 0));
        std::vector<double> per;
        for (int rep = 0; rep < 23; ++rep) {
            CUDA_OK(cudaEventRecord(e0, stream));
            CUDA_OK(cudaGraphLaunch(exec, stream));
            CUDA_OK(cudaEventRecord(e1, stream));
            CUDA_OK(cudaEventSynchronize(e1));
            float ms = 0;
            CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
            if (rep >= 3) per.push_back(1000.0 * ms / nsets);
        }
        FP8BS_CHECK(fp8bs_last_device_status(stream, nullptr));
        std::sort(per.begin(), per.end());
        const double tmin = per.front(), tmed = per[per.size() / 2];
        int sp = splits, tn = tile, chosen = path;
        if (path == FP8BS_PATH_AUTO) chosen = fp8bs_select_path(s.M, s.N, s.K, &sp, &tn);
        const double tf = flops / tmed / 1e6, gbs = bytes / tmed / 1e3;
        std::printf("%6d %6d %6d %-9s %2d %4d | %9.2f | %9.2f %9.2f | %8.1f %6.1f%% %8.1f %5.1f%%\n", s.M, s.N, s.K,
                    chosen == FP8BS_PATH_MN_SMALL ? "mn_small" : "mn_large", sp, tn, event_us, tmin, tmed, tf,
                    tf / 4500.0 * 100, gbs, gbs / 8000.0 * 100);
        if (jf)
            std::fprintf(jf, "{\"M\": %d, \"N\": %d, \"K\": %d, \"path\": \"%s\", \"splits\": %d, \"tile_n\": %d, "
                             "\"event_us\": %.3f, \"graph_min_us\": %.3f, \"graph_median_us\": %.3f, \"tflops\": %.1f, "
                             "\"GBps\": %.1f, \"buffer_sets\": %d}\n",
                         s.M, s.N, s.K, chosen == FP8BS_PATH_MN_SMALL ? "mn_small" : "mn_large", sp, tn, event_us, tmin,
                         tmed, tf, gbs, nsets);
        log_sum += std::log(tmed);
        CUDA_OK(cudaGraphExecDestroy(exec));
        CUDA_OK(cudaGraphDestroy(graph));
        cudaFree(ws);
    }
    std::printf("geomean of graph-median latency over %zu shape(s): %.2f us\n", shapes.size(),
                std::exp(log_sum / shapes.size()));
    if (jf) std::fclose(jf);
    return 0;
}

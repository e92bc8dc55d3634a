// check -- correctness harness (role of the reference's check.cu:132-184): seeded inputs, the
// ground-truth kernel (fp8bs_gemm_ref, the reference's option 2) and the optimised kernel on the
// same device buffers, then a tolerance comparison.  Unlike the reference it returns a non-zero
// exit code on a mismatch and takes the shape and kernel choice from the command line.
//
//   check [--shape M,N,K | --sweep] [--path auto|large|small] [--splits S] [--tile 128|256]
//         [--seed S] [--ref-style]      (--ref-style: scales from U(-5,5) as check.cu:161-162)
#include "harness.h"

int main(int argc, char** argv)
{
    std::vector<Shape> shapes = {{128, 128, 256}};      // the reference's active shape (check.cu:137-139)
    int path = FP8BS_PATH_AUTO, splits = 0, tile = 0;
    uint64_t seed = 7;                                  // the reference's seed (utils.h:26)
    bool ref_style = false;
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
        else if (a == "--seed" && i + 1 < argc) seed = std::strtoull(argv[++i], nullptr, 10);
        else if (a == "--ref-style") ref_style = true;
        else { std::fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
    }
    size_t total_bad = 0;
    for (size_t si = 0; si < shapes.size(); ++si) {
        const Shape s = shapes[si];
        HostProblem hp(s, seed + 100 * si, ref_style ? -5.0f : 0.01f, ref_style ? 5.0f : 1.0f);
        DeviceProblem dp(hp);
        const size_t cn = static_cast<size_t>(s.M) * s.N;
        std::vector<uint16_t> c_ref(cn), c_my(cn);
        CUDA_OK(cudaMemset(dp.C, 0xFF, cn * 2));         // NaN canary
        FP8BS_CHECK(fp8bs_gemm_ref(dp.A, dp.B, dp.As, dp.Bs, dp.C, s.M, s.N, s.K, nullptr));
        CUDA_OK(cudaMemcpy(c_ref.data(), dp.C, cn * 2, cudaMemcpyDeviceToHost));
        void* ws = nullptr;
        const size_t wbytes = fp8bs_workspace_bytes_ex(s.M, s.N, s.K, path, splits, tile);
        if (wbytes) {
            CUDA_OK(cudaMalloc(&ws, wbytes));
            FP8BS_CHECK(fp8bs_workspace_init(ws, wbytes, nullptr));
        }
        CUDA_OK(cudaMemset(dp.C, 0xFF, cn * 2));
        FP8BS_CHECK(fp8bs_gemm_ex(dp.A, dp.B, dp.As, dp.Bs, dp.C, s.M, s.N, s.K, 0, s.N, path, splits, tile, ws, wbytes, nullptr));
        FP8BS_CHECK(fp8bs_last_device_status(nullptr, nullptr));
        CUDA_OK(cudaMemcpy(c_my.data(), dp.C, cn * 2, cudaMemcpyDeviceToHost));
        cudaFree(ws);
        const size_t bad = all_close(c_ref, c_my, 2e-2f, 1e-3f);
        int sp = 0, tn = 0;
        const int chosen = fp8bs_select_path(s.M, s.N, s.K, &sp, &tn);
        std::printf("M=%d N=%d K=%d (auto would pick %s, splits %d, tile %d): %s", s.M, s.N, s.K,
                    chosen == FP8BS_PATH_MN_SMALL ? "mn_small" : "mn_large", sp, tn,
                    bad ? "MISMATCH" : "2 matrices are equal\n");
        if (bad) std::printf(" (%zu of %zu elements)\n", bad, cn);
        total_bad += bad;
    }
    return total_bad ? 1 : 0;
}

// Harness around the REFERENCE's own device code for the library pipeline (variant E).
// TEST INFRASTRUCTURE ONLY.  Compiled by oracle/Makefile from the reference sources where they
// lie (nothing is copied): the truncation / zero-padding copy kernels defined in
//   fusion_variants/1D_E_baseline/fused.cu:13-63   and   fusion_variants/2D_E_baseline/fused_trunc_2D.cu:13-71
// and the hand-written cgemm kernel of fusion_variants/1D_E_baseline/cgemm.cuh, launched with the
// grid / block / shared-memory sizes the reference drivers use, around cuFFT calls in the
// reference's order.  Arithmetic follows FNO semantics by default (alpha = 1, beta = 0,
// CUFFT_INVERSE, 1/len scale) so that the result is comparable with the oracle; the reference's
// main() is compiled too (renamed) but never called.
//
// Usage:  ref_harness_{1d,2d} <x.bin> <w.bin> <y.bin> <bs> <dimX|DX> <DY> <N> <K> [cublas] [as-shipped]
//   x.bin: complex64, reference layout [K][bs*dimX][DY] or [K][bs][DX][DY];  w.bin: [N][K];
//   y.bin (written): [N][...] like x.  With "cublas" the GEMM is cublasCgemm as in variant E,
//   otherwise the reference's cgemm kernel.  With "as-shipped" the arithmetic is the one the
//   reference drivers run (fusion_variants/1D_E_baseline/fused.cu:116,186-190): alpha = (1,-1),
//   beta = (-1,1) applied once to a zeroed C, second transform CUFFT_FORWARD, no scaling.
#define main tfno_reference_main_unused
#if HARNESS_RANK == 1
#include "fusion_variants/1D_E_baseline/fused.cu"
#else
#include "fusion_variants/2D_E_baseline/fused_trunc_2D.cu"
#endif
#undef main
#include "fusion_variants/1D_E_baseline/cgemm.cuh"

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

static bool read_file(const char* path, void* dst, size_t bytes) {
    FILE* f = fopen(path, "rb");
    if (!f) return false;
    size_t n = fread(dst, 1, bytes, f);
    fclose(f);
    return n == bytes;
}

#define REQUIRE(cond, msg) do { if (!(cond)) { fprintf(stderr, "ref_harness: %s\n", msg); return 1; } } while (0)

int main(int argc, char** argv) {
    REQUIRE(argc >= 9, "usage: <x.bin> <w.bin> <y.bin> <bs> <dimX|DX> <DY> <N> <K> [cublas] [as-shipped]");
    const long long bs = atoll(argv[4]);
    const int d1 = atoi(argv[5]), DY = atoi(argv[6]), N = atoi(argv[7]), K = atoi(argv[8]);
    bool use_cublas = false, as_shipped = false;
    for (int a = 9; a < argc; ++a) {
        if (!strcmp(argv[a], "cublas")) use_cublas = true;
        else if (!strcmp(argv[a], "as-shipped")) as_shipped = true;
    }
#if HARNESS_RANK == 1
    const long long rows = bs * d1, unit = DY;          // signals per channel, elements per signal
    const long long M = rows * 64;
#else
    const int DX = d1;
    const long long rows = bs, unit = (long long)DX * DY;
    const long long M = bs * 64 * 64;
#endif
    const size_t xin = (size_t)(K * rows * unit), yout = (size_t)(N * rows * unit);
    std::vector<float2> hx(xin), hw((size_t)K * N), hy(yout);
    REQUIRE(read_file(argv[1], hx.data(), xin * sizeof(float2)), "cannot read x");
    REQUIRE(read_file(argv[2], hw.data(), hw.size() * sizeof(float2)), "cannot read w");
    float2 *dx, *dF, *dA, *dB, *dC, *dY2;
    REQUIRE(cudaMalloc(&dx, xin * 8) == cudaSuccess && cudaMalloc(&dF, xin * 8) == cudaSuccess &&
            cudaMalloc(&dA, (size_t)M * K * 8) == cudaSuccess && cudaMalloc(&dB, hw.size() * 8) == cudaSuccess &&
            cudaMalloc(&dC, (size_t)M * N * 8) == cudaSuccess && cudaMalloc(&dY2, yout * 8) == cudaSuccess, "cudaMalloc");
    cudaMemcpy(dx, hx.data(), xin * 8, cudaMemcpyHostToDevice);
    cudaMemcpy(dB, hw.data(), hw.size() * 8, cudaMemcpyHostToDevice);
    cudaMemset(dC, 0, (size_t)M * N * 8);

    cufftHandle plan, iplan;
#if HARNESS_RANK == 1
    REQUIRE(cufftPlan1d(&plan, DY, CUFFT_C2C, (int)(K * rows)) == CUFFT_SUCCESS, "cufftPlan1d");
    REQUIRE(cufftPlan1d(&iplan, DY, CUFFT_C2C, (int)(N * rows)) == CUFFT_SUCCESS, "cufftPlan1d");
#else
    int n2[2] = {DX, DY};
    REQUIRE(cufftPlanMany(&plan, 2, n2, nullptr, 1, DX * DY, nullptr, 1, DX * DY, CUFFT_C2C, (int)(K * rows)) == CUFFT_SUCCESS, "cufftPlanMany");
    REQUIRE(cufftPlanMany(&iplan, 2, n2, nullptr, 1, DX * DY, nullptr, 1, DX * DY, CUFFT_C2C, (int)(N * rows)) == CUFFT_SUCCESS, "cufftPlanMany");
#endif
    REQUIRE(cufftExecC2C(plan, (cufftComplex*)dx, (cufftComplex*)dF, CUFFT_FORWARD) == CUFFT_SUCCESS, "cufft forward");

    // copy-kernel launch shapes as in the reference drivers
#if HARNESS_RANK == 1
    const long long FFT_bs = K * rows, iFFT_bs = N * rows;
    dim3 blockDim_copy(THREADBLOCK_M / 2, 32, 1);                                   // fused.cu:166
    dim3 gridDim_copy((THREADBLOCK_M / 2 + blockDim_copy.x - 1) / blockDim_copy.x, (unsigned)((FFT_bs + blockDim_copy.y - 1) / blockDim_copy.y));
    gridDim_copy.y = gridDim_copy.y > 2048 ? 2048 : gridDim_copy.y;
    direct_copy_colmajor_float4_truncation<<<gridDim_copy, blockDim_copy>>>(dF, dA, DY, (int)FFT_bs, THREADBLOCK_M);
#else
    const long long FFT_bs = bs * 64 * K;
    dim3 blockDim_copy(32, 32, 1);                                                  // fused_trunc_2D.cu:182
    dim3 gridDim_copy(1, (unsigned)((FFT_bs + 31) / 32));
    gridDim_copy.y = gridDim_copy.y > 2048 ? 2048 : gridDim_copy.y;
    direct_copy_colmajor_float4_truncation_2d<<<gridDim_copy, blockDim_copy>>>(dF, dA, DY, DX, (int)(bs * K), 64, 64);
#endif
    REQUIRE(cudaDeviceSynchronize() == cudaSuccess, "truncation kernel");

    float2 alpha = {1.f, 0.f}, beta = {0.f, 0.f};
    if (as_shipped) { alpha = {1.f, -1.f}; beta = {-1.f, 1.f}; }
    if (use_cublas) {
        cublasHandle_t handle;
        REQUIRE(cublasCreate(&handle) == CUBLAS_STATUS_SUCCESS, "cublasCreate");
        REQUIRE(cublasCgemm(handle, CUBLAS_OP_N, CUBLAS_OP_N, (int)M, N, K, (cuFloatComplex*)&alpha, (cuFloatComplex*)dA, (int)M,
                            (cuFloatComplex*)dB, K, (cuFloatComplex*)&beta, (cuFloatComplex*)dC, (int)M) == CUBLAS_STATUS_SUCCESS, "cublasCgemm");
        cublasDestroy(handle);
    } else {
        dim3 grid((unsigned)((M + THREADBLOCK_M - 1) / THREADBLOCK_M), (N + THREADBLOCK_N - 1) / THREADBLOCK_N, 1);   // 1D_A fused.cu:182-184
        dim3 block(THREADBLOCK_M * THREADBLOCK_N / (THREAD_M * THREAD_N), 1, 1);
        int shmem = sizeof(float2) * (THREADBLOCK_M + THREADBLOCK_N) * THREADBLOCK_K * 2;
        cgemm<<<grid, block, shmem>>>((int)M, N, K, dA, dB, dC, alpha, beta);
    }
    REQUIRE(cudaDeviceSynchronize() == cudaSuccess, "gemm");

#if HARNESS_RANK == 1
    dim3 gridDim_copy2(gridDim_copy.x, (unsigned)((iFFT_bs + blockDim_copy.y - 1) / blockDim_copy.y));
    gridDim_copy2.y = gridDim_copy2.y > 2048 ? 2048 : gridDim_copy2.y;
    direct_copy_colmajor_float4_zero_padding<<<gridDim_copy2, blockDim_copy>>>(dC, dY2, DY, (int)iFFT_bs, THREADBLOCK_M);
#else
    dim3 gridDim_copy2(1, (unsigned)((bs * 64 * N + 31) / 32));
    gridDim_copy2.y = gridDim_copy2.y > 2048 ? 2048 : gridDim_copy2.y;
    direct_copy_colmajor_float4_zero_padding_2d<<<gridDim_copy2, blockDim_copy>>>(dC, dY2, DY, DX, (int)(bs * N), 64, 64);
#endif
    REQUIRE(cudaDeviceSynchronize() == cudaSuccess, "zero-padding kernel");
    REQUIRE(cufftExecC2C(iplan, (cufftComplex*)dY2, (cufftComplex*)dY2, as_shipped ? CUFFT_FORWARD : CUFFT_INVERSE) == CUFFT_SUCCESS, "second cufft");
    REQUIRE(cudaMemcpy(hy.data(), dY2, yout * 8, cudaMemcpyDeviceToHost) == cudaSuccess, "copy back");
    const float s = as_shipped ? 1.0f : 1.0f / (float)unit;
    for (auto& v : hy) { v.x *= s; v.y *= s; }
    FILE* f = fopen(argv[3], "wb");
    REQUIRE(f, "cannot write y");
    fwrite(hy.data(), sizeof(float2), hy.size(), f);
    fclose(f);
    return 0;
}

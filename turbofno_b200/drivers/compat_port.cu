// A driver written against the reference's kernel tables, ported by the two edits the integration
// notes describe: `#include "TurboFNO.h"` from this repository instead of the reference's
// utils/TurboFNO.h + generated FFT headers, and every `table[i]<<<grid, block, smem>>>(args)`
// launch turned into the plain call `table[i](args)`.
//
// It runs the launch sequences of the reference drivers on one small problem and writes the
// results to a file that the test-suite compares with the CPU oracle:
//   variant D  fused_fft_cgemm_ifft[log2(DY)-7](M, N, K, in, B, C, out, alpha, beta)
//              (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:15-16,126)
//   variant A  fft_stride_DY[i](in, A, threadblock_bs, signals) ; cgemm(M, N, K, A, B, C, alpha, beta) ;
//              ifft_stride_DY[i](C, out, threadblock_bs, signals)
//              (fusion_variants/1D_A_exp_fft+cgemm+ifft/fused.cu:195-203)
//   variant B  fused_fft_cgemm[i](M, N, K, in, B, C, alpha, beta) ; ifft_stride_DY[i](...)
//              (fusion_variants/1D_B_exp_fused_fft_cgemm+ifft/fused.cu:141-144)
//   variant C  fft_stride_DY[i](...) ; fused_cgemm_ifft[i](M, N, K, A, B, C, out, alpha, beta)
//              (fusion_variants/1D_C_exp_fft+fused_cgemm_ifft/fused.cu:139-147)
//
// usage: compat_port <in.bin> <out.bin>
//   in.bin : int32 bs, dimX, DY, N, K, then x [K][bs*dimX][DY] and w [N][K] as complex64
//   out.bin: four results [N][bs*dimX][DY] complex64 (variants D, A, B, C), unnormalised inverse
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "TurboFNO.h"

using DataT = float2;

int main(int argc, char** argv) {
    if (argc != 3) { fprintf(stderr, "usage: %s <in.bin> <out.bin>\n", argv[0]); return 2; }
    FILE* f = fopen(argv[1], "rb");
    if (!f) { fprintf(stderr, "cannot open %s\n", argv[1]); return 2; }
    int hdr[5];
    if (fread(hdr, sizeof(int), 5, f) != 5) return 2;
    const int bs = hdr[0], dimX = hdr[1], DY = hdr[2], N = hdr[3], K = hdr[4];
    const long long rows = (long long)bs * dimX;
    const int M = (int)(rows * THREADBLOCK_M);              // the reference's M = bs * dimX * 64
    const size_t in_elems = (size_t)K * rows * DY, out_elems = (size_t)N * rows * DY;
    std::vector<DataT> hx(in_elems), hw((size_t)K * N), hy(out_elems);
    if (fread(hx.data(), sizeof(DataT), in_elems, f) != in_elems || fread(hw.data(), sizeof(DataT), hw.size(), f) != hw.size()) return 2;
    fclose(f);

    DataT *FFT_input, *dB, *dA, *dC, *FFT_output;
    cudaMalloc(&FFT_input, sizeof(DataT) * in_elems);
    cudaMalloc(&dB, sizeof(DataT) * hw.size());
    cudaMalloc(&dA, sizeof(DataT) * (size_t)M * K);
    cudaMalloc(&dC, sizeof(DataT) * (size_t)M * N);
    cudaMalloc(&FFT_output, sizeof(DataT) * out_elems);
    cudaMemcpy(FFT_input, hx.data(), sizeof(DataT) * in_elems, cudaMemcpyHostToDevice);
    cudaMemcpy(dB, hw.data(), sizeof(DataT) * hw.size(), cudaMemcpyHostToDevice);
    const DataT alpha = {1.0f, 0.0f}, beta = {0.0f, 0.0f};
    int i = 0;
    while ((128 << i) < DY) ++i;                            // table slot log2(DY) - 7

    FILE* out = fopen(argv[2], "wb");
    if (!out) return 2;
    auto emit = [&](const char* what) {
        if (cudaDeviceSynchronize() != cudaSuccess || turbofno_compat::last_status() != TFNO_OK) {
            fprintf(stderr, "%s failed: %s\n", what, tfno_status_string(turbofno_compat::last_status()));
            exit(1);
        }
        cudaMemcpy(hy.data(), FFT_output, sizeof(DataT) * out_elems, cudaMemcpyDeviceToHost);
        fwrite(hy.data(), sizeof(DataT), out_elems, out);
        cudaMemset(FFT_output, 0xFF, sizeof(DataT) * out_elems);   // NaN pattern: the next variant must overwrite everything
    };

    // variant D: one table call
    fused_fft_cgemm_ifft[i](M, N, K, FFT_input, dB, dC, FFT_output, alpha, beta);
    emit("fused_fft_cgemm_ifft");

    // variant A: three table calls
    fft_stride_DY[i](FFT_input, dA, threadblock_bs, (int)(dimX * K * bs));
    cgemm(M, N, K, dA, dB, dC, alpha, beta);
    ifft_stride_DY[i](dC, FFT_output, threadblock_bs, (int)(dimX * N * bs));
    emit("fft_stride_DY + cgemm + ifft_stride_DY");

    // variant B
    fused_fft_cgemm[i](M, N, K, FFT_input, dB, dC, alpha, beta);
    ifft_stride_DY[i](dC, FFT_output, threadblock_bs, (int)(dimX * N * bs));
    emit("fused_fft_cgemm + ifft_stride_DY");

    // variant C
    fft_stride_DY[i](FFT_input, dA, threadblock_bs, (int)(dimX * K * bs));
    fused_cgemm_ifft[i](M, N, K, dA, dB, dC, FFT_output, alpha, beta);
    emit("fft_stride_DY + fused_cgemm_ifft");

    fclose(out);
    printf("compat_port: bs=%d dimX=%d DY=%d N=%d K=%d ntest=%d\n", bs, dimX, DY, N, K, ntest);
    return 0;
}

/* TurboFNO.h -- source-compatibility header for drivers written against the reference's
 * utils/TurboFNO.h and its kernel tables.
 *
 * Two things made up the reference's "header API":
 *   1. the tile / tuning macros of utils/TurboFNO.h:2-20 (README.md:205-215 documents them as
 *      the tuning surface).  They are kept here under the same names because drivers size their
 *      problems with them (M = bs * dimX * THREADBLOCK_M, fused.cu:104).  The B200 kernels do not
 *      read them: their tiling is fixed inside the library.
 *   2. the per-length kernel tables indexed by log2(DY) - 7, launched as
 *      table[i]<<<grid, block, smem>>>(M, N, K, in, B, C, out, alpha, beta)
 *      (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:15-16,126).  Here the same tables
 *      hold host functions with the same argument lists; a driver replaces the <<<...>>> launch by
 *      a plain call.  They run on the current device's default stream through the C ABI.
 */
#ifndef TURBOFNO_COMPAT_H
#define TURBOFNO_COMPAT_H

#include <cuda_runtime.h>
#include "turbofno_b200.h"

/* retained modes per row tile and the reference's GEMM tile shape */
#define THREADBLOCK_M 64
#define THREADBLOCK_N 64
#define THREADBLOCK_K 8
#define WARP_M 32
#define WARP_N 16
#define THREAD_M 4
#define THREAD_N 4
#define THREAD_NUM (THREADBLOCK_M * THREADBLOCK_N / (THREAD_M * THREAD_N))

#ifdef __cplusplus
static int ntest = 5;            /* timed repetitions per configuration (utils/TurboFNO.h:19) */
static int threadblock_bs = 4;   /* accepted and ignored by the stride kernels (utils/TurboFNO.h:20) */

namespace turbofno_compat {

inline tfno_handle* current_handle() {
    static tfno_handle* handles[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!handles[dev] && tfno_create(&handles[dev], dev) != TFNO_OK) handles[dev] = nullptr;
    return handles[dev];
}
/* status of the most recent table call on this thread (the reference checked cudaGetLastError) */
inline int& last_status() { static thread_local int s = TFNO_OK; return s; }

template <int LOG2>
void fused_fft_cgemm_ifft_fn(int M, int N, int K, float2* in, float2* B, float2* C, float2* out, float2 alpha, float2 beta) {
    last_status() = tfno_fused_fft_cgemm_ifft(current_handle(), LOG2, M, N, K, in, B, C, out, alpha.x, alpha.y, beta.x, beta.y, nullptr);
}
template <int LOG2>
void fused_fft_cgemm_fn(int M, int N, int K, float2* in, float2* B, float2* C, float2 alpha, float2 beta) {
    last_status() = tfno_fused_fft_cgemm(current_handle(), LOG2, M, N, K, in, B, C, alpha.x, alpha.y, beta.x, beta.y, nullptr);
}
template <int LOG2>
void fused_cgemm_ifft_fn(int M, int N, int K, float2* A, float2* B, float2* C, float2* out, float2 alpha, float2 beta) {
    last_status() = tfno_fused_cgemm_ifft(current_handle(), LOG2, M, N, K, A, B, C, out, alpha.x, alpha.y, beta.x, beta.y, nullptr);
}
template <int LOG2>
void fft_stride_DY_fn(float2* in, float2* out, int /*threadblock_bs*/, int total_signals) {
    last_status() = tfno_fft_stride_DY(current_handle(), LOG2, in, out, total_signals, nullptr);
}
template <int LOG2>
void ifft_stride_DY_fn(float2* in, float2* out, int /*threadblock_bs*/, int total_signals) {
    last_status() = tfno_ifft_stride_DY(current_handle(), LOG2, in, out, total_signals, nullptr);
}
template <int LOG2>
void fft_stride_fn(float2* in, float2* out, int /*threadblock_bs*/, int DY, int total_columns, int /*dimX*/) {
    last_status() = tfno_fft_stride(current_handle(), LOG2, in, out, DY, total_columns, nullptr);
}
template <int LOG2>
void ifft_stride_fn(float2* in, float2* out, int /*threadblock_bs*/, int DY, int total_columns, int /*dimX*/) {
    last_status() = tfno_ifft_stride(current_handle(), LOG2, in, out, DY, total_columns, nullptr);
}
inline void cgemm(int M, int N, int K, float2* A, float2* B, float2* C, float2 alpha, float2 beta) {
    last_status() = tfno_cgemm(current_handle(), M, N, K, A, B, C, alpha.x, alpha.y, beta.x, beta.y, nullptr);
}

}  // namespace turbofno_compat

/* the tables, under the reference's names */
#define TFNO_TABLE4(fn) { turbofno_compat::fn<7>, turbofno_compat::fn<8>, turbofno_compat::fn<9>, turbofno_compat::fn<10> }
static void (*fused_fft_cgemm_ifft[4])(int, int, int, float2*, float2*, float2*, float2*, float2, float2) = TFNO_TABLE4(fused_fft_cgemm_ifft_fn);
static void (*fused_fft_cgemm[4])(int, int, int, float2*, float2*, float2*, float2, float2) = TFNO_TABLE4(fused_fft_cgemm_fn);
static void (*fused_cgemm_ifft[4])(int, int, int, float2*, float2*, float2*, float2*, float2, float2) = TFNO_TABLE4(fused_cgemm_ifft_fn);
static void (*fft_stride_DY[4])(float2*, float2*, int, int) = TFNO_TABLE4(fft_stride_DY_fn);
static void (*ifft_stride_DY[4])(float2*, float2*, int, int) = TFNO_TABLE4(ifft_stride_DY_fn);
static void (*fft_stride[4])(float2*, float2*, int, int, int, int) = TFNO_TABLE4(fft_stride_fn);
static void (*ifft_stride[4])(float2*, float2*, int, int, int, int) = TFNO_TABLE4(ifft_stride_fn);
using turbofno_compat::cgemm;
#undef TFNO_TABLE4
#endif /* __cplusplus */

#endif /* TURBOFNO_COMPAT_H */

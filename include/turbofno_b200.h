/* turbofno_b200 -- C ABI of the FNO spectral-convolution path for NVIDIA B200 (sm_100a).
 *
 *     y = iFFT( zero-pad( alpha * ( keep-64-modes( FFT(x) ) x W ) ) )          1D and 2D, complex64
 *
 * The reference project (shixun404/TurboFNO) has no library interface: its operator surface is
 * a set of __global__ kernels with fixed launch contracts, selected through function-pointer
 * tables inside ten benchmark executables.  Each entry point below names the reference
 * interface it stands in for (path inside the reference tree : line).
 *
 * Conventions
 *   - every function returns a tfno_status (0 = TFNO_OK); nothing prints, nothing calls exit()
 *     (the reference's CHECK_CUDA_KERNEL / CUBLAS_CALL macros exit, utils/utils.cuh:17-25,82-92)
 *   - all tensors are interleaved complex64 (float re, float im); pointers are plain device
 *     pointers unless a function says "host"; 16-byte alignment is required and checked
 *   - `stream` is a cudaStream_t passed as void*; execution is asynchronous and stream-ordered,
 *     with no host synchronisation and no allocation inside tfno_exec
 *   - strides are in complex elements.  The reference memory layout is channel-outermost:
 *       1D  x[(k*B + b)*DY + y],           B = bs*dimX   (fusion_variants/1D_E_baseline/fused.cu:186: lda = M)
 *       2D  x[((k*bs + b)*DX + ix)*DY + iy]              (fusion_variants/2D_E_baseline/fused_trunc_2D.cu:200-208)
 *       W   w[k + n*K]                                   (fusion_variants/1D_E_baseline/cgemm.cuh:42-43)
 *     A stride of 0 in tfno_problem selects these defaults; any other batch/channel strides
 *     (for instance [bs][K][DY] with W[K][N]) are served by the same kernels.
 *   - the retained-mode count is 64 per transformed axis, as in the reference
 *     (THREADBLOCK_M, utils/TurboFNO.h:2); K must be a multiple of 8 and N of 64.
 */
#ifndef TURBOFNO_B200_H
#define TURBOFNO_B200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    TFNO_OK = 0,
    TFNO_ERR_INVALID_ARG = 1,   /* null pointer, misaligned pointer, non-positive size          */
    TFNO_ERR_UNSUPPORTED = 2,   /* size outside DY,DX in {128,256,512,1024}, K%8, N%64, modes!=64 */
    TFNO_ERR_CUDA = 3,          /* a CUDA runtime call or kernel launch failed                    */
    TFNO_ERR_ALLOC = 4,         /* host or device allocation failed                               */
    TFNO_ERR_LIBRARY = 5,       /* cuFFT / cuBLAS failure (variant E only)                        */
    TFNO_ERR_WORKSPACE = 6,     /* workspace missing or smaller than tfno_workspace_bytes()       */
    TFNO_ERR_SCRATCH_LIMIT = 7, /* tfno_spectral_conv2d_static: problem exceeds the static scratch */
    TFNO_ERR_KERNEL_WAIT = 8    /* tfno_exec_host: a kernel-side bounded wait ran out, y incomplete */
} tfno_status;

/* Fusion variants, named after the reference executables TurboFNO_{1D,2D}_{A..E}
 * (fusion_variants/<variant>/CMakeLists.txt:5-9). */
typedef enum {
    TFNO_VARIANT_A = 0,   /* FFT ; CGEMM ; iFFT                 (three to five kernels)            */
    TFNO_VARIANT_B = 1,   /* fused FFT+CGEMM ; iFFT                                                */
    TFNO_VARIANT_C = 2,   /* FFT ; fused CGEMM+iFFT                                                */
    TFNO_VARIANT_D = 3,   /* 1D: one fused kernel.  2D: image FFT ; CGEMM ; image iFFT, with the
                             X/Y intermediate in shared memory                                     */
    TFNO_VARIANT_E = 4    /* cuFFT ; truncate ; cuBLAS CGEMM ; zero-pad ; cuFFT   (library path)   */
} tfno_variant;

typedef struct {
    int rank;                 /* 1 or 2                                                            */
    long long bs;             /* batch                                                             */
    int dimX;                 /* 1D: independent rows per batch item (reference dimX); 2D: unused   */
    int DX;                   /* 2D: image rows (transformed, strided axis); 1D: unused             */
    int DY;                   /* transformed contiguous axis                                        */
    int K, N;                 /* input / output channels                                            */
    int modes;                /* retained modes per axis; must be 64                                */
    int variant;              /* tfno_variant                                                       */
    long long x_stride_b, x_stride_k;   /* 1D: b indexes bs*dimX rows.  0 = reference layout        */
    long long y_stride_b, y_stride_n;
    long long w_stride_k, w_stride_n;
    float alpha_re, alpha_im; /* scales the channel contraction (reference: alpha, fused.cu:116)    */
    float beta_re, beta_im;   /* variants A, B, C, E: C = alpha*A*W + beta*C on the workspace C;
                                 ignored by D exactly as the reference's fused kernel ignores it
                                 (fused_fft_cgemm_ifft_7.cuh:184-187)                                */
    int second_transform_forward;  /* 0: true inverse transform (FNO semantics).  1: run the second
                                      transform forward, as the reference drivers do
                                      (fusion_variants/1D_E_baseline/fused.cu:190)                   */
    int scale_inverse;        /* 1: multiply by 1/DY (1D) or 1/(DX*DY) (2D); 0: unnormalised        */
    int x_modes_centered;     /* 2D, variant D: keep X modes -32..31 (low positive AND low negative
                                 frequencies, what an FNO layer keeps along a non-last axis) instead
                                 of the reference's corner 0..63
                                 (fusion_variants/2D_E_baseline/fused_trunc_2D.cu:30-39); Y modes
                                 stay 0..63.  0 = reference behaviour.                               */
    long long w_stride_m;     /* 0: one K x N weight matrix shared by all modes, as in the reference
                                 (fusion_variants/1D_E_baseline/cgemm.cuh:42-43).  Non-zero: per-mode
                                 weights, what an FNO layer trains: element (k, n, m) at
                                 k*w_stride_k + n*w_stride_n + m*w_stride_m, m = mode (1D) or
                                 kx*64 + ky (2D).  With w_stride_k = w_stride_n = 0 the layout is
                                 w[(n*K + k)*modes + m] (w_stride_m is then taken as 1).  Fast when
                                 w_stride_m = 1.  1D variants A and D and the 2D variant D (all run
                                 transform ; per-mode contraction ; transform), K <= 96, beta = 0.  */
} tfno_problem;

typedef struct tfno_handle_s tfno_handle;   /* one per device                                      */
typedef struct tfno_plan_s tfno_plan;       /* immutable after creation; usable from any thread
                                               with external per-stream ordering                   */

/* Fill *p with FNO defaults: modes 64, alpha 1, beta 0, true inverse, scaled, variant D,
 * reference layout.  Stands in for the constants at fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:25-35. */
int tfno_problem_init(tfno_problem* p, int rank);

/* Replaces the implicit device-0 context of every reference driver (no cudaSetDevice anywhere). */
int tfno_create(tfno_handle** out, int device);
int tfno_destroy(tfno_handle* h);
/* Device-side status word of the handle: 0, or the code of the first bounded wait that ran out
 * inside a kernel (the kernel then stops early and its output is incomplete).  Synchronises the
 * whole device (all streams) before reading.  tfno_exec is asynchronous and cannot report this
 * itself: callers that need the guarantee read the word after synchronising; tfno_exec_host does
 * so and returns TFNO_ERR_KERNEL_WAIT.  The reference has no counterpart: its kernels contain no waits. */
int tfno_device_status(tfno_handle* h, int* out);
/* Sets the status word back to 0 (after the caller has dealt with a reported time-out). */
int tfno_device_status_reset(tfno_handle* h);
/* Launches one warp that waits on a barrier nothing completes: the wait gives up after its limit
 * (one second), the kernel returns normally and tfno_device_status then reads 99.  Shows that a
 * kernel-side wait of this library cannot hang the device; no counterpart in the reference. */
int tfno_selftest_bounded_wait(tfno_handle* h, void* stream);
/* number of SMs of the handle's device (148 on B200); grids are sized from it */
int tfno_sm_count(const tfno_handle* h, int* out);

/* Replaces the per-configuration set-up block of the drivers: grid/block/shared-memory sizing and
 * kernel-table lookup by log2(DY)-7 (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:15-16,119-126),
 * and for variant E cublasCreate + cufftPlan1d / cufftPlanMany
 * (fusion_variants/1D_E_baseline/fused.cu:171-179, fusion_variants/2D_E_baseline/fused_trunc_2D.cu:193-208). */
int tfno_plan_create(tfno_handle* h, const tfno_problem* problem, tfno_plan** out);
int tfno_plan_destroy(tfno_plan* plan);

/* Bytes of caller-provided device scratch tfno_exec needs (intermediates A, C and, for E, the
 * full-size transform buffer -- dA, dC, dFFT_output at fusion_variants/1D_E_baseline/fused.cu:95-100).
 * 0 for the fused 1D variant D. */
size_t tfno_workspace_bytes(const tfno_plan* plan);

/* One spectral-convolution layer.  Replaces the timed body of the drivers
 * (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:135-139 and the A/B/C/E equivalents). */
int tfno_exec(const tfno_plan* plan, const void* x, const void* w, void* y,
              void* workspace, void* stream);

/* Same layer with HOST buffers: copies x and w to the device, runs tfno_exec, copies y back,
 * pipelined over batch chunks on internal streams; returns when y is complete.  Staging memory
 * is allocated on the first call and kept by the plan (so this entry point is not thread-safe
 * per plan).  Replaces the cudaMemcpy + launch sequence at
 * fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:116-128.  Requires the reference layout. */
int tfno_exec_host(tfno_plan* plan, const void* x_host, const void* w_host, void* y_host);

/* Batch items per pipeline chunk of tfno_exec_host (0 = choose: about 64 MiB of input per chunk,
 * at least eight chunks per call).  Call before the first tfno_exec_host of the plan.  A tuning
 * knob with no counterpart in the reference, whose drivers copy the whole input with one
 * cudaMemcpy (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:116). */
int tfno_plan_set_host_chunk(tfno_plan* plan, long long batch_items);

/* Writes the names of the kernels (and library calls) one tfno_exec of this plan launches, in
 * launch order and separated by ';', e.g. "spectral_tc_kernel<8,1>" or
 * "fft2d_trunc_kernel<4,4,paired,256>;cgemm_tc_kernel<128>;ifft2d_pad_kernel<4,4,paired,256>".
 * It is produced by a dry run of the dispatch code tfno_exec itself executes.  Stands in for reading
 * which table entry a reference driver launches
 * (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:15-16,126). */
int tfno_plan_kernels(const tfno_plan* plan, char* buf, size_t cap);

const char* tfno_status_string(int status);

/* ---- stage-level entry points, shaped like the reference's kernel tables ------------------------
 * M = rows*64 everywhere, log2_len = log2(transform length) in 7..10, exactly the table index + 7
 * of the reference.  All are asynchronous on `stream`.                                           */

/* fused_fft_cgemm_ifft_{7..10}(M,N,K,in,B,C,out,alpha,beta) <<<(M/64,N/64),256>>>
 * (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:15-16,126).  C is unused, as in the reference. */
int tfno_fused_fft_cgemm_ifft(tfno_handle* h, int log2_len, long long M, int N, int K, const void* in,
                              const void* B, void* C, void* out, float alpha_re, float alpha_im,
                              float beta_re, float beta_im, void* stream);
/* fused_fft_cgemm_{7..10}(M,N,K,in,B,C,alpha,beta) (fusion_variants/1D_B_exp_fused_fft_cgemm+ifft/fused.cu:21-22,141) */
int tfno_fused_fft_cgemm(tfno_handle* h, int log2_len, long long M, int N, int K, const void* in,
                         const void* B, void* C, float alpha_re, float alpha_im, float beta_re,
                         float beta_im, void* stream);
/* fused_cgemm_ifft_{7..10}(M,N,K,A,B,C,out,alpha,beta) (fusion_variants/1D_C_exp_fft+fused_cgemm_ifft/fused.cu:139-147) */
int tfno_fused_cgemm_ifft(tfno_handle* h, int log2_len, long long M, int N, int K, const void* A,
                          const void* B, void* C, void* out, float alpha_re, float alpha_im,
                          float beta_re, float beta_im, void* stream);
/* cgemm(M,N,K,A,B,C,alpha,beta): C[m+n*M] = alpha*sum_k A[m+k*M]*B[k+n*K] + beta*C[m+n*M]
 * (fusion_variants/1D_E_baseline/cgemm.cuh:4-205; launch fusion_variants/1D_A_exp_fft+cgemm+ifft/fused.cu:182-199) */
int tfno_cgemm(tfno_handle* h, long long M, int N, int K, const void* A, const void* B, void* C,
               float alpha_re, float alpha_im, float beta_re, float beta_im, void* stream);
/* fft_{7..10}_stride_DY(in,out,threadblock_bs,total_signals): [signal][len] -> [signal][64]
 * (fusion_variants/1D_A_exp_fft+cgemm+ifft/fused.cu:27-28,195) */
int tfno_fft_stride_DY(tfno_handle* h, int log2_len, const void* in, void* out, long long total_signals,
                       void* stream);
/* ifft_{7..10}_stride_DY: [signal][64] -> zero-pad -> [signal][len]; true inverse, unnormalised
 * (fusion_variants/1D_A_exp_fft+cgemm+ifft/fused.cu:203) */
int tfno_ifft_stride_DY(tfno_handle* h, int log2_len, const void* in, void* out, long long total_signals,
                        void* stream);
/* fft_{7..10}_stride(in,out,threadblock_bs,stride=DY,total=DY*images,dimX=64):
 * [image][len][DY] -> [image][64][DY] along the strided axis
 * (fusion_variants/2D_A_exp_fft+cgemm+ifft/fused_trunc_2D.cu:34,189) */
int tfno_fft_stride(tfno_handle* h, int log2_len, const void* in, void* out, int DY, long long total_columns,
                    void* stream);
/* ifft_{7..10}_stride: [image][64][DY] -> zero-pad -> [image][len][DY]; true inverse, unnormalised
 * (fusion_variants/2D_A_exp_fft+cgemm+ifft/fused_trunc_2D.cu:35,219) */
int tfno_ifft_stride(tfno_handle* h, int log2_len, const void* in, void* out, int DY, long long total_columns,
                     void* stream);

/* ---- allocation-free 2D layer ---------------------------------------------------------------------
 * This entry point has no counterpart in the reference.
 *
 * It is for callers that are not allowed to allocate device memory when they run a layer and have
 * no scratch buffer to pass to tfno_exec: code running inside an arena or memory-pool scheme that
 * already owns the whole device, pipelines whose rules forbid allocation after start-up, and
 * plug-ins called between another framework's allocator operations, where a cudaMalloc would
 * force a device-wide synchronisation.  It computes one 2D spectral-convolution layer (FNO
 * semantics: alpha * contraction, true inverse, 1/(DX*DY)) in the reference layout
 * x[K][bs][DX][DY], w[k + n*K], y[N][bs][DX][DY], with the kernel sequence of a variant-D tfno_exec
 * (image transform, channel contraction, image inverse), but takes its two spectrum buffers from
 * a fixed 64 MiB device array inside the library image.  Every GPU that loads the library carries
 * that array until the process exits.  The contraction always runs on the FP32 kernel here (a
 * plan may pick the tensor-core contraction, which rounds differently in the last bits and is
 * about three times faster on that step), so results agree with tfno_exec to rounding
 * (relative L2 difference around 1e-7), not bit for bit.
 *
 *   - no cudaMalloc / cudaFree / allocating library call is made, on any call
 *   - limit: 8*4096*bs*(K + N) bytes (each term rounded up to 256) must fit in
 *     tfno_static_scratch_bytes(); larger problems return TFNO_ERR_SCRATCH_LIMIT, and a K too
 *     large for the contraction's shared memory returns TFNO_ERR_UNSUPPORTED; a refused call
 *     enqueues nothing
 *   - DX, DY in {128, 256}; K a multiple of 8, N a multiple of 64; 16-byte aligned pointers
 *   - runs on the CURRENT device, asynchronously on `stream`
 *   - the first call on a device looks up the array's device address and the device limits
 *     (host-side work only); make that first call before starting any stream capture, and not
 *     from two threads at once
 *   - all calls on a device share the one array: two calls that can overlap on the GPU (different
 *     streams without an ordering between them) race on it.  Calls on one stream are safe, and
 *     nothing in the array needs clearing between calls.
 */
size_t tfno_static_scratch_bytes(void);
int tfno_spectral_conv2d_static(long long bs, int DX, int DY, int K, int N, const void* x, const void* w,
                                void* y, float alpha_re, float alpha_im, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TURBOFNO_B200_H */

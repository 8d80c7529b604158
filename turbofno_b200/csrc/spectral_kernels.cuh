// Hand-written sm_100a kernels of the spectral-convolution path (SIMT FP32 generation).
//
//   spectral_tile_kernel<R, FWD, INV>    one 64-mode row tile per CTA: [forward transform ->]
//                                        complex GEMM over channels [-> inverse transform]
//        <R,1,1>  fused FFT+CGEMM+iFFT   fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused_fft_cgemm_ifft_7.cuh:9-222
//        <R,1,0>  fused FFT+CGEMM        fusion_variants/1D_B_exp_fused_fft_cgemm+ifft/fused_fft_cgemm_7.cuh:8-197
//        <R,0,1>  fused CGEMM+iFFT       fusion_variants/1D_C_exp_fft+fused_cgemm_ifft/fused_cgemm_ifft_7.cuh:9-222
//        <R,0,0>  CGEMM                  fusion_variants/1D_E_baseline/cgemm.cuh:4-205
//   fft_rows_trunc_kernel<R>, ifft_rows_pad_kernel<R>     contiguous-axis transforms
//        (fft_N_stride_DY / ifft_N_stride_DY, launches at fusion_variants/1D_A_exp_fft+cgemm+ifft/fused.cu:187-203)
//   fft_cols_trunc_kernel<R>, ifft_cols_pad_kernel<R>     strided-axis transforms
//        (fft_N_stride / ifft_N_stride, launches at fusion_variants/2D_D_exp_fused_fft_cgemm_ifft/fused_trunc_2D.cu:153-170)
//   fft2d_trunc_kernel<RX,RY>, ifft2d_pad_kernel<RX,RY>   whole-image 2-D transforms with the
//        DX x 64 intermediate kept in shared memory (no counterpart in the reference, which
//        round-trips the X-transformed image through global memory)
//
// Unlike the reference's fused kernel, one CTA produces ALL N output channels of its row, so the
// forward transform of a row is never recomputed per N-tile (grid.y = N/64 in the reference).
#pragma once
#include "fft64.cuh"

namespace tfno {

constexpr int kThreads = 256;      // threads per CTA for every kernel in this file
constexpr int kModes = 64;         // retained modes per transformed axis
constexpr int kSlabK = 8;          // channels per weight slab in the GEMM main loop
constexpr int kWPad = 2;           // row padding of the weight slab (bank spread for k-fastest fills)

// A [rows][64] complex tile in shared memory: 512-byte rows of 32 16-byte chunks.  The low three
// bits of the chunk index are XOR-swizzled so that (a) the R lanes of a group storing chunks
// 128*r bytes apart, (b) two adjacent rows written in the same phase, and (c) column reads that
// walk rows at a fixed chunk, all spread over distinct banks.
TFNO_HD int swz_chunk(int row, int c) {
    int x = ((((c >> 3) & 3) + ((row & 1) << 2)) ^ (((row >> 1) & 1) << 1)) & 7;
    return (c & ~7) | ((c & 7) ^ x);
}
// byte-free helpers: index in float2 units of element m of row `row`
TFNO_HD int tile_index(int row, int m) { return row * kModes + swz_chunk(row, m >> 1) * 2 + (m & 1); }

// The [n][64] tile handed from the GEMM to the inverse transform: chunk ^ (n & 7).
TFNO_HD int ctile_chunk(int n, int c) { return (c & ~7) | ((c & 7) ^ (n & 7)); }

struct TileParams {
    // problem
    long long rows;          // number of 64-mode row tiles: bs*dimX (1D), bs*64 (2D, per X-mode row)
    int K, N;
    // operand addressing, in complex elements
    const float2* x;         // FWD: signals; !FWD: compact spectrum A[m + k*M], M = rows*64
    long long x_stride_row;  // FWD: between rows
    long long x_stride_k;    // FWD: between channels
    const float2* w;
    long long w_stride_k, w_stride_n;
    float2* y;               // INV: signals out; !INV: compact C[m + n*M]
    long long y_stride_row, y_stride_n;
    float2 alpha, beta;      // beta only read when !INV
    float2 inv_gain;         // alpha * scale folded into the inverse twiddles (INV)
    int conj_inverse;        // 1: true inverse, 0: second forward transform
};

// ----------------------------------------------------------------------------------------------
// lane-level load / store of one decimated signal
// ----------------------------------------------------------------------------------------------
template <int R>
TFNO_D void load_decimated(float2 (&v)[64], const float2* __restrict__ sig, long long elem_stride, int r) {
#pragma unroll
    for (int n = 0; n < 64; ++n) v[n] = __ldg(sig + (long long)(R * n + r) * elem_stride);
}

template <int R>
TFNO_D void store_decimated(const float2 (&v)[64], float2* __restrict__ sig, long long elem_stride, int j1) {
#pragma unroll
    for (int j2 = 0; j2 < 64; ++j2) sig[(long long)(R * j2 + j1) * elem_stride] = v[slot(j2)];
}

// The same for contiguous, 16-byte aligned signals whose R lanes are ADJACENT lanes of a warp: a
// lane and its neighbour (lane ^ 1) want samples that alternate in memory (R*n + r and
// R*n + r + 1), so each of them moves 16 bytes (two samples, one its own and one the
// neighbour's) for every second n and they swap the foreign halves with one shuffle.  Half as
// many load / store instructions, each touching 64 instead of 32 contiguous bytes per signal.
template <int R>
TFNO_D void load_decimated_paired(float2 (&v)[64], const float2* __restrict__ sig, int r) {
    const bool odd = (r & 1) != 0;
    const float2* base = sig + (odd ? R : 0) + (r & ~1);
#pragma unroll
    for (int n2 = 0; n2 < 32; ++n2) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(base + 2 * R * n2));   // samples R*(2*n2 + odd) + (r & ~1), +1
        const float2 mine = odd ? make_float2(q.z, q.w) : make_float2(q.x, q.y);
        const float2 send = odd ? make_float2(q.x, q.y) : make_float2(q.z, q.w);
        float2 got;
        got.x = __shfl_xor_sync(0xffffffffu, send.x, 1);
        got.y = __shfl_xor_sync(0xffffffffu, send.y, 1);
        v[2 * n2] = odd ? got : mine;          // even lane: its sample of n = 2*n2; odd lane: received
        v[2 * n2 + 1] = odd ? mine : got;
    }
}

template <int R>
TFNO_D void store_decimated_paired(const float2 (&v)[64], float2* __restrict__ sig, int j1, bool live = true) {
    const bool odd = (j1 & 1) != 0;
    float2* base = sig + (odd ? R : 0) + (j1 & ~1);
#pragma unroll
    for (int n2 = 0; n2 < 32; ++n2) {
        const float2 even_j2 = v[slot(2 * n2)], odd_j2 = v[slot(2 * n2 + 1)];
        // an even lane writes (own, neighbour's) of j2 = 2*n2, an odd lane (neighbour's, own) of j2 = 2*n2 + 1
        const float2 send = odd ? even_j2 : odd_j2;
        float2 got;
        got.x = __shfl_xor_sync(0xffffffffu, send.x, 1);
        got.y = __shfl_xor_sync(0xffffffffu, send.y, 1);
        const float4 q = odd ? make_float4(got.x, got.y, odd_j2.x, odd_j2.y) : make_float4(even_j2.x, even_j2.y, got.x, got.y);
        if (live) *reinterpret_cast<float4*>(base + 2 * R * n2) = q;
    }
}

// After forward_trunc<R>: lane r holds modes 64/R*r + j in v[slot(j)].  Write them as 16-byte
// chunks into a swizzled tile row.
template <int R>
TFNO_D void store_modes_to_tile(const float2 (&v)[64], float2* tile, int row, int r) {
    constexpr int PER = 64 / R;
#pragma unroll
    for (int j = 0; j < PER; j += 2) {
        int m = PER * r + j;
        float4 q = make_float4(v[slot(j)].x, v[slot(j)].y, v[slot(j + 1)].x, v[slot(j + 1)].y);
        *reinterpret_cast<float4*>(tile + row * kModes + swz_chunk(row, m >> 1) * 2) = q;
    }
}

// ----------------------------------------------------------------------------------------------
// The row-tile kernel
// ----------------------------------------------------------------------------------------------
template <int R, bool FWD, bool INV, int NB>   // NB = N / 64
__global__ void __launch_bounds__(kThreads, 1) spectral_tile_kernel(TileParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* sA = reinterpret_cast<float2*>(smem_raw);                 // [K][64] swizzled
    float2* sC = sA + (size_t)p.K * kModes;                            // [N][64] swizzled (INV only)
    float2* sW = sC + (INV ? (size_t)p.N * kModes : 0);                // [2][kSlabK][N]
    float2* twF = sW + 2 * kSlabK * (p.N + kWPad);                               // [R][64]
    float2* twI = twF + (FWD ? R * 64 : 0);                            // [R][64]

    const int tid = threadIdx.x;
    const int K = p.K, N = p.N;
    if (FWD) fill_forward_table<R>(twF, tid, kThreads);
    if (INV) fill_inverse_table<R>(twI, tid, kThreads, p.inv_gain, p.conj_inverse != 0);
    __syncthreads();

    const long long M = p.rows * kModes;
    const int tm = tid & 15, tn = tid >> 4;        // GEMM thread tile: modes {2tm,2tm+1,32+2tm,33+2tm} x 4 n
    // blockIdx.y selects a block of N output channels: small batches of a wide layer are spread
    // over more CTAs that way (each repeats the row's forward transform, in parallel)
    const float2* wbase = p.w + (long long)blockIdx.y * N * p.w_stride_n;
    float2* ybase = p.y + (long long)blockIdx.y * N * (INV ? p.y_stride_n : M);

    for (long long row = blockIdx.x; row < p.rows; row += gridDim.x) {
        // ---------------- stage 1: spectrum tile sA[k][m] ----------------
        if (FWD) {
            constexpr int GROUPS = kThreads / R;
            const int g = tid / R, r = tid % R;
            const int warp_g0 = (tid & ~31) / R;        // first group of this warp
            for (int k0 = 0; k0 < K; k0 += GROUPS) {
                // Whole warps beyond K skip; inside a partly filled warp the spare lanes redo
                // channel K-1 so that every lane takes part in the shuffles of forward_trunc.
                if (k0 + warp_g0 >= K) continue;
                const bool live = k0 + g < K;
                const int k = live ? k0 + g : K - 1;
                float2 v[64];
                load_decimated_paired<R>(v, p.x + row * p.x_stride_row + (long long)k * p.x_stride_k, r);
                forward_trunc<R>(v, twF, r);
                if (live) store_modes_to_tile<R>(v, sA, k, r);
            }
        } else {
            // compact spectrum: 64 consecutive m per channel
            for (int i = tid; i < K * 32; i += kThreads) {
                int k = i >> 5, c = i & 31;
                float4 q = __ldg(reinterpret_cast<const float4*>(p.x + row * kModes + (long long)k * M) + c);
                *reinterpret_cast<float4*>(sA + k * kModes + swz_chunk(k, c) * 2) = q;
            }
        }

        // ---------------- stage 2: C[m][n] = sum_k A[k][m] W[k][n] ----------------
        float2 acc[NB][4][4];
#pragma unroll
        for (int b = 0; b < NB; ++b)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[b][i][j] = make_float2(0.f, 0.f);

        constexpr int WPT = kSlabK * 64 * NB / kThreads;     // weight elements per thread per slab
        float2 wreg[WPT];
        auto fetch_slab = [&](int k0) {
#pragma unroll
            for (int i = 0; i < WPT; ++i) {
                int e = tid + i * kThreads;
                int kk, n;
                if (p.w_stride_n == 1) { n = e % N; kk = e / N; } else { kk = e % kSlabK; n = e / kSlabK; }
                wreg[i] = __ldg(wbase + (long long)(k0 + kk) * p.w_stride_k + (long long)n * p.w_stride_n);
            }
        };
        auto stash_slab = [&](int buf) {
#pragma unroll
            for (int i = 0; i < WPT; ++i) {
                int e = tid + i * kThreads;
                int kk, n;
                if (p.w_stride_n == 1) { n = e % N; kk = e / N; } else { kk = e % kSlabK; n = e / kSlabK; }
                sW[(buf * kSlabK + kk) * (N + kWPad) + n] = wreg[i];
            }
        };
        fetch_slab(0);
        stash_slab(0);
        __syncthreads();   // sA complete, slab 0 visible

        for (int k0 = 0, buf = 0; k0 < K; k0 += kSlabK, buf ^= 1) {
            const bool more = k0 + kSlabK < K;
            if (more) fetch_slab(k0 + kSlabK);
#pragma unroll
            for (int kk = 0; kk < kSlabK; ++kk) {
                const int k = k0 + kk;
                const float4 a01 = *reinterpret_cast<const float4*>(sA + k * kModes + swz_chunk(k, tm) * 2);
                const float4 a23 = *reinterpret_cast<const float4*>(sA + k * kModes + swz_chunk(k, 16 + tm) * 2);
                const float2 a[4] = {make_float2(a01.x, a01.y), make_float2(a01.z, a01.w),
                                     make_float2(a23.x, a23.y), make_float2(a23.z, a23.w)};
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const float4* wp = reinterpret_cast<const float4*>(sW + (buf * kSlabK + kk) * (N + kWPad) + 64 * b + 4 * tn);
                    const float4 w01 = wp[0], w23 = wp[1];
                    const float2 w[4] = {make_float2(w01.x, w01.y), make_float2(w01.z, w01.w),
                                         make_float2(w23.x, w23.y), make_float2(w23.z, w23.w)};
#pragma unroll
                    for (int i = 0; i < 4; ++i)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            acc[b][i][j].x = fmaf(a[i].x, w[j].x, acc[b][i][j].x);
                            acc[b][i][j].x = fmaf(-a[i].y, w[j].y, acc[b][i][j].x);
                            acc[b][i][j].y = fmaf(a[i].x, w[j].y, acc[b][i][j].y);
                            acc[b][i][j].y = fmaf(a[i].y, w[j].x, acc[b][i][j].y);
                        }
                }
            }
            if (more) stash_slab(buf ^ 1);
            __syncthreads();
        }

        // ---------------- stage 3: epilogue ----------------
        if (INV) {
            // alpha and the 1/DY scale live in the inverse twiddles; hand C to the transform lanes
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = 64 * b + 4 * tn + j;
                    float4 q0 = make_float4(acc[b][0][j].x, acc[b][0][j].y, acc[b][1][j].x, acc[b][1][j].y);
                    float4 q1 = make_float4(acc[b][2][j].x, acc[b][2][j].y, acc[b][3][j].x, acc[b][3][j].y);
                    *reinterpret_cast<float4*>(sC + n * kModes + ctile_chunk(n, tm) * 2) = q0;
                    *reinterpret_cast<float4*>(sC + n * kModes + ctile_chunk(n, 16 + tm) * 2) = q1;
                }
            __syncthreads();
            constexpr int GROUPS = kThreads / R;
            const int g = tid / R, j1 = tid % R;
            for (int n0 = 0; n0 < N; n0 += GROUPS) {
                int n = n0 + g;
                if (n < N) {
                    float2 v[64];
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        float4 q = *reinterpret_cast<const float4*>(sC + n * kModes + ctile_chunk(n, c) * 2);
                        v[2 * c] = make_float2(q.x, q.y);
                        v[2 * c + 1] = make_float2(q.z, q.w);
                    }
                    if (p.conj_inverse) inverse_pad_lane<+1, R>(v, twI, j1);
                    else inverse_pad_lane<-1, R>(v, twI, j1);
                    store_decimated_paired<R>(v, ybase + row * p.y_stride_row + (long long)n * p.y_stride_n, j1);   // whole warps: N is a multiple of 64
                }
            }
            __syncthreads();   // sC and sA are rewritten by the next row
        } else {
            const bool use_beta = (p.beta.x != 0.f || p.beta.y != 0.f);
#pragma unroll
            for (int b = 0; b < NB; ++b)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = 64 * b + 4 * tn + j;
                    float2* dst = ybase + row * kModes + (long long)n * M;
                    float2 o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[i] = cmul(acc[b][i][j], p.alpha);
                    float4* d0 = reinterpret_cast<float4*>(dst + 2 * tm);
                    float4* d1 = reinterpret_cast<float4*>(dst + 32 + 2 * tm);
                    if (use_beta) {
                        float4 c0 = *d0, c1 = *d1;
                        o[0] = cadd(o[0], cmul(make_float2(c0.x, c0.y), p.beta));
                        o[1] = cadd(o[1], cmul(make_float2(c0.z, c0.w), p.beta));
                        o[2] = cadd(o[2], cmul(make_float2(c1.x, c1.y), p.beta));
                        o[3] = cadd(o[3], cmul(make_float2(c1.z, c1.w), p.beta));
                    }
                    *d0 = make_float4(o[0].x, o[0].y, o[1].x, o[1].y);
                    *d1 = make_float4(o[2].x, o[2].y, o[3].x, o[3].y);
                }
            __syncthreads();   // sA is rewritten by the next row
        }
    }
}

// ----------------------------------------------------------------------------------------------
// Stand-alone transforms along the contiguous axis
// ----------------------------------------------------------------------------------------------
struct RowsParams {
    long long nsig;            // number of signals
    long long per_k;           // signals per channel (rows): signal s -> channel s / per_k, row s % per_k
    const float2* in;
    float2* out;
    long long stride_row, stride_k;   // strides of the full-length side (complex elements)
    float2 gain;
    int conj_inverse;
};

// [signal][DY] -> compact [signal][64]
template <int R>
__global__ void __launch_bounds__(kThreads, 1) fft_rows_trunc_kernel(RowsParams p) {
    __shared__ __align__(16) float2 twF[R * 64];
    fill_forward_table<R>(twF, threadIdx.x, kThreads);
    __syncthreads();
    constexpr int GROUPS = kThreads / R, PER = 64 / R;
    const int g = threadIdx.x / R, r = threadIdx.x % R;
    const long long nblk = (p.nsig + GROUPS - 1) / GROUPS;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        // clamp instead of branching so that every lane of a warp takes part in the shuffles
        long long s = blk * GROUPS + g;
        const bool live = s < p.nsig;
        if (!live) s = p.nsig - 1;
        float2 v[64];
        load_decimated_paired<R>(v, p.in + (s % p.per_k) * p.stride_row + (s / p.per_k) * p.stride_k, r);
        forward_trunc<R>(v, twF, r);
        if (live) {
            float2* dst = p.out + s * kModes + PER * r;
#pragma unroll
            for (int j = 0; j < PER; j += 2)
                *reinterpret_cast<float4*>(dst + j) =
                    make_float4(v[slot(j)].x, v[slot(j)].y, v[slot(j + 1)].x, v[slot(j + 1)].y);
        }
    }
}

// compact [signal][64] -> zero-padded inverse -> [signal][DY]
template <int R>
__global__ void __launch_bounds__(kThreads, 1) ifft_rows_pad_kernel(RowsParams p) {
    __shared__ __align__(16) float2 twI[R * 64];
    fill_inverse_table<R>(twI, threadIdx.x, kThreads, p.gain, p.conj_inverse != 0);
    __syncthreads();
    constexpr int GROUPS = kThreads / R;
    const int g = threadIdx.x / R, j1 = threadIdx.x % R;
    const long long nblk = (p.nsig + GROUPS - 1) / GROUPS;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        // clamp instead of branching so that every lane of a warp takes part in the store's shuffles
        long long s = blk * GROUPS + g;
        const bool live = s < p.nsig;
        if (!live) s = p.nsig - 1;
        float2 v[64];
        const float4* src = reinterpret_cast<const float4*>(p.in + s * kModes);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            float4 q = __ldg(src + c);
            v[2 * c] = make_float2(q.x, q.y);
            v[2 * c + 1] = make_float2(q.z, q.w);
        }
        if (p.conj_inverse) inverse_pad_lane<+1, R>(v, twI, j1);
        else inverse_pad_lane<-1, R>(v, twI, j1);
        store_decimated_paired<R>(v, p.out + (s % p.per_k) * p.stride_row + (s / p.per_k) * p.stride_k, j1, live);
    }
}

// ----------------------------------------------------------------------------------------------
// Stand-alone transforms along the strided (X) axis of [image][DX][DY] data
// ----------------------------------------------------------------------------------------------
struct ColsParams {
    long long nimg;
    long long per_k;           // images per channel: image i -> channel i / per_k, batch i % per_k
    int DY;                    // row length = element stride along X
    const float2* in;
    float2* out;
    long long stride_b, stride_k;   // image strides of the full-size side; the 64-row side is compact
    float2 gain;
    int conj_inverse;
};

// [img][DX][DY] -> [img][64][DY]   (DX = 64*R)
template <int R>
__global__ void __launch_bounds__(kThreads, 1) fft_cols_trunc_kernel(ColsParams p) {
    __shared__ __align__(16) float2 twF[R * 64];
    fill_forward_table<R>(twF, threadIdx.x, kThreads);
    __syncthreads();
    constexpr int GROUPS = kThreads / R, PER = 64 / R;
    const int g = threadIdx.x / R, r = threadIdx.x % R;
    const long long ncol = p.nimg * p.DY;
    const long long nblk = (ncol + GROUPS - 1) / GROUPS;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        long long c = blk * GROUPS + g;
        const bool live = c < ncol;
        if (!live) c = ncol - 1;
        const long long img = c / p.DY;
        const int col = (int)(c % p.DY);
        float2 v[64];
        load_decimated<R>(v, p.in + (img % p.per_k) * p.stride_b + (img / p.per_k) * p.stride_k + col, p.DY, r);
        forward_trunc<R>(v, twF, r);
        if (live) {
            float2* dst = p.out + img * (long long)kModes * p.DY + col;
#pragma unroll
            for (int j = 0; j < PER; ++j) dst[(long long)(PER * r + j) * p.DY] = v[slot(j)];
        }
    }
}

// [img][64][DY] -> zero-pad rows -> inverse along X -> [img][DX][DY]
template <int R>
__global__ void __launch_bounds__(kThreads, 1) ifft_cols_pad_kernel(ColsParams p) {
    __shared__ __align__(16) float2 twI[R * 64];
    fill_inverse_table<R>(twI, threadIdx.x, kThreads, p.gain, p.conj_inverse != 0);
    __syncthreads();
    constexpr int GROUPS = kThreads / R;
    const int g = threadIdx.x / R, j1 = threadIdx.x % R;
    const long long ncol = p.nimg * p.DY;
    const long long nblk = (ncol + GROUPS - 1) / GROUPS;
    for (long long blk = blockIdx.x; blk < nblk; blk += gridDim.x) {
        long long c = blk * GROUPS + g;
        if (c >= ncol) continue;
        const long long img = c / p.DY;
        const int col = (int)(c % p.DY);
        float2 v[64];
        const float2* src = p.in + img * (long long)kModes * p.DY + col;
#pragma unroll
        for (int m = 0; m < 64; ++m) v[m] = __ldg(src + (long long)m * p.DY);
        if (p.conj_inverse) inverse_pad_lane<+1, R>(v, twI, j1);
        else inverse_pad_lane<-1, R>(v, twI, j1);
        store_decimated<R>(v, p.out + (img % p.per_k) * p.stride_b + (img / p.per_k) * p.stride_k + col, p.DY, j1);
    }
}

// ----------------------------------------------------------------------------------------------
// Whole-image 2-D transforms (one CTA per image, DX x 64 intermediate in shared memory)
// ----------------------------------------------------------------------------------------------
struct ImageParams {
    long long nimg;
    long long per_k;                   // images per channel: image i -> channel i / per_k, batch i % per_k
    const float2* in;
    float2* out;
    long long stride_b, stride_k;      // strides of the full-size side
    float2 gain;
    int conj_inverse;
    int centered_x;                    // kept X modes are -32..31 (row kx + 32 of the 64 x 64 block) instead of 0..63
};

// [image][DX][DY] -> [image][64][64]: Y transform of every row (kept modes only) into shared
// memory, then X transform of the 64 kept columns.
// Ask the L2 for `bytes` of contiguous global memory, one 128-byte line per thread and round.
__device__ __forceinline__ void prefetch_l2_block(const void* base, int bytes, int tid, int nthreads) {
    const char* b = static_cast<const char*>(base);
    for (int off = tid * 128; off < bytes; off += nthreads * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(b + off));
}

template <int RX, int RY, bool PAIRED, int THREADS>
__global__ void __launch_bounds__(THREADS, 1) fft2d_trunc_kernel(ImageParams p) {
    constexpr int DX = 64 * RX, DY = 64 * RY;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* sY = reinterpret_cast<float2*>(smem_raw);          // [DX][64] swizzled
    float2* twY = sY + DX * kModes;                             // [RY][64]
    float2* twX = twY + RY * 64;                                // [RX][64]
    const int tid = threadIdx.x;
    fill_forward_table<RY>(twY, tid, THREADS);
    fill_forward_table<RX>(twX, tid, THREADS, p.centered_x != 0);
    __syncthreads();
    for (long long img = blockIdx.x; img < p.nimg; img += gridDim.x) {
        const float2* src = p.in + (img % p.per_k) * p.stride_b + (img / p.per_k) * p.stride_k;
        {
            constexpr int GROUPS = THREADS / RY;
            const int g = tid / RY, r = tid % RY;
#pragma unroll 1
            for (int x0 = 0; x0 < DX; x0 += GROUPS) {
                const int x = x0 + g;
                if (x >= DX) continue;          // last round of a thread count that does not divide DX; whole warps
                float2 v[64];
                if constexpr (PAIRED) load_decimated_paired<RY>(v, src + (long long)x * DY, r);
                else load_decimated<RY>(v, src + (long long)x * DY, 1, r);
                // While these rows are transformed, the rows of the next round (or the first rows
                // of this CTA's next image) travel from DRAM to the L2: a warp has no other loads
                // in flight while it computes, and only two warps share a scheduler.
                if (x0 + GROUPS < DX) {
                    const int next_rows = (DX - (x0 + GROUPS) < GROUPS) ? DX - (x0 + GROUPS) : GROUPS;      // stay inside the image
                    prefetch_l2_block(src + (long long)(x0 + GROUPS) * DY, next_rows * DY * 8, tid, THREADS);
                } else if (img + gridDim.x < p.nimg) {
                    const long long nx = img + gridDim.x;
                    prefetch_l2_block(p.in + (nx % p.per_k) * p.stride_b + (nx / p.per_k) * p.stride_k, GROUPS * DY * 8, tid, THREADS);
                }
                forward_trunc<RY>(v, twY, r);
                store_modes_to_tile<RY>(v, sY, x, r);
            }
        }
        __syncthreads();
        {
            constexpr int GROUPS = THREADS / RX, PER = 64 / RX;
            const int g = tid / RX, r = tid % RX;
            float2* dst = p.out + img * (long long)(kModes * kModes);
#pragma unroll 1
            for (int c0 = 0; c0 < kModes; c0 += GROUPS) {
                const int ky = c0 + g;
                if (ky >= kModes) continue;      // whole warps only (32/RX groups per warp divides 64)
                float2 v[64];
#pragma unroll
                for (int n = 0; n < 64; ++n) v[n] = sY[tile_index(RX * n + r, ky)];
                forward_trunc<RX>(v, twX, r, p.centered_x != 0);
#pragma unroll
                for (int j = 0; j < PER; ++j) dst[(PER * r + j) * kModes + ky] = v[slot(j)];
            }
        }
        __syncthreads();
    }
}

// [image][64][64] -> zero-pad -> inverse along X into shared memory -> inverse along Y -> [image][DX][DY]
template <int RX, int RY, bool PAIRED, int THREADS, bool CENTERED_X = false>
__global__ void __launch_bounds__(THREADS, 1) ifft2d_pad_kernel(ImageParams p) {
    constexpr int DX = 64 * RX, DY = 64 * RY;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float2* sY = reinterpret_cast<float2*>(smem_raw);          // [DX][64] swizzled
    float2* twY = sY + DX * kModes;
    float2* twX = twY + RY * 64;
    const int tid = threadIdx.x;
    fill_inverse_table<RY>(twY, tid, THREADS, make_float2(1.f, 0.f), p.conj_inverse != 0);
    fill_inverse_table<RX>(twX, tid, THREADS, p.gain, p.conj_inverse != 0, CENTERED_X);
    __syncthreads();
    for (long long img = blockIdx.x; img < p.nimg; img += gridDim.x) {
        const float2* src = p.in + img * (long long)(kModes * kModes);
        float2* dst = p.out + (img % p.per_k) * p.stride_b + (img / p.per_k) * p.stride_k;
        {
            constexpr int GROUPS = THREADS / RX;
            const int g = tid / RX, j1 = tid % RX;
#pragma unroll 1
            for (int c0 = 0; c0 < kModes; c0 += GROUPS) {
                const int ky = c0 + g;
                if (ky >= kModes) continue;
                float2 v[64];
#pragma unroll
                for (int m = 0; m < 64; ++m) v[m] = __ldg(src + m * kModes + ky);
                if (p.conj_inverse) inverse_pad_lane<+1, RX, CENTERED_X>(v, twX, j1);
                else inverse_pad_lane<-1, RX>(v, twX, j1);
#pragma unroll
                for (int j2 = 0; j2 < 64; ++j2) sY[tile_index(RX * j2 + j1, ky)] = v[slot(j2)];
            }
        }
        __syncthreads();
        {
            constexpr int GROUPS = THREADS / RY;
            const int g = tid / RY, j1 = tid % RY;
#pragma unroll 1
            for (int x0 = 0; x0 < DX; x0 += GROUPS) {
                const int x = x0 + g;
                if (x >= DX) continue;          // whole warps, as in the forward kernel
                float2 v[64];
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    float4 q = *reinterpret_cast<const float4*>(sY + x * kModes + swz_chunk(x, c) * 2);
                    v[2 * c] = make_float2(q.x, q.y);
                    v[2 * c + 1] = make_float2(q.z, q.w);
                }
                if (p.conj_inverse) inverse_pad_lane<+1, RY>(v, twY, j1);
                else inverse_pad_lane<-1, RY>(v, twY, j1);
                if constexpr (PAIRED) store_decimated_paired<RY>(v, dst + (long long)x * DY, j1);
                else store_decimated<RY>(v, dst + (long long)x * DY, 1, j1);
            }
        }
        __syncthreads();
    }
}

// ----------------------------------------------------------------------------------------------
// Data-movement kernels of the library (cuFFT + cuBLAS) pipeline: keep the first 64 of DY
// entries of each signal / zero-fill back (fusion_variants/1D_E_baseline/fused.cu:13-63), and
// the corner-block forms for images (fusion_variants/2D_E_baseline/fused_trunc_2D.cu:13-71).
// One float4 = two complex per thread, grid-stride.
// ----------------------------------------------------------------------------------------------
__global__ void truncate_rows_kernel(const float4* __restrict__ in, float4* __restrict__ out,
                                     long long nsig, int DY) {
    const long long total = nsig * 32;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        long long s = i >> 5; int c = (int)(i & 31);
        out[i] = __ldg(in + s * (DY / 2) + c);
    }
}
__global__ void zero_pad_rows_kernel(const float4* __restrict__ in, float4* __restrict__ out,
                                     long long nsig, int DY) {
    const int per = DY / 2;
    const long long total = nsig * per;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        long long s = i / per; int c = (int)(i % per);
        out[i] = c < 32 ? __ldg(in + s * 32 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}
__global__ void truncate_corner_kernel(const float4* __restrict__ in, float4* __restrict__ out,
                                       long long nimg, int DX, int DY) {
    const long long total = nimg * 64 * 32;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int c = (int)(i & 31); long long t = i >> 5; int x = (int)(t & 63); long long img = t >> 6;
        out[i] = __ldg(in + (img * DX + x) * (DY / 2) + c);
    }
}
__global__ void zero_pad_corner_kernel(const float4* __restrict__ in, float4* __restrict__ out,
                                       long long nimg, int DX, int DY) {
    const int per = DY / 2;
    const long long total = nimg * DX * per;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int c = (int)(i % per); long long t = i / per; int x = (int)(t % DX); long long img = t / DX;
        out[i] = (c < 32 && x < 64) ? __ldg(in + (img * 64 + x) * 32 + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

}  // namespace tfno

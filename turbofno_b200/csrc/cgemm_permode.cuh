// Channel contraction of compact spectra with PER-MODE weights (what an FNO layer trains):
//
//     C[(n*rows + b)*modes + m] = alpha * sum_k W[k, n, m] * A[(k*rows + b)*modes + m]
//
// The reference contracts with one K x N matrix shared by all modes
// (fusion_variants/1D_E_baseline/cgemm.cuh:42-43, B[k + n*K]); this is the extension its README
// names as the FNO use case, with the reference's compact-spectrum layouts on both sides.  It is
// 64 (1D) or 4096 (2D) independent [rows x K] x [K x N] products whose operands are interleaved
// mode-fastest in memory, so a CTA takes FOUR adjacent modes (one 32-byte sector per (row, channel)
// on the A and C side), keeps their weights W[4][K][64 outputs] in shared memory for as long as it
// stays on those modes, and streams row tiles of 32 past them.  FP32 SIMT: each thread owns one mode,
// four rows and four output channels.
#pragma once
#include <cuda_runtime.h>

namespace tfno {

constexpr int kPmThreads = 512;        // 4 modes x 8 row groups x 16 output groups
constexpr int kPmModes = 4;            // adjacent modes per CTA
constexpr int kPmRowTile = 32;         // rows per tile: 8 row groups of 4
constexpr int kPmNB = 64;              // output channels per pass

struct PerModeParams {
    long long rows;                    // B (1D: bs*dimX, 2D: bs)
    long long modes;                   // 64 (1D) or 4096 (2D); a multiple of 4
    int K, N;
    const float2* a;                   // A[(k*rows + b)*modes + m]
    const float2* w;                   // W[k*w_sk + n*w_sn + m*w_sm]
    long long w_sk, w_sn, w_sm;
    float2* c;                         // C[(n*rows + b)*modes + m]
    float2 alpha;
    int splits;                        // row tiles of a mode group are dealt to this many CTAs
    int stage_a;                       // 1: the A tile goes through shared memory
};

// weights of one mode in shared memory: [K][64] complex, plus 32 bytes so that the four modes a
// warp reads in one instruction fall into different banks
__host__ __device__ inline size_t pm_mode_stride_bytes(int K) { return (size_t)K * kPmNB * sizeof(float2) + 32; }
// A tile of 32 rows x K channels x 4 modes, staged in shared memory when it fits next to the weights
// (K <= 64): all 16 warps of a CTA read the same A values, and reading them from global memory
// through L1 costs the load/store unit 2.4x what the arithmetic costs the FMA pipe.
__host__ __device__ inline size_t pm_atile_bytes(int K) { return (size_t)K * kPmRowTile * kPmModes * sizeof(float2); }
inline bool pm_stage_a(int K, int max_smem) { return (long long)(kPmModes * pm_mode_stride_bytes(K) + pm_atile_bytes(K)) <= max_smem; }
inline size_t pm_smem_bytes(int K, bool stage_a) { return kPmModes * pm_mode_stride_bytes(K) + (stage_a ? pm_atile_bytes(K) : 0); }

__global__ void __launch_bounds__(kPmThreads, 1) cgemm_permode_kernel(PerModeParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x;
    const int j = tid & 3;                       // mode inside the group
    const int rg = (tid >> 2) & 7;               // rows 4*rg .. 4*rg+3 of the tile
    const int nb = tid >> 5;                     // outputs 4*nb .. 4*nb+3 of the pass (warp-uniform)
    const size_t mode_stride = pm_mode_stride_bytes(p.K);
    const long long groups = p.modes / kPmModes;
    const long long tiles = (p.rows + kPmRowTile - 1) / kPmRowTile;
    const int passes = p.N / kPmNB;
    // work item = (mode group, output pass, split): consecutive CTAs take consecutive splits of the
    // same weights, so a weight slice is fetched from DRAM once and then served by the L2
    const long long items = groups * passes * p.splits;
    for (long long item = blockIdx.x; item < items; item += gridDim.x) {
        const int split = (int)(item % p.splits);
        const int pass = (int)((item / p.splits) % passes);
        const long long mg = item / ((long long)p.splits * passes);
        const long long m0 = mg * kPmModes;
        const int n_base = pass * kPmNB;
        __syncthreads();                         // the previous item's weights are no longer read
        for (int i = tid; i < kPmModes * p.K * kPmNB; i += kPmThreads) {
            const int jj = i & 3, n = (i >> 2) & (kPmNB - 1), k = i >> 8;      // mode fastest: one sector per (k, n)
            const float2 wv = __ldg(p.w + (long long)k * p.w_sk + (long long)(n_base + n) * p.w_sn + (m0 + jj) * p.w_sm);
            *reinterpret_cast<float2*>(smem_raw + jj * mode_stride + ((size_t)k * kPmNB + n) * sizeof(float2)) = wv;
        }
        __syncthreads();
        const float2* wj = reinterpret_cast<const float2*>(smem_raw + j * mode_stride) + 4 * nb;
        // staged A tile: sA[k][r][rg][mode] (the 32 lanes of a warp read 256 contiguous bytes)
        float2* sA = reinterpret_cast<float2*>(smem_raw + kPmModes * mode_stride);
        for (long long tile = split; tile < tiles; tile += p.splits) {
            const long long b0 = tile * kPmRowTile + 4 * rg;
            float2 acc[4][4];
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int n = 0; n < 4; ++n) acc[r][n] = make_float2(0.f, 0.f);
            // rows beyond the batch are clamped for the loads and dropped at the store
            long long rowoff[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) rowoff[r] = ((b0 + r < p.rows) ? b0 + r : p.rows - 1) * p.modes + m0 + j;
            if (p.stage_a) {
                __syncthreads();                 // the previous tile is no longer read
                // one 16-byte load = two modes of one (channel, row): 2 * 32 * K of them
                for (int i = tid; i < 2 * kPmRowTile * p.K; i += kPmThreads) {
                    const int half = i & 1, row = (i >> 1) & (kPmRowTile - 1), k = i >> 6;
                    long long b = tile * kPmRowTile + row;
                    if (b >= p.rows) b = p.rows - 1;
                    const float4 q = __ldg(reinterpret_cast<const float4*>(p.a + ((long long)k * p.rows + b) * p.modes + m0) + half);
                    *reinterpret_cast<float4*>(sA + (((size_t)k * 4 + (row & 3)) * 8 + (row >> 2)) * kPmModes + 2 * half) = q;
                }
                __syncthreads();
            }
#pragma unroll 4
            for (int k = 0; k < p.K; ++k) {
                const float4 w01 = *reinterpret_cast<const float4*>(wj + (size_t)k * kPmNB);
                const float4 w23 = *reinterpret_cast<const float4*>(wj + (size_t)k * kPmNB + 2);
                const float2 wv[4] = {make_float2(w01.x, w01.y), make_float2(w01.z, w01.w), make_float2(w23.x, w23.y), make_float2(w23.z, w23.w)};
                const float2* ak = p.a + (long long)k * p.rows * p.modes;
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float2 av = p.stage_a ? sA[(((size_t)k * 4 + r) * 8 + rg) * kPmModes + j] : __ldg(ak + rowoff[r]);
#pragma unroll
                    for (int n = 0; n < 4; ++n) {
                        acc[r][n].x = fmaf(av.x, wv[n].x, fmaf(-av.y, wv[n].y, acc[r][n].x));
                        acc[r][n].y = fmaf(av.x, wv[n].y, fmaf(av.y, wv[n].x, acc[r][n].y));
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                if (b0 + r >= p.rows) continue;
#pragma unroll
                for (int n = 0; n < 4; ++n) {
                    const float2 v = acc[r][n];
                    p.c[((long long)(n_base + 4 * nb + n) * p.rows + b0 + r) * p.modes + m0 + j] =
                        make_float2(p.alpha.x * v.x - p.alpha.y * v.y, p.alpha.x * v.y + p.alpha.y * v.x);
                }
            }
        }
    }
}

}  // namespace tfno

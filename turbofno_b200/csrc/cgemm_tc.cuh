// Channel contraction of compact spectra on the 5th-generation tensor cores:
//
//     C[m + n*M] = alpha * sum_k W[k,n] * A[m + k*M],      m < M = 64 * tiles,  n < 64,  K <= 64
//
// the stand-alone CGEMM of the path (reference: fusion_variants/1D_E_baseline/cgemm.cuh:4-205, a
// SIMT FP32 kernel), used between the two image transforms of the 2-D layer.  Same contraction
// machinery as spectral_tc_kernel: the weights sit in tensor memory as the A operand for the whole
// kernel, a 64-mode tile of the spectra is the B operand S[mode][kk] (K-major, tf32 hi and lo
// parts), fp32 accuracy from three tf32 products.  There is no transform here, so the compute
// warps only move data:
//
//   warps 0,2,4,6  convert  half-teams {0,2} and {4,6}; a half-team takes a chunk of 16 channels
//                           (16 rows of TN*8 bytes, brought by cp.async.bulk into one of ITS two
//                           ring stages), splits the values into tf32 hi/lo and stores them as S
//   warps 1,3,5,7  write    read the Re/Im planes of 16 output channels each, interleave, and store
//                           whole rows with 16-byte stores
//   warps 8-11     hand-off tcgen05.ld of one accumulator row per thread -> planes
//   warp 12        producer
//   warp 13        MMA      D[128 x TN modes] += Wt[128 x 8] * S[8 x TN], three products per k-step
//
// TN = 128 modes per tile when M is a multiple of 128, else 64.  One tcgen05.mma of this shape
// costs about the same for 64 and for 128 columns (measured: the 48 instructions of a 64-mode tile
// took ~7k cycles, more than the tile's HBM time), so the wide tile halves the tensor-core time.
//
// Every ring stage and every S buffer has exactly one consuming half-team, so each waiter sees all
// phases of the barriers it waits on.  Every wait is bounded (see tc::mbar_wait).
#pragma once
#include "spectral_tc.cuh"

namespace tfno {
namespace tcg {

using namespace tc;

constexpr int kGemmThreads = 448;        // 14 warps
constexpr int kCH = 16;                  // channels per chunk
constexpr int kGemmStages = 4;           // two per half-team
template <int TN> struct GemmGeom {
    static constexpr int ROW_BYTES = TN * 8;                 // TN modes of one channel
    static constexpr int ROW_STRIDE = ROW_BYTES + 16;        // the 8 rows read by a quarter-warp cover all banks
    static constexpr int STAGE_BYTES = kCH * ROW_STRIDE;
};

struct CgemmTcParams {
    long long tiles;                     // M / TN
    int K;
    const float2* a; long long a_stride_k;       // A[m + k * a_stride_k]
    const float2* w; long long w_stride_k, w_stride_n;
    float2* c; long long c_stride_n;             // C[m + n * c_stride_n]
    float2 alpha;
    int accumulate;                      // 1: C += alpha A W (the second of two launches over the halves of K > 64)
    int* status;
};

template <int TN>
__host__ inline size_t cgemm_tc_smem_bytes() {
    size_t b = 0;
    b += (size_t)kGemmStages * GemmGeom<TN>::STAGE_BYTES;    // ring
    b += 2 * 2 * (size_t)(TN / 8) * s_sbo(4);                // two S chunk buffers (one per half-team), hi and lo each
    b += 2 * 64 * (size_t)TN * 4;                            // Re / Im planes
    b += 256;                                                // barriers, tmem base, abort flag
    return b + 1024;
}

template <int TN>
__global__ void __launch_bounds__(kGemmThreads, 1) cgemm_tc_kernel(CgemmTcParams p) {
    static_assert(TN == 64 || TN == 128, "tile of 64 or 128 modes");
    constexpr int R = 4;                          // lanes per channel row: lane r converts modes 64q + 16r .. +15, q < TN/64
    constexpr int CH = kCH;
    constexpr int PASSES = TN / 64;
    constexpr int kRowBytes = GemmGeom<TN>::ROW_BYTES, kRowStride = GemmGeom<TN>::ROW_STRIDE, kStageBytes = GemmGeom<TN>::STAGE_BYTES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int K = p.K;                            // a multiple of 8
    const int NC = (K + CH - 1) / CH;             // chunks per tile; a last chunk of 8 channels is padded:
    const int Kp = NC * CH;                       // zero weights, and ring rows no copy writes are zeroed once
    const int SBO = s_sbo(R), SBYTES = (TN / 8) * SBO;            // hi or lo array of one chunk buffer
    unsigned char* ring = base;
    unsigned char* sS = ring + kGemmStages * kStageBytes;           // [buffer 0: hi | lo][buffer 1: hi | lo]
    float* planes = reinterpret_cast<float*>(sS + 4 * SBYTES);      // [2][64][TN]
    uint64_t* bars = reinterpret_cast<uint64_t*>(planes + 2 * 64 * TN);
    constexpr int B_FULL = 0, B_EMPTY = 4, B_SFULL = 8, B_SEMPTY = 10, B_AFULL = 12, B_AEMPTY = 14, B_PFULL = 16, B_PEMPTY = 17,
                  B_COUNT = 18;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool is_compute = warp < 8;
    const bool is_conv = is_compute && !(warp & 1);
    const bool is_xfer = warp >= 8 && warp < 12;

    if (tid == 0) {
        for (int s = 0; s < kGemmStages; ++s) { mbar_init(bar(B_FULL + s), 1); mbar_init(bar(B_EMPTY + s), 2); }
        for (int h = 0; h < 2; ++h) { mbar_init(bar(B_SFULL + h), 2); mbar_init(bar(B_SEMPTY + h), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar(B_AFULL + b), 1); mbar_init(bar(B_AEMPTY + b), 4); }
        mbar_init(bar(B_PFULL), 4);
        mbar_init(bar(B_PEMPTY), 4);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (Kp != K) {
        for (int i = tid; i < kGemmStages * kStageBytes / 16; i += kGemmThreads) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0u, 0u, 0u, 0u);
        fence_async_smem();                       // before the copy engine writes other rows of the same stages
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t TM_WHI = 0, TM_WLO = 2 * Kp, TM_ACC = 4 * Kp;

    const long long first = blockIdx.x;
    const int n_it = first < p.tiles ? (int)((p.tiles - first + gridDim.x - 1) / gridDim.x) : 0;
    // chunk c of a tile belongs to half-team h = c & 1; tph[h] = chunks of half-team h per tile
    const int tph0 = (NC + 1) / 2, tph1 = NC / 2;

    // Weights (times alpha) into tensor memory; TMEM row i = 32 * (warp % 4) + lane; rows 0-63 produce
    // Re, rows 64-127 Im of output channel n = i & 63.  A thread needs eight adjacent channels of its n,
    // which in memory are 64 bytes every K*8 (or 8 bytes every N*8): read that way every warp-wide load
    // touches 32 lines, and four warps doing 2K such loads each made the set-up of a launch ~10 us.  So
    // all warps fetch the weights as contiguous runs with asynchronous 8-byte copies (one trip to memory)
    // into the S buffers and planes, which nothing uses yet, as [n][K channels + 16 bytes], and warps
    // 0-11 (three per TMEM quarter) convert from there.
    {
        // K <= 64 with 128-mode tiles, K <= 96 with 64-mode tiles (tensor memory: 4K + 2 TN <= 512 columns)
        static_assert(2 * 2 * (TN / 8) * s_sbo(4) + 2 * 64 * TN * 4 >= 64 * ((TN == 64 ? 96 : 64) * 8 + 16), "weight staging area");
        unsigned char* wst = sS;
        const int wrow = K * 8 + 16;
        const bool k_fast = p.w_stride_k == 1;
#pragma unroll 1
        for (int idx = tid; idx < 64 * K; idx += kGemmThreads) {
            const int kk = k_fast ? idx % K : idx >> 6, nn = k_fast ? idx / K : idx & 63;
            const float2* src = p.w + (long long)kk * p.w_stride_k + (long long)nn * p.w_stride_n;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(wst + nn * wrow + kk * 8)), "l"(src) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        __syncthreads();
        if (warp < 12) {
            const int i = 32 * (warp & 3) + lane, n = i & 63, im_row = i >> 6;
            const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16);
            for (int blk = warp >> 2; blk < Kp / 8; blk += 3) {     // eight channels c*CH + k0 .. +7
                const int c = (8 * blk) / CH, k0 = (8 * blk) % CH;
                const bool real = 8 * blk < K;                       // channels K .. Kp-1 get zero weights
                float2 wv[8];
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float4 t = real ? *reinterpret_cast<const float4*>(wst + n * wrow + (8 * blk + j) * 8) : make_float4(0.f, 0.f, 0.f, 0.f);
                    wv[j] = cmul(make_float2(t.x, t.y), p.alpha);
                    wv[j + 1] = cmul(make_float2(t.z, t.w), p.alpha);
                }
#pragma unroll
                for (int part = 0; part < 2; ++part) {
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // Re row: [ Wr | -Wi ],  Im row: [ Wi | Wr ]  against  S = [ Ar ; Ai ]
                        const float v = im_row ? (part ? wv[j].x : wv[j].y) : (part ? -wv[j].y : wv[j].x);
                        const float h = tf32_hi(v);
                        hi[j] = __float_as_uint(h);
                        lo[j] = __float_as_uint(tf32_hi(v - h));
                    }
                    const uint32_t col = (uint32_t)(c * 2 * CH + part * CH + k0);
                    TFNO_TMEM_ST8(trow + TM_WHI + col, hi);
                    TFNO_TMEM_ST8(trow + TM_WLO + col, lo);
                }
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (is_xfer) {
        // accumulator row i = (part, channel) of this thread -> Re / Im planes in shared memory
        const int i = tid - 256;
        const int q = warp & 3;
        float* prow = planes + (i >> 6) * (64 * TN) + (i & 63) * TN;
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const int buf = it & 1;
            ok = mbar_wait(bar(B_AFULL + buf), (it >> 1) & 1, abort_flag, p.status, 71, kHelperIdleNs);
            if (ok) ok = mbar_wait(bar(B_PEMPTY), (it & 1) ^ 1, abort_flag, p.status, 72, kHelperIdleNs);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + TM_ACC + TN * buf;
#pragma unroll 1
            for (int c0 = 0; c0 < TN; c0 += 8) {
                uint32_t acc[8];
                TFNO_TMEM_LD8(taddr + c0, acc);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int cc = c0 >> 2;
                *reinterpret_cast<uint4*>(prow + plane_chunk(i & 63, cc) * 4) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
                *reinterpret_cast<uint4*>(prow + plane_chunk(i & 63, cc + 1) * 4) = make_uint4(acc[4], acc[5], acc[6], acc[7]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(bar(B_AEMPTY + buf)); mbar_arrive(bar(B_PFULL)); }
        }
    } else if (warp == 12) {
        // producer: chunk c of tile `it` goes to stage h + 2*(j & 1), j = chunks half-team h has had before
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const long long tile = first + (long long)it * gridDim.x;
            for (int c = 0; c < NC && ok; ++c) {
                const int h = c & 1;
                const uint32_t j = (uint32_t)it * (uint32_t)(h ? tph1 : tph0) + (uint32_t)(c >> 1);
                const int s = h + 2 * (int)(j & 1);
                ok = __all_sync(0xffffffffu, mbar_wait(bar(B_EMPTY + s), ((j >> 1) & 1) ^ 1, abort_flag, p.status, 73, kHelperIdleNs));
                if (!ok) break;
                const int valid = (K - c * CH < CH) ? K - c * CH : CH;      // channels of this chunk
                if (lane == 0) mbar_arrive_expect_tx(bar(B_FULL + s), valid * kRowBytes);
                __syncwarp();
                if (lane < valid) {
                    const float2* src = p.a + (long long)(c * CH + lane) * p.a_stride_k + tile * TN;
                    bulk_load(smem_u32(ring + s * kStageBytes + lane * kRowStride), src, kRowBytes, bar(B_FULL + s));
                }
            }
        }
    } else if (warp == 13 && lane == 0) {
        const uint32_t idesc = make_idesc_tf32(TN);
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const int buf = it & 1;
            const uint32_t d_tmem = tmem + TM_ACC + TN * buf;
            for (int c = 0; c < NC && ok; ++c) {
                const int h = c & 1;
                const uint32_t j = (uint32_t)it * (uint32_t)(h ? tph1 : tph0) + (uint32_t)(c >> 1);
                const int sb = h;
                ok = mbar_wait(bar(B_SFULL + sb), j & 1, abort_flag, p.status, 74);
                if (ok && c == 0) ok = mbar_wait(bar(B_AEMPTY + buf), ((it >> 1) & 1) ^ 1, abort_flag, p.status, 75, kHelperIdleNs);
                if (!ok) break;
                tc_fence_after();
                const uint32_t s_hi = smem_u32(sS) + (uint32_t)(2 * sb * SBYTES), s_lo = s_hi + SBYTES;
                constexpr int KSTEPS = 2 * CH / 8;
#pragma unroll 1
                for (int jj = 0; jj < KSTEPS; ++jj) {
                    const int ks = c * KSTEPS + jj;
                    const uint64_t dhi = make_kmajor_desc(s_hi + 2 * jj * kLBO, kLBO, SBO);
                    const uint64_t dlo = make_kmajor_desc(s_lo + 2 * jj * kLBO, kLBO, SBO);
                    const uint32_t a_hi = tmem + TM_WHI + 8 * ks, a_lo = tmem + TM_WLO + 8 * ks;
                    umma_tf32_ts(d_tmem, a_hi, dhi, idesc, (c | jj) ? 1u : 0u);
                    umma_tf32_ts(d_tmem, a_lo, dhi, idesc, 1u);
                    umma_tf32_ts(d_tmem, a_hi, dlo, idesc, 1u);
                }
                umma_commit(bar(B_SEMPTY + sb));
                if (c == NC - 1) umma_commit(bar(B_AFULL + buf));
            }
        }
    } else if (is_conv) {
        // ---------------- convert: ring rows -> S (tf32 hi / lo, K-major) ----------------
        constexpr int GPW = 32 / R;
        const int g = lane % GPW, r = lane / GPW;
        const int half = (warp >> 2) & 1, wl = (warp >> 1) & 1;
        const int kl = wl * GPW + g;                      // channel inside the chunk
        const int tph = half ? tph1 : tph0;
        bool alive = true;
        for (int it = 0; it < n_it && alive; ++it) {
            for (int t = 0; t < tph && alive; ++t) {
                const uint32_t j = (uint32_t)it * (uint32_t)tph + (uint32_t)t;
                const int s = half + 2 * (int)(j & 1);
                alive = __all_sync(0xffffffffu, mbar_wait(bar(B_FULL + s), (j >> 1) & 1, abort_flag, p.status, 76));
                if (!alive) break;
                const float4* srow = reinterpret_cast<const float4*>(ring + s * kStageBytes + kl * kRowStride + r * 128);
                float4 q[8 * PASSES];
#pragma unroll
                for (int pq = 0; pq < PASSES; ++pq)
#pragma unroll
                    for (int i = 0; i < 8; ++i) q[8 * pq + i] = srow[32 * pq + i];       // 512 bytes per 64 modes
                __threadfence_block();          // the loads have returned before the stage is handed back
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_EMPTY + s));
                // this half-team's S buffer is free once the MMAs of its previous chunk have completed
                alive = __all_sync(0xffffffffu, mbar_wait(bar(B_SEMPTY + half), (j & 1) ^ 1, abort_flag, p.status, 77));
                if (!alive) break;
                const int kk_re = kl, kk_im = CH + kl;
                unsigned char* sbuf = sS + 2 * half * SBYTES;
                unsigned char* hi_re = sbuf + (kk_re >> 2) * kLBO + (kk_re & 3) * 4;
                unsigned char* hi_im = sbuf + (kk_im >> 2) * kLBO + (kk_im & 3) * 4;
#pragma unroll
                for (int i = 0; i < 8 * PASSES; ++i) {
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        // the four lanes of a channel store modes 16 apart (two 8-mode groups): with
                        // SBO = 16 mod 64 bytes the warp's 32 stores fall into 32 banks
                        const int m = 64 * (i >> 3) + 16 * r + 2 * (i & 7) + e;
                        const int off = (m >> 3) * SBO + (m & 7) * 16;
                        const float xr = e ? q[i].z : q[i].x, xi = e ? q[i].w : q[i].y;
                        const float hr = tf32_hi(xr), hi = tf32_hi(xi);
                        *reinterpret_cast<float*>(hi_re + off) = hr;
                        *reinterpret_cast<float*>(hi_re + SBYTES + off) = xr - hr;
                        *reinterpret_cast<float*>(hi_im + off) = hi;
                        *reinterpret_cast<float*>(hi_im + SBYTES + off) = xi - hi;
                    }
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_SFULL + half));
            }
        }
    } else if (is_compute) {
        // ---------------- write: planes -> C rows ----------------
        const int qi = warp >> 1;                         // 0..3: output channels 16*qi .. 16*qi+15
        bool alive = true;
        for (int it = 0; it < n_it && alive; ++it) {
            const long long tile = first + (long long)it * gridDim.x;
            alive = __all_sync(0xffffffffu, mbar_wait(bar(B_PFULL), it & 1, abort_flag, p.status, 78));
            if (!alive) break;
#pragma unroll 4
            for (int i = 0; i < 16; ++i) {
                const int n = qi * 16 + i;
                float2* crow = p.c + (long long)n * p.c_stride_n + tile * TN;
#pragma unroll
                for (int pq = 0; pq < PASSES; ++pq) {
                    const int off = n * TN + plane_chunk(n, 16 * pq + (lane >> 1)) * 4 + (lane & 1) * 2;
                    const float2 re = *reinterpret_cast<const float2*>(planes + off);
                    const float2 im = *reinterpret_cast<const float2*>(planes + 64 * TN + off);
                    float4 o = make_float4(re.x, im.x, re.y, im.y);
                    if (p.accumulate) {
                        const float4 prev = *reinterpret_cast<const float4*>(crow + 64 * pq + 2 * lane);
                        o.x += prev.x; o.y += prev.y; o.z += prev.z; o.w += prev.w;
                    }
                    *reinterpret_cast<float4*>(crow + 64 * pq + 2 * lane) = o;
                }
            }
            // release orders this lane's plane reads before the arrive, __syncwarp those of the others
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_PEMPTY));
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace tcg
}  // namespace tfno

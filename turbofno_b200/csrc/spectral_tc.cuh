// Fused 1D spectral convolution for sm_100a with the channel contraction on the 5th-generation
// tensor cores (tcgen05 + TMEM) and bulk-copy (TMA engine) input staging.
// Same operator as spectral_tile_kernel<R,true,true,1>
// (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused_fft_cgemm_ifft_7.cuh:9-222 in the
// reference), restricted to N = 64 output channels, K <= 64, DY in {128, 256}.
//
// One persistent CTA per SM, 320 threads in four roles that overlap through mbarriers:
//
//   warp 8      producer   cp.async.bulk of whole input rows (DY*8 bytes each) into a 3-stage
//                          shared-memory ring, CH = 64/R channels per stage
//   warps 0-3   forward    two half-teams of 64 threads; a half-team takes one ring stage, each
//                          group of R lanes transforms one channel (64-point register FFT +
//                          reduce-scatter), splits the 64 kept modes into tf32 hi/lo parts and
//                          stores them as the B operand S[mode][kk] (K-major core matrices)
//   warp 9      MMA        one thread issues tcgen05.mma kind::tf32:
//                              D[128 x 64 modes] += Wt[128 x 8] * S[8 x 64]
//                          Wt (the weights, rows 0-63 -> Re, 64-127 -> Im of output channel n,
//                          columns kk = (chunk, Re|Im part, channel)) lives in tensor memory for
//                          the whole kernel; fp32 accuracy comes from three tf32 products
//                          (hi*hi + lo*hi + hi*lo).  Accumulators are double-buffered in TMEM.
//   warps 4-7   inverse    tcgen05.ld of one accumulator row per thread -> Re/Im planes in shared
//                          memory -> groups of R lanes run the zero-padded inverse transform of
//                          one output channel and store it.
//
// Every wait is bounded: a wait that runs out sets `*status` and an abort flag, all roles leave
// their loops, tensor memory is released, and the kernel returns.
#pragma once
#include <cstdint>
#include "fft64.cuh"

namespace tfno {
namespace tc {

constexpr int kTcThreads = 320;
constexpr int kStages = 3;
constexpr int kLBO = 144;                   // bytes between K-adjacent core matrices of S (128 + 16 pad)
constexpr uint32_t kSpinLimit = 1u << 22;   // polls (with back-off) before a wait gives up

struct TcParams {
    long long rows;
    int K;
    const float2* x; long long x_stride_row, x_stride_k;
    const float2* w; long long w_stride_k, w_stride_n;
    float2* y; long long y_stride_row, y_stride_n;
    float2 inv_gain;
    int conj_inverse;
    int* status;                // device-visible word; 0 = ok
};

// SBO: bytes between 8-mode groups of S: all K chunks, rounded up to 64 (mod 256) so that lanes
// holding modes 16 apart fall into different banks
__host__ __device__ inline int s_sbo(int K) { int span = (2 * K / 4) * kLBO; return ((span + 255) / 256) * 256 + 64; }
__host__ __device__ inline int s_bytes(int K) { return 8 * s_sbo(K); }           // one of the hi / lo arrays

template <int R> struct Geometry {
    static constexpr int DY = 64 * R;
    static constexpr int CH = 64 / R;                       // channels per chunk (= per ring stage)
    static constexpr int ROW_BYTES = DY * 8;
    static constexpr int ROW_STRIDE = ROW_BYTES + 16;       // pad: 8 rows x 16 B tile the 128-byte bank window
    static constexpr int STAGE_BYTES = CH * ROW_STRIDE;
    static constexpr int KSTEPS_PER_CHUNK = 2 * CH / 8;
};

template <int R>
__host__ inline size_t tc_smem_bytes(int K) {
    using G = Geometry<R>;
    size_t b = 0;
    b += (size_t)kStages * G::STAGE_BYTES;        // ring
    b += 2 * (size_t)s_bytes(K);                  // S hi, S lo
    b += 2 * 64 * 256;                            // Re / Im planes [64 channels][64 modes] fp32
    b += 2 * (size_t)R * 64 * 8;                  // twiddle tables
    b += 256;                                     // barriers, tmem base, abort flag
    return b + 1024;                              // slack for 1024-byte alignment of the base
}

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the barrier did not complete within the limit or another role
// has already given up; the caller leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if (spin > 64) {
            if (*abort_flag) return false;
            __nanosleep(spin > 4096 ? 256 : 32);
        }
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}
__device__ __forceinline__ void bulk_load(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void named_barrier(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// barrier over `nthreads` threads that also ORs a predicate: every participant gets the same answer
__device__ __forceinline__ bool named_barrier_any(int id, int nthreads, bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, %2, %3, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"((uint32_t)pred), "r"(id), "r"(nthreads) : "memory");
    return r != 0;
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem desc], tf32 inputs, fp32 accumulate
__device__ __forceinline__ void umma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// shared-memory matrix descriptor: K-major, no swizzle, 8-row x 16-byte core matrices
__device__ __forceinline__ uint64_t make_kmajor_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3FFF);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;       // descriptor version of this architecture
    return d;
}
// instruction descriptor: D fp32, A and B tf32, both K-major, M = 128, N = n
__device__ __forceinline__ uint32_t make_idesc_tf32(int n) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ float tf32_hi(float v) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    return __uint_as_float(u);
}

#define TFNO_TMEM_ST16(taddr, r, o)                                                                                      \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"   \
                 ::"r"(taddr), "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]),   \
                 "r"(r[o + 6]), "r"(r[o + 7]), "r"(r[o + 8]), "r"(r[o + 9]), "r"(r[o + 10]), "r"(r[o + 11]),               \
                 "r"(r[o + 12]), "r"(r[o + 13]), "r"(r[o + 14]), "r"(r[o + 15]) : "memory")
#define TFNO_TMEM_LD16(taddr, r, o)                                                                                      \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"   \
                 : "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]),         \
                   "=r"(r[o + 6]), "=r"(r[o + 7]), "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]),       \
                   "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15])                                      \
                 : "r"(taddr) : "memory")

// plane[part][channel n][mode m] fp32, 16-byte chunks XOR-swizzled with the channel
__device__ __forceinline__ int plane_chunk(int n, int c) { return (c & ~7) | ((c & 7) ^ (n & 7)); }

// ---------------------------------------------------------------------------------------------
template <int R>
__global__ void __launch_bounds__(kTcThreads, 1) spectral_tc_kernel(TcParams p) {
    using G = Geometry<R>;
    constexpr int CH = G::CH;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int K = p.K;
    const int NC = K / CH;                            // chunks per row
    const int SBO = s_sbo(K), SBYTES = s_bytes(K);
    unsigned char* ring = base;
    unsigned char* sS = ring + kStages * G::STAGE_BYTES;            // [hi | lo]
    float* planes = reinterpret_cast<float*>(sS + 2 * SBYTES);      // [2][64][64]
    float2* twF = reinterpret_cast<float2*>(planes + 2 * 64 * 64);
    float2* twI = twF + R * 64;
    uint64_t* bars = reinterpret_cast<uint64_t*>(twI + R * 64);
    // barrier indices
    constexpr int B_FULL = 0, B_EMPTY = kStages, B_SFULL = 2 * kStages, B_SEMPTY = B_SFULL + 8, B_AFULL = B_SEMPTY + 8,
                  B_AEMPTY = B_AFULL + 2, B_COUNT = B_AEMPTY + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---------------- set-up ----------------
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar(B_FULL + s), 1); mbar_init(bar(B_EMPTY + s), 2); }
        for (int c = 0; c < 8; ++c) { mbar_init(bar(B_SFULL + c), 2); mbar_init(bar(B_SEMPTY + c), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar(B_AFULL + b), 1); mbar_init(bar(B_AEMPTY + b), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 9) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fill_forward_table<R>(twF, tid, kTcThreads);
    fill_inverse_table<R>(twI, tid, kTcThreads, p.inv_gain, p.conj_inverse != 0);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t TM_WHI = 0, TM_WLO = 2 * K, TM_ACC = 4 * K;        // column offsets; accumulators 2 x 64 columns

    // weights into tensor memory: thread i of warps 4-7 owns row i = (part_out, n)
    if (warp >= 4 && warp < 8) {
        const int i = tid - 128, n = i & 63, im_row = i >> 6;
        const uint32_t trow = tmem + ((uint32_t)((warp & 3) * 32) << 16);
        for (int c = 0; c < NC; ++c) {
            for (int part = 0; part < 2; ++part) {
                for (int k0 = 0; k0 < CH; k0 += 16) {
                    uint32_t hi[16], lo[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int k = c * CH + k0 + j;
                        const float2 wv = __ldg(p.w + (long long)k * p.w_stride_k + (long long)n * p.w_stride_n);
                        // Re row: [ Wr | -Wi ],  Im row: [ Wi | Wr ]  against  S = [ Xr ; Xi ]
                        float v = im_row ? (part ? wv.x : wv.y) : (part ? -wv.y : wv.x);
                        float h = tf32_hi(v);
                        hi[j] = __float_as_uint(h);
                        lo[j] = __float_as_uint(tf32_hi(v - h));
                    }
                    const uint32_t col = (uint32_t)(c * 2 * CH + part * CH + k0);
                    TFNO_TMEM_ST16(trow + TM_WHI + col, hi, 0);
                    TFNO_TMEM_ST16(trow + TM_WLO + col, lo, 0);
                }
            }
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    const long long first = blockIdx.x;
    const int n_it = first < p.rows ? (int)((p.rows - first + gridDim.x - 1) / gridDim.x) : 0;

    if (warp == 8) {
        // ======================= producer =======================
        long long L = 0;
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const long long row = first + (long long)it * gridDim.x;
            for (int c = 0; c < NC && ok; ++c, ++L) {
                const int s = (int)(L % kStages);
                const uint32_t u = (uint32_t)(L / kStages);
                ok = __all_sync(0xffffffffu, mbar_wait(bar(B_EMPTY + s), (u & 1) ^ 1, abort_flag, p.status, 11));
                if (!ok) break;
                if (lane == 0) mbar_arrive_expect_tx(bar(B_FULL + s), CH * G::ROW_BYTES);
                __syncwarp();
                for (int j = lane; j < CH; j += 32) {
                    const float2* src = p.x + row * p.x_stride_row + (long long)(c * CH + j) * p.x_stride_k;
                    bulk_load(smem_u32(ring + s * G::STAGE_BYTES + j * G::ROW_STRIDE), src, G::ROW_BYTES, bar(B_FULL + s));
                }
            }
        }
    } else if (warp == 9) {
        // ======================= MMA issuer =======================
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(64);
            const uint32_t s_hi = smem_u32(sS), s_lo = s_hi + SBYTES;
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int buf = it & 1;
                const uint32_t d_tmem = tmem + TM_ACC + 64 * buf;
                for (int c = 0; c < NC && ok; ++c) {
                    ok = mbar_wait(bar(B_SFULL + c), it & 1, abort_flag, p.status, 21);
                    if (ok && c == 0) ok = mbar_wait(bar(B_AEMPTY + buf), ((it >> 1) & 1) ^ 1, abort_flag, p.status, 22);
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll 1
                    for (int j = 0; j < G::KSTEPS_PER_CHUNK; ++j) {
                        const int ks = c * G::KSTEPS_PER_CHUNK + j;               // global k-step: kk in [8ks, 8ks+8)
                        const uint64_t dhi = make_kmajor_desc(s_hi + 2 * ks * kLBO, kLBO, SBO);
                        const uint64_t dlo = make_kmajor_desc(s_lo + 2 * ks * kLBO, kLBO, SBO);
                        const uint32_t a_hi = tmem + TM_WHI + 8 * ks, a_lo = tmem + TM_WLO + 8 * ks;
                        umma_tf32_ts(d_tmem, a_hi, dhi, idesc, (c | j) ? 1u : 0u);
                        umma_tf32_ts(d_tmem, a_lo, dhi, idesc, 1u);
                        umma_tf32_ts(d_tmem, a_hi, dlo, idesc, 1u);
                    }
                    umma_commit(bar(B_SEMPTY + c));
                }
                if (ok) umma_commit(bar(B_AFULL + buf));
            }
        }
    } else if (warp < 4) {
        // ======================= forward transform =======================
        const int half = warp >> 1;                       // half-team: chunks c = half, half+2, ...
        const int wl = warp & 1;                          // warp inside the half-team
        constexpr int GPW = 32 / R;                       // channels per warp
        const int g = lane % GPW, r = lane / GPW;         // lane = g + GPW*r: the R lanes of a group are GPW apart
        const int kl = wl * GPW + g;                      // channel inside the chunk
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            for (int c = half; c < NC && ok; c += 2) {
                const long long L = (long long)it * NC + c;
                const int s = (int)(L % kStages);
                const uint32_t u = (uint32_t)(L / kStages);
                ok = __all_sync(0xffffffffu, mbar_wait(bar(B_FULL + s), u & 1, abort_flag, p.status, 31));
                if (!ok) break;
                float2 v[64];
                const float2* srow = reinterpret_cast<const float2*>(ring + s * G::STAGE_BYTES + kl * G::ROW_STRIDE);
#pragma unroll
                for (int n = 0; n < 64; ++n) v[n] = srow[R * n + r];
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_EMPTY + s));
                // 64-point transforms + twiddles, then the reduce-scatter over the R lanes (GPW apart)
                forward_local<R>(v, twF + 64 * r, r);
#pragma unroll
                for (int j = 0; j < 32; ++j) v[slot(j)] = cadd(v[slot(j)], shfl_xor2(v[slot(32 + j)], (R >> 1) * GPW));
                if constexpr (R >= 4) exchange_round<16>(v, (R >> 2) * GPW, (r & (R >> 2)) != 0);
                // lane r now holds modes 64/R*r + j, j < 64/R, in v[slot(j)]
                ok = __all_sync(0xffffffffu, mbar_wait(bar(B_SEMPTY + c), (it & 1) ^ 1, abort_flag, p.status, 32));
                if (!ok) break;
                constexpr int PER = 64 / R;
                const int kk_re = c * 2 * CH + kl, kk_im = kk_re + CH;
                unsigned char* hi_re = sS + (kk_re >> 2) * kLBO + (kk_re & 3) * 4;
                unsigned char* hi_im = sS + (kk_im >> 2) * kLBO + (kk_im & 3) * 4;
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int m = PER * r + j;
                    const int off = (m >> 3) * SBO + (m & 7) * 16;
                    const float xr = v[slot(j)].x, xi = v[slot(j)].y;
                    const float hr = tf32_hi(xr), hi = tf32_hi(xi);
                    *reinterpret_cast<float*>(hi_re + off) = hr;
                    *reinterpret_cast<float*>(hi_re + SBYTES + off) = xr - hr;
                    *reinterpret_cast<float*>(hi_im + off) = hi;
                    *reinterpret_cast<float*>(hi_im + SBYTES + off) = xi - hi;
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_SFULL + c));
            }
        }
    } else {
        // ======================= inverse transform =======================
        const int i = tid - 128;                          // accumulator row: part = i >> 6, channel n = i & 63
        const int q = warp & 3;
        constexpr int GROUPS = 128 / R;                   // channels per pass
        constexpr int GPW = 32 / R;
        const int g = lane % GPW, j1 = lane / GPW;
        const int ch_in_pass = q * GPW + g;
        bool ok = true;
        (void)ok;
        for (int it = 0; it < n_it; ++it) {
            const long long row = first + (long long)it * gridDim.x;
            const int buf = it & 1;
            ok = mbar_wait(bar(B_AFULL + buf), (it >> 1) & 1, abort_flag, p.status, 41);
            // one answer for the whole team: nobody may be left alone at a later named barrier
            if (named_barrier_any(1, 128, !ok)) break;
            tc_fence_after();
            {
                uint32_t acc[64];
                const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + TM_ACC + 64 * buf;
                TFNO_TMEM_LD16(taddr + 0, acc, 0);
                TFNO_TMEM_LD16(taddr + 16, acc, 16);
                TFNO_TMEM_LD16(taddr + 32, acc, 32);
                TFNO_TMEM_LD16(taddr + 48, acc, 48);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_AEMPTY + buf));
                float* prow = planes + (i >> 6) * 4096 + (i & 63) * 64;
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    *reinterpret_cast<uint4*>(prow + plane_chunk(i & 63, c) * 4) =
                        make_uint4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
            }
            named_barrier(2, 128);
#pragma unroll 1
            for (int n0 = 0; n0 < 64; n0 += GROUPS) {
                const int n = n0 + ch_in_pass;
                float2 v[64];
                const float* pre = planes + n * 64;
                const float* pim = planes + 4096 + n * 64;
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float4 a = *reinterpret_cast<const float4*>(pre + plane_chunk(n, c) * 4);
                    const float4 b = *reinterpret_cast<const float4*>(pim + plane_chunk(n, c) * 4);
                    v[4 * c] = make_float2(a.x, b.x); v[4 * c + 1] = make_float2(a.y, b.y);
                    v[4 * c + 2] = make_float2(a.z, b.z); v[4 * c + 3] = make_float2(a.w, b.w);
                }
                if (n0 + GROUPS >= 64) named_barrier(3, 128);      // planes may be overwritten from here on
                if (p.conj_inverse) inverse_pad_lane<+1>(v, twI + 64 * j1);
                else inverse_pad_lane<-1>(v, twI + 64 * j1);
                float2* dst = p.y + row * p.y_stride_row + (long long)n * p.y_stride_n;
#pragma unroll
                for (int j2 = 0; j2 < 64; ++j2) dst[R * j2 + j1] = v[slot(j2)];
            }
        }
    }

    // ---------------- teardown ----------------
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace tc
}  // namespace tfno

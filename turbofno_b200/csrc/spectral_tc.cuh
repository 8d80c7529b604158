// Fused 1D spectral convolution for sm_100a with the channel contraction on the 5th-generation
// tensor cores (tcgen05 + TMEM) and bulk-copy (TMA engine) staging of input and output rows.
// Same operator as spectral_tile_kernel<R,true,true,1>
// (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused_fft_cgemm_ifft_7.cuh:9-222 in the
// reference), restricted to N = 64 output channels, K a multiple of 4 up to 96 (the launcher sends
// multiples of 8; a last chunk of fewer than CH channels gets zero weights), DY in {128, 256,
// 512, 1024}.  With `accumulate` the result is ADDED to y (the copy engine's reduce-add): the
// launcher covers K up to 192 with two launches over the halves of the channels.
//
// One persistent CTA per SM, 768 threads in six warpgroups.  The transforms run on the 32-point
// register FFT (fft32.cuh): a signal is spread over R = DY/32 lanes, a thread holds 32 samples, so
// a compute thread needs 104 registers and FOUR compute warps share a scheduler (the earlier
// 64-point design had two at 216 registers and was bound by exposed latency: issue slots 37 % used).
// setmaxnreg moves registers from the two helper warpgroups to the four compute warpgroups.
//
//   warps 0,2,..,14  forward  two half-teams {0,2,4,6} and {8,10,12,14}.  Input rows (DY*8 bytes
//                             each) arrive by cp.async.bulk in a 2-stage shared-memory ring,
//                             CH = 128/R channels per stage; a half-team takes one stage, each
//                             group of R lanes transforms one channel (32-point register FFT +
//                             exchange rounds), splits the 64 kept modes into tf32 hi/lo parts and
//                             stores them as the B operand S[mode][kk] (K-major core matrices) in
//                             the half-team's own S buffer.
//   warps 1,3,..,15  inverse  groups of R lanes read one output channel's 64 modes from the Re/Im
//                             planes and run the zero-padded inverse transform; from DY = 256 up
//                             the rows are staged in shared memory and leave through the copy
//                             engine (DY = 256: the four rows of a task as one tiled copy over a
//                             tensor map of y), at DY = 128 the lanes store directly.  The inverse
//                             tasks of a CTA's LAST row are shared with the forward warps.
//   warps 16-19      hand-off tcgen05.ld of one accumulator row per thread -> Re/Im planes in
//                             shared memory (a warp may only touch its own quarter of tensor
//                             memory, so this needs four warps with distinct warp%4).
//   warp 20          producer one thread arms a ring stage, CH lanes issue the bulk copies.
//   warp 21          MMA      one thread issues tcgen05.mma kind::tf32, in chunk order:
//                                 D[128 x 64 modes] += Wt[128 x 8] * S[8 x 64]
//                             Wt (the weights, rows 0-63 -> Re, 64-127 -> Im of output channel n,
//                             columns kk = (chunk, channel, Re|Im part)) lives in tensor memory for
//                             the whole kernel; fp32 accuracy comes from three tf32 products
//                             (hi*hi + lo*hi + hi*lo).  Accumulators are double-buffered in TMEM.
//
// A scheduler partition hosts warps w, w+4, ...: its four compute warps have the same role, and
// both roles funnel through ONE copy of the unrolled 32-point transform (the inverse is computed
// as swap(FFT(swap(u)))); together this keeps the instruction stream a partition fetches short.
//
// Every wait is bounded: a wait that runs out sets `*status` and an abort flag, all roles leave
// their loops, outstanding copies and MMAs are drained, tensor memory is released, and the kernel
// returns.
#pragma once
#include <cstdint>
#include <type_traits>
#include <cuda.h>          // CUtensorMap (types only: the encoder is fetched from the runtime)
#include "fft32.cuh"

namespace tfno {
namespace tc {

constexpr int kTcThreads = 768;             // 6 warpgroups, see the role table above
constexpr int kComputeWarps = 16;           // 8 forward + 8 inverse
constexpr int kHalfWarps = 4;               // forward warps per half-team
constexpr int kInvWarps = 8;
// setmaxnreg only moves registers inside the pool the CTA got at launch (threads x registers per
// thread at launch: 768 x 80), and an increase that the pool cannot cover blocks for ever.
constexpr int kLaunchRegs = 80;             // what ptxas reports for __launch_bounds__(768, 1)
constexpr int kComputeRegs = 104;
constexpr int kHelperRegs = 32;
static_assert(512 * kComputeRegs + 256 * kHelperRegs <= kTcThreads * kLaunchRegs, "register pool of the CTA");
constexpr int kStages = 2;                  // ring stages: one in flight per forward half-team
constexpr int kLBO = 144;                   // bytes between K-adjacent core matrices of S (128 + 16 pad)
constexpr uint32_t kSpinLimit = 1u << 22;   // polls (with back-off) before a wait gives up
constexpr unsigned long long kWaitLimitNs = 1000000000ull;   // and wall-clock limit of one wait: 1 s
#ifndef TFNO_HELPER_IDLE_NS
#define TFNO_HELPER_IDLE_NS 200
#endif
constexpr unsigned kHelperIdleNs = TFNO_HELPER_IDLE_NS;   // sleep between polls of the helper warps

#ifdef TFNO_TC_TRACE
#define TFNO_TRACE_DECL long long tr_wait[11] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}; long long tr_t0 = clock64(); long long tr_mark = 0;
#define TFNO_TRACE_MARK() tr_mark = clock64()
#define TFNO_TRACE_STEP(slot, expr) [&]() { bool r_ = (expr); long long n_ = clock64(); tr_wait[slot] += n_ - tr_mark; tr_mark = n_; return r_; }()
#define TFNO_TRACE_SINCE(slot) do { long long n_ = clock64(); tr_wait[slot] += n_ - tr_mark; tr_mark = n_; } while (0)
#define TFNO_TRACE_WAIT(slot, expr) [&]() { long long t_ = clock64(); bool r_ = (expr); tr_wait[slot] += clock64() - t_; return r_; }()
#define TFNO_TRACE_FLUSH() if (lane == 0 && p.trace && warp < 24) { long long* d_ = p.trace + ((long long)blockIdx.x * 24 + warp) * 12; d_[0] = clock64() - tr_t0; for (int i_ = 0; i_ < 11; ++i_) d_[1 + i_] = tr_wait[i_]; }
#else
#define TFNO_TRACE_DECL
#define TFNO_TRACE_MARK()
#define TFNO_TRACE_SINCE(slot)
#define TFNO_TRACE_STEP(slot, expr) (expr)
#define TFNO_TRACE_WAIT(slot, expr) (expr)
#define TFNO_TRACE_FLUSH()
#endif

struct TcParams {
    long long rows;
    int K;
    const float2* x; long long x_stride_row, x_stride_k;
    const float2* w; long long w_stride_k, w_stride_n;
    float2* y; long long y_stride_row, y_stride_n;
    float2 inv_gain;
    int conj_inverse;
    int* status;                // device-visible word; 0 = ok
    long long* trace;           // optional per-warp cycle counters (builds with TFNO_TC_TRACE only)
    // Tiled view of y as [channel][row][DY] 8-byte elements, box = {DY, 1, channels of one inverse
    // warp}: with it an inverse warp hands all its output rows of a task to the copy engine in ONE
    // instruction instead of one per row (each costs the issuing warp ~175 cycles).  DY = 256 only
    // (a box is at most 256 elements wide); 0 = not available, the rows leave one by one.
    int use_ymap;
    // 1: y += result instead of y = result (the copy engine adds: cp.reduce.async.bulk .add.f32).  This
    // is how K > 96 runs: the channels are split into two launches, the second accumulating.  The
    // tiled copy is not used then (its map has 8-byte elements; a float map's box could hold only
    // half a row).
    int accumulate;
    alignas(64) CUtensorMap ymap;
};

// SBO: bytes between 8-mode groups of the B operand S.  The contraction kernel of compact spectra
// (cgemm_tc.cuh) stores 4-byte elements and uses s_sbo(4); the fused kernel stores the Re and Im
// parts of a channel as one 8-byte element (column kk = 2*channel + part) and uses s_sbo_fused.
__host__ __device__ constexpr int s_sbo(int R64) {
    const int span = (2 * (64 / R64) / 4) * kLBO;           // one chunk: CH channels, Re and Im rows
    return ((span + 63) / 64) * 64 + 16;
}
// R = DY/32 lanes per signal (adjacent lanes: lane = r + R*g), CH = 128/R channels per chunk.  A
// half-warp's 8-byte stores (16/R channels, R lanes each 64/R modes apart) must cover all 32 banks:
//   R = 8: two channels give {0,8} bytes, lanes r, r+1 are ONE mode group apart   -> SBO = 16 mod 128
//   R = 4: four channels give 32 bytes, lanes r, r+1 are TWO mode groups apart    -> 2*SBO = 32 mod 128
// both hold for a span that is a multiple of 64, plus 16.
__host__ __device__ constexpr int s_sbo_fused(int R) {
    const int span = (2 * (128 / R) / 4) * kLBO;
    return ((span + 63) / 64) * 64 + 16;
}
__host__ __device__ constexpr int s_bytes(int R) { return 8 * s_sbo_fused(R); }   // the hi or the lo array of one chunk buffer

template <int R> struct Geometry {
    static constexpr int DY = 32 * R;
    static constexpr int GPW = 32 / R;                      // groups (channels) per warp
    static constexpr int CH = kHalfWarps * GPW;             // channels per chunk (= per ring stage)
    static constexpr int ROW_BYTES = DY * 8;
    static constexpr int ROW_STRIDE = ROW_BYTES + 8 * R;    // pad: the 16/R rows a half-warp reads (8R bytes each) tile the 128-byte bank window
    static constexpr int STAGE_BYTES = CH * ROW_STRIDE;
    static constexpr int KSTEPS_PER_CHUNK = 2 * CH / 8;
    // Output rows are staged in shared memory and leave through the bulk-copy engine when there is
    // room (DY >= 256); at DY = 128 the S buffers are twice as large and the lanes store directly.
    static constexpr bool STAGED_OUT = (R >= 8);
    static constexpr int OUT_ROWS = GPW;                    // output rows staged per inverse warp and task
    static constexpr int OUT_STRIDE = ROW_BYTES + 8 * R;    // padded like the input rows
    static constexpr bool TENSOR_OUT = (R == 8);            // all rows of a task in one tiled copy
    static constexpr int OUT_BYTES = STAGED_OUT ? OUT_ROWS * OUT_STRIDE : 0;   // per inverse warp
};

template <int R>
__host__ inline size_t tc_smem_bytes(int K) {
    using G = Geometry<R>;
    size_t b = 0;
    b += (size_t)kStages * G::STAGE_BYTES;        // ring
    (void)K;
    b += 2 * 2 * (size_t)s_bytes(R);              // two chunk buffers of S, hi and lo each
    b += (size_t)kInvWarps * G::OUT_BYTES;        // output staging, one per inverse warp
    b += 2 * 64 * 256;                            // Re / Im planes [64 channels][64 modes] fp32
    b += 2 * (size_t)R * 32 * 8;                  // twiddle tables
    b += 512;                                     // barriers, tmem base, abort flag
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
// `idle_ns` > 0 marks a helper warp: it sleeps that long between polls from the first miss on, so
// that its polling does not take issue slots from the compute warps of its scheduler partition.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code,
                                          unsigned idle_ns = 0) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 1023) == 1023) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) break;
        }
        if (idle_ns) {
            __nanosleep(idle_ns);
            if ((spin & 15) == 15 && *abort_flag) return false;
        } else if (spin > 64) {
            if (*abort_flag) return false;
            __nanosleep(spin > 4096 ? 256 : 32);
        }
    }
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, code);
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

#define TFNO_TMEM_ST8(taddr, r)                                                                            \
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"                     \
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory")
#define TFNO_TMEM_LD8(taddr, r)                                                                            \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"                     \
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])  \
                 : "r"(taddr) : "memory")
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

// Bounded wait that ignores the abort flag: used at teardown to let copies and MMAs that are
// already in flight finish before shared and tensor memory are given back.
__device__ __forceinline__ void mbar_drain(uint32_t bar, uint32_t parity) {
    for (uint32_t spin = 0; spin < (1u << 16); ++spin) {
        if (mbar_try_wait(bar, parity)) return;
        __nanosleep(64);
    }
}

// ---------------------------------------------------------------------------------------------
// INVERSE = true: second transform is the true inverse (done as swap(FFT(swap(u))), so that both
// roles run the same forward 32-point code); false: a second forward transform.
// R = DY / 32 lanes per signal.
template <int R, bool INVERSE>
__global__ void __launch_bounds__(kTcThreads, 1) spectral_tc_kernel(const __grid_constant__ TcParams p) {
    static_assert(R == 4 || R == 8 || R == 16 || R == 32, "DY = 32 R in {128, 256, 512, 1024}");
    using G = Geometry<R>;
    constexpr int CH = G::CH, GPW = G::GPW;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int K = p.K;                                // a multiple of 4
    const int NC = (K + CH - 1) / CH;                 // chunks per row (a compile-time NC measured 4 % slower)
    // A last chunk with fewer than CH channels: the copies bring only its channels, the weights of
    // the missing ones are zero in tensor memory, and the rows of the ring that no copy ever writes
    // are zeroed once below -- the forward warps transform whatever the other rows hold (finite
    // values of earlier chunks) and the zero weights remove it.  The task loops do not change.
    const int Kp = NC * CH;
    const int SBO = s_sbo_fused(R), SBYTES = s_bytes(R);
    unsigned char* ring = base;
    unsigned char* sS = ring + kStages * G::STAGE_BYTES;            // [buffer 0: hi | lo][buffer 1: hi | lo]
    float* planes = reinterpret_cast<float*>(sS + 4 * SBYTES);      // [2][64][64]
    unsigned char* ostage = reinterpret_cast<unsigned char*>(planes + 2 * 64 * 64);   // [8 warps][OUT_ROWS][OUT_STRIDE]
    float2* twF = reinterpret_cast<float2*>(ostage + kInvWarps * G::OUT_BYTES);      // [R][32]
    float2* twI = twF + R * 32;                                                       // [R][32]
    uint64_t* bars = reinterpret_cast<uint64_t*>(twI + R * 32);
    // barrier indices
    constexpr int B_FULL = 0, B_EMPTY = kStages, B_SFULL = 2 * kStages, B_SEMPTY = B_SFULL + 2, B_AFULL = B_SEMPTY + 2,
                  B_AEMPTY = B_AFULL + 2, B_PFULL = B_AEMPTY + 2, B_PEMPTY = B_PFULL + 1, B_STAGGER = B_PEMPTY + 1,
                  B_DRAIN = B_STAGGER + 2, B_HELP = B_DRAIN + 1, B_COUNT = B_HELP + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * (uint32_t)i; };

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef TFNO_TC_TRACE
    const long long tr_entry = clock64();
    long long tr_dep = 0, tr_staged = 0, tr_conv = 0;
#endif
    // Roles.  A scheduler partition hosts warps w, w+4, ...; giving it compute warps of the SAME role
    // keeps its instruction cache on one role's code.
    const bool is_compute = warp < kComputeWarps;
    const bool is_fwd = is_compute && !(warp & 1);          // warps 0,2,..,14
    const bool is_inv = is_compute && (warp & 1);           // warps 1,3,..,15
    const bool is_xfer = warp >= 16 && warp < 20;           // TMEM quarter = warp & 3
    constexpr int kProducerWarp = 20, kMmaWarp = 21;

    // ---------------- set-up ----------------
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(bar(B_FULL + s), 1); mbar_init(bar(B_EMPTY + s), kHalfWarps); }
        for (int c = 0; c < 2; ++c) { mbar_init(bar(B_SFULL + c), kHalfWarps); mbar_init(bar(B_SEMPTY + c), 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(bar(B_AFULL + b), 1); mbar_init(bar(B_AEMPTY + b), 4); }
        mbar_init(bar(B_PFULL), 4);
        mbar_init(bar(B_PEMPTY), kInvWarps);
        mbar_init(bar(B_STAGGER), 4);
        mbar_init(bar(B_STAGGER + 1), 4);
        mbar_init(bar(B_DRAIN), 1);
        mbar_init(bar(B_HELP), 4);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (Kp != K) {
        for (int i = tid; i < kStages * G::STAGE_BYTES / 16; i += kTcThreads) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0u, 0u, 0u, 0u);
        fence_async_smem();                            // before the copy engine writes other rows of the same stages
    }
    fill_forward_table32<R>(twF, tid, kTcThreads);
    fill_inverse_table32_folded<R>(twI, tid, kTcThreads, p.inv_gain, INVERSE);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t TM_WHI = 0, TM_WLO = 2 * Kp, TM_ACC = 4 * Kp;      // column offsets; accumulators 2 x 64 columns

#ifndef TFNO_NO_PDL
    // Programmatic dependent launch: everything above touched only this CTA's shared and tensor
    // memory, so it may run while the previous kernel of the stream is still finishing on other
    // SMs.  From here on global memory is read and written: wait for the previous kernel to
    // complete, then let the next launch begin its own set-up as SMs become free.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
#ifdef TFNO_TC_TRACE
    tr_dep = clock64();
#endif
    const long long first = blockIdx.x;
    const int n_it = first < p.rows ? (int)((p.rows - first + gridDim.x - 1) / gridDim.x) : 0;
    const long long n_loads = (long long)n_it * NC;
    // Chunk c of a row belongs to forward half-team c & 1 and travels through ring stage c & 1, so a
    // stage has ONE consuming half-team, which sees every phase of its barriers (a parity wait
    // cannot tell "not yet" from "two phases on").  The k-th use of a stage is counted per stage.
    // A row with a single chunk alternates the two stages between rows (one consumer again).
    auto stage_of = [&](int it, int c) { return NC == 1 ? (it & 1) : (c & 1); };
    auto use_of = [&](int it, int c) {
        return NC == 1 ? (uint32_t)(it >> 1) : (uint32_t)it * (uint32_t)((NC - (c & 1) + 1) / 2) + (uint32_t)(c >> 1);
    };

    // Weights into tensor memory.  Lane l of a warp with warp % 4 == q reaches TMEM row i = 32 q + l:
    // rows 0-63 produce Re, rows 64-127 produce Im of output channel n = i & 63.  Twenty warps take
    // part (five per quarter, each a fifth of the four-channel blocks), so that the set-up of a short
    // launch stays short.  Column kk of a chunk = 2 * channel + part: Re and Im of a channel are adjacent,
    // matching the 8-byte stores of the forward warps.
    auto issue_load = [&](long long L) {       // whole producer warp; lanes < CH copy one row each
        const int s = stage_of((int)(L / NC), (int)(L % NC));
        const long long row = first + (L / NC) * gridDim.x;
        const int c = (int)(L % NC);
        const int valid = (K - c * CH < CH) ? K - c * CH : CH;     // channels of this chunk
        if (lane == 0) mbar_arrive_expect_tx(bar(B_FULL + s), valid * G::ROW_BYTES);
        __syncwarp();
        for (int j = lane; j < valid; j += 32) {
            const float2* src = p.x + row * p.x_stride_row + (long long)(c * CH + j) * p.x_stride_k;
            bulk_load(smem_u32(ring + s * G::STAGE_BYTES + j * G::ROW_STRIDE), src, G::ROW_BYTES, bar(B_FULL + s));
        }
    };
    // The producer warp starts the copies of the first ring stages and goes straight to its role
    // (issuing them takes it ~5 k cycles); the other 23 warps bring the weights in meanwhile and
    // meet at a named barrier of their own.
    long long preloaded = 0;
    if (warp == kProducerWarp) {
        for (; preloaded < kStages && preloaded < n_loads; ++preloaded) issue_load(preloaded);
    } else {
        // Through shared memory: a thread needs (output n = its TMEM row, four adjacent channels),
        // which in memory are 32 bytes every K*8 (or 8 bytes every N*8) -- read that way, every
        // warp-wide load touches 32 lines and the set-up of a launch took 6 us.  Instead the warps
        // fetch the weights as contiguous runs with asynchronous 8-byte copies, all in flight
        // together (one trip to memory), into the S buffers and planes, which nothing uses yet, as
        // [n][K channels + 16 bytes] (row stride = 16 mod 128 for K a multiple of 16: the 16-byte
        // reads of a quarter-warp fall into distinct banks), and the 20 warps below the producer
        // pick their values from there (five per TMEM quarter).
        constexpr int kStagers = kTcThreads - 32, kConvShares = 5;
        static_assert(kProducerWarp == 4 * kConvShares, "warps 0..19 convert");
        static_assert(4 * s_bytes(R) + 2 * 64 * 256 + kInvWarps * G::OUT_BYTES >= 64 * (96 * 8 + 16), "weight staging area");
        auto stagers_sync = [] { asm volatile("bar.sync 1, %0;" ::"n"(kStagers) : "memory"); };
        unsigned char* wst = sS;
        const int wrow = K * 8 + 16;
        const bool k_fast = p.w_stride_k == 1;
        const int stid = warp < kProducerWarp ? tid : tid - 32;
        const int q = warp & 3, share = warp >> 2;                    // share 0..4 of quarter q (warps 0..19)
        const int i = 32 * q + lane, n = i & 63, im_row = i >> 6;
        const uint32_t trow = tmem + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
        for (int idx = stid; idx < 64 * K; idx += kStagers) {
            const int kk = k_fast ? idx % K : idx >> 6, nn = k_fast ? idx / K : idx & 63;
            const float2* src = p.w + (long long)kk * p.w_stride_k + (long long)nn * p.w_stride_n;
            asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(wst + nn * wrow + kk * 8)), "l"(src) : "memory");
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        stagers_sync();
#ifdef TFNO_TC_TRACE
        tr_staged = clock64();
#endif
        if (warp < kProducerWarp) {
            for (int blk = share; blk < Kp / 4; blk += kConvShares) {
                const bool real = 4 * blk < K;                        // channels K .. Kp-1 get zero weights
                const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
                const float4 a = real ? *reinterpret_cast<const float4*>(wst + n * wrow + blk * 32) : zero4;
                const float4 c = real ? *reinterpret_cast<const float4*>(wst + n * wrow + blk * 32 + 16) : zero4;
                const float2 w4[4] = {make_float2(a.x, a.y), make_float2(a.z, a.w), make_float2(c.x, c.y), make_float2(c.z, c.w)};
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int part = j & 1;
                    const float2 w1 = w4[j >> 1];
                    // Re row: [ Wr | -Wi ],  Im row: [ Wi | Wr ]  against  S = [ Xr ; Xi ]
                    const float v = im_row ? (part ? w1.x : w1.y) : (part ? -w1.y : w1.x);
                    const float h = tf32_hi(v);
                    hi[j] = __float_as_uint(h);
                    lo[j] = __float_as_uint(tf32_hi(v - h));
                }
                TFNO_TMEM_ST8(trow + TM_WHI + 8 * blk, hi);
                TFNO_TMEM_ST8(trow + TM_WLO + 8 * blk, lo);
            }
        }
        if (warp < kProducerWarp) asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
#ifdef TFNO_TC_TRACE
        tr_conv = clock64();
#endif
        // the MMA thread may read the weights, and the planes area is free, once all of them are here
        tc_fence_before();
        stagers_sync();
        tc_fence_after();
    }

    TFNO_TRACE_DECL
#ifdef TFNO_TC_TRACE
    // helpers: from kernel entry until the dependency wait returned (out) / the first pass of the weights is
    // in shared memory (in) / the weights are in tensor memory (mid) / the roles start (loop)
    if (!is_compute) { tr_wait[9] = tr_dep - tr_entry; tr_wait[7] = tr_staged - tr_entry; tr_wait[8] = tr_conv - tr_entry; tr_wait[10] = tr_t0 - tr_entry; }
#endif
    if (!is_compute) {
        // ============ warpgroups 4 and 5: accumulator hand-off, data movement, MMA issue ============
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs) : "memory");
        if (is_xfer) {
            // accumulator row i = (part, channel) of this thread -> Re / Im planes in shared memory
            const int i = tid - 512;
            const int q = warp & 3;
            float* prow = planes + (i >> 6) * 4096 + (i & 63) * 64;
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int buf = it & 1;
                ok = TFNO_TRACE_WAIT(0, mbar_wait(bar(B_AFULL + buf), (it >> 1) & 1, abort_flag, p.status, 41, kHelperIdleNs));
                if (ok) ok = TFNO_TRACE_WAIT(1, mbar_wait(bar(B_PEMPTY), (it & 1) ^ 1, abort_flag, p.status, 42, kHelperIdleNs));
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + TM_ACC + 64 * buf;
#pragma unroll 1
                for (int c0 = 0; c0 < 64; c0 += 8) {
                    uint32_t acc[8];
                    TFNO_TMEM_LD8(taddr + c0, acc);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int cc = c0 >> 2;
                    *reinterpret_cast<uint4*>(prow + plane_chunk(i & 63, cc) * 4) = make_uint4(acc[0], acc[1], acc[2], acc[3]);
                    *reinterpret_cast<uint4*>(prow + plane_chunk(i & 63, cc + 1) * 4) = make_uint4(acc[4], acc[5], acc[6], acc[7]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar(B_AEMPTY + buf));
                    mbar_arrive(bar(B_PFULL));
                    if (it == n_it - 1) mbar_arrive(bar(B_HELP));      // the forward warps help with the last row
                }
            }
        } else if (warp == kProducerWarp) {
            // producer: keeps the ring full
            bool ok = true;
            long long L = preloaded;      // the first stages were started before the weights
            for (; L < n_loads && ok; ++L) {
                const int s = stage_of((int)(L / NC), (int)(L % NC));
                const uint32_t u = use_of((int)(L / NC), (int)(L % NC));
                ok = __all_sync(0xffffffffu, TFNO_TRACE_WAIT(0, mbar_wait(bar(B_EMPTY + s), (u & 1) ^ 1, abort_flag, p.status, 11, kHelperIdleNs)));
                if (!ok) break;
                issue_load(L);
            }
            if (*abort_flag) {
                // copies already issued still write into this CTA's shared memory: let them land
                for (long long j = (L >= kStages ? L - kStages : 0); j < L; ++j)
                    mbar_drain(bar(B_FULL + stage_of((int)(j / NC), (int)(j % NC))), use_of((int)(j / NC), (int)(j % NC)) & 1);
            }
        } else if (warp == kMmaWarp && lane == 0) {
            // MMA issuer
            const uint32_t idesc = make_idesc_tf32(64);
            bool ok = true;
            for (int it = 0; it < n_it && ok; ++it) {
                const int buf = it & 1;
                const uint32_t d_tmem = tmem + TM_ACC + 64 * buf;
                for (int c = 0; c < NC && ok; ++c) {
                    // chunk c sits in S buffer h = c & 1; it is the j-th chunk its half-team has produced
                    const int h = c & 1;
                    const uint32_t j = (uint32_t)it * (uint32_t)((NC - h + 1) / 2) + (uint32_t)(c >> 1);
                    ok = TFNO_TRACE_WAIT(0, mbar_wait(bar(B_SFULL + h), j & 1, abort_flag, p.status, 21, kHelperIdleNs));
                    if (ok && c == 0) ok = TFNO_TRACE_WAIT(1, mbar_wait(bar(B_AEMPTY + buf), ((it >> 1) & 1) ^ 1, abort_flag, p.status, 22, kHelperIdleNs));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t s_hi = smem_u32(sS) + (uint32_t)(2 * h * SBYTES), s_lo = s_hi + SBYTES;
#pragma unroll 1
                    for (int jj = 0; jj < G::KSTEPS_PER_CHUNK; ++jj) {
                        const int ks = c * G::KSTEPS_PER_CHUNK + jj;              // k-step of the row: kk in [8ks, 8ks+8)
                        const uint64_t dhi = make_kmajor_desc(s_hi + 2 * jj * kLBO, kLBO, SBO);
                        const uint64_t dlo = make_kmajor_desc(s_lo + 2 * jj * kLBO, kLBO, SBO);
                        const uint32_t a_hi = tmem + TM_WHI + 8 * ks, a_lo = tmem + TM_WLO + 8 * ks;
                        umma_tf32_ts(d_tmem, a_hi, dhi, idesc, (c | jj) ? 1u : 0u);
                        umma_tf32_ts(d_tmem, a_lo, dhi, idesc, 1u);
                        umma_tf32_ts(d_tmem, a_hi, dlo, idesc, 1u);
                    }
                    umma_commit(bar(B_SEMPTY + h));
                    if (c == NC - 1) umma_commit(bar(B_AFULL + buf));
                }
            }
            // every MMA issued so far has finished before tensor memory is released
            umma_commit(bar(B_DRAIN));
            mbar_drain(bar(B_DRAIN), 0);
        }
    } else {
    // ======================= forward and inverse warps =======================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kComputeRegs) : "memory");
    const int g = lane / R, r = lane % R;             // lane = r + R*g: the R lanes of a group are adjacent
    // forward: half-teams {0,2,4,6} and {8,..,14}: a scheduler partition hosts two warps of each,
    // and the second half-team starts half a task late, so that one half's arithmetic overlaps the
    // other's shuffles, shared-memory traffic and waits instead of colliding with it
    const int half = (warp >> 3) & 1, wl = (warp >> 1) & 3;
    bool stagger_pending = true;
    const int kl = wl * GPW + g;                      // forward: channel inside the chunk
    const int qi = warp >> 1;                         // inverse: 0..7
    constexpr int GROUPS = kInvWarps * GPW;           // inverse: channels per pass
    const int fwd_tasks = (NC - half + 1) / 2;
    constexpr int kInvTasks = 64 / GROUPS;
    // Drain: while the inverse warps finish the last row of the CTA the forward warps would idle, so
    // they turn into inverse warps and take the upper half of that row's tasks (phase 1 below).
    // They stage their output rows in the ring: warp qi = 4*half + wl gets the bytes of ITS rows of
    // ITS half-team's stage (OUT_BYTES = GPW * ROW_STRIDE), which it has read for the last time and
    // which no copy targets any more.  Needs staged output (DY >= 256: two or more tasks per row)
    // and a stage per half-team (two or more chunks per row).
#ifndef TFNO_NO_DRAIN_HELP
    const bool drain_help = G::STAGED_OUT && kInvTasks >= 2 && NC >= 2 && n_it > 0;
#else
    const bool drain_help = false;
#endif
    static_assert(!G::STAGED_OUT || kStages * G::STAGE_BYTES == kInvWarps * G::OUT_BYTES, "the ring holds one staging buffer per helping warp");
    bool alive = true;

    TFNO_TRACE_MARK();
    // The task loops exist twice in the binary: the main copy (phase 0, both roles) and a copy that
    // runs the inverse tasks of the CTA's last row on all sixteen compute warps (phase 1).  Two
    // instantiations rather than a run-time phase: the extra live state of a shared copy cost the
    // main loop 10 %.
    auto run_tasks = [&](auto phase_tag) {
    constexpr int phase = decltype(phase_tag)::value;
    const bool fwd = phase ? false : is_fwd;          // the role this warp plays in this phase
    const float2 coef = fwd ? round1_coef32<R>(r) : inverse_fold_coef32<R>(r, INVERSE);   // forward: round 1; inverse: W_R^{-+r}
    // phase 0: all rows (inverse warps: all but the last when the forward warps help); phase 1: the
    // last row's inverse tasks, lower half on the inverse warps, upper half on the forward warps
    const int it_end = (phase == 0 && !fwd && drain_help) ? n_it - 1 : n_it;
    const int t_lo = phase ? (is_fwd ? kInvTasks / 2 : 0) : 0;
    const int t_hi = phase ? (is_fwd ? kInvTasks : kInvTasks / 2) : (fwd ? fwd_tasks : kInvTasks);
    const bool wait_planes = phase == 0 || !is_fwd;
    for (int it = phase ? n_it - 1 : 0; it < it_end && alive; ++it) {
        const long long row = first + (long long)it * gridDim.x;
        for (int t = t_lo; t < t_hi && alive; ++t) {
            TFNO_TRACE_SINCE(10);
            float2 v[32];
            float sgn = 1.0f;
            int n = 0, s = 0;
            // ------------------------------ prologue ------------------------------
            if (fwd) {
                const int c = half + 2 * t;
                s = stage_of(it, c);
                const uint32_t u = use_of(it, c);
                alive = __all_sync(0xffffffffu, TFNO_TRACE_STEP(0, mbar_wait(bar(B_FULL + s), u & 1, abort_flag, p.status, 31)));
                if (!alive) break;
                const float2* srow = reinterpret_cast<const float2*>(ring + s * G::STAGE_BYTES + kl * G::ROW_STRIDE);
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = srow[R * i + r];
                // Hand the stage back for the next asynchronous (bulk-copy) overwrite.  The fence
                // waits until this thread's loads have returned: __syncwarp alone does not, and a
                // stage released with loads still in flight was overwritten under them.
                __threadfence_block();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_EMPTY + s));
                TFNO_TRACE_SINCE(7);
                sgn = lane_rotated32<R>(r) ? -1.0f : 1.0f;
            } else {
                if (t == t_lo && wait_planes) {
                    alive = __all_sync(0xffffffffu, TFNO_TRACE_STEP(0, mbar_wait(bar(B_PFULL), it & 1, abort_flag, p.status, 43)));
                    if (!alive) break;
                }
                n = t * GROUPS + qi * GPW + g;
                const float* pre = planes + n * 64;
                const float* pim = planes + 4096 + n * 64;
                // u[m'] = T[m'] (C[m'] + c C[m'+32]), c = the lane's W_R^{-+r}; four m' per step
#pragma unroll
                for (int cc = 0; cc < 8; ++cc) {
                    const float4 a0 = *reinterpret_cast<const float4*>(pre + plane_chunk(n, cc) * 4);
                    const float4 b0 = *reinterpret_cast<const float4*>(pim + plane_chunk(n, cc) * 4);
                    const float4 a1 = *reinterpret_cast<const float4*>(pre + plane_chunk(n, cc + 8) * 4);
                    const float4 b1 = *reinterpret_cast<const float4*>(pim + plane_chunk(n, cc + 8) * 4);
                    const float4 t0 = *reinterpret_cast<const float4*>(twI + tw_index<R>(r, 4 * cc));
                    const float4 t1 = *reinterpret_cast<const float4*>(twI + tw_index<R>(r, 4 * cc + 2));
                    const float2 u0 = cmul(cmadd(make_float2(a0.x, b0.x), coef, make_float2(a1.x, b1.x)), make_float2(t0.x, t0.y));
                    const float2 u1 = cmul(cmadd(make_float2(a0.y, b0.y), coef, make_float2(a1.y, b1.y)), make_float2(t0.z, t0.w));
                    const float2 u2 = cmul(cmadd(make_float2(a0.z, b0.z), coef, make_float2(a1.z, b1.z)), make_float2(t1.x, t1.y));
                    const float2 u3 = cmul(cmadd(make_float2(a0.w, b0.w), coef, make_float2(a1.w, b1.w)), make_float2(t1.z, t1.w));
                    // inverse as swap(FFT(swap(u))): exchange re/im going in (and coming out below)
                    v[4 * cc] = INVERSE ? make_float2(u0.y, u0.x) : u0;
                    v[4 * cc + 1] = INVERSE ? make_float2(u1.y, u1.x) : u1;
                    v[4 * cc + 2] = INVERSE ? make_float2(u2.y, u2.x) : u2;
                    v[4 * cc + 3] = INVERSE ? make_float2(u3.y, u3.x) : u3;
                }
                if (phase == 0 && t == t_hi - 1) {
                    // the planes have been read for the last time this row; the fence orders the
                    // loads above before the release (their values are consumed only later)
                    __threadfence_block();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(B_PEMPTY));
                }
                TFNO_TRACE_SINCE(8);
            }

            // ------------------------------ the one 32-point transform ------------------------------
            if (stagger_pending && (warp >> 3) == 1) {
                // once: the second half waits until its partition mates have finished a first transform
                alive = __all_sync(0xffffffffu, mbar_wait(bar(B_STAGGER + (fwd ? 0 : 1)), 0, abort_flag, p.status, 51));
                if (!alive) break;
            }
            fft32<-1>(v, sgn);
            TFNO_TRACE_SINCE(6);
            if (stagger_pending && (warp >> 3) == 0) {
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_STAGGER + (fwd ? 0 : 1)));
            }
            stagger_pending = false;

            // ------------------------------ epilogue ------------------------------
            if (fwd) {
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float4 tt = *reinterpret_cast<const float4*>(twF + tw_index<R>(r, j));
                    v[slot32(j)] = cmul(v[slot32(j)], make_float2(tt.x, tt.y));
                    v[slot32(j + 1)] = cmul(v[slot32(j + 1)], make_float2(tt.z, tt.w));
                }
                // exchange rounds over the R adjacent lanes of the group
                exchange_round1_32(v, R >> 1, coef);
                exchange_round2_32(v, R >> 2);
                if constexpr (R >= 8) exchange_round_32<8>(v, R >> 3, (r & (R >> 3)) != 0);
                if constexpr (R >= 16) exchange_round_32<4>(v, R >> 4, (r & (R >> 4)) != 0);
                if constexpr (R >= 32) exchange_round_32<2>(v, R >> 5, (r & (R >> 5)) != 0);
                // lane r now holds modes 64/R*r + j, j < 64/R, in v[slot32(j)]
                TFNO_TRACE_SINCE(8);
                // this half-team's S buffer is free once the MMAs of its previous chunk have completed
                const uint32_t jchunk = (uint32_t)it * (uint32_t)fwd_tasks + (uint32_t)t;
                alive = __all_sync(0xffffffffu, TFNO_TRACE_STEP(1, mbar_wait(bar(B_SEMPTY + half), (jchunk & 1) ^ 1, abort_flag, p.status, 32)));
                if (!alive) break;
                constexpr int PER = 64 / R;
                unsigned char* sbuf = sS + 2 * half * SBYTES;
                unsigned char* hi_base = sbuf + (kl >> 1) * kLBO + (kl & 1) * 8;     // kk = 2*kl (Re), 2*kl + 1 (Im)
#pragma unroll
                for (int j = 0; j < PER; ++j) {
                    const int m = PER * r + j;
                    const int off = (m >> 3) * SBO + (m & 7) * 16;
                    const float xr = v[slot32(j)].x, xi = v[slot32(j)].y;
                    const float hr = tf32_hi(xr), hi = tf32_hi(xi);
                    *reinterpret_cast<float2*>(hi_base + off) = make_float2(hr, hi);
                    *reinterpret_cast<float2*>(hi_base + SBYTES + off) = make_float2(xr - hr, xi - hi);
                }
                fence_async_smem();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_SFULL + half));
                TFNO_TRACE_SINCE(9);
            } else {
                if constexpr (!G::STAGED_OUT) {
                    // Lanes r and r ^ 1 of a group (adjacent) own samples that alternate in
                    // memory: each stores 16 bytes (its own sample and the neighbour's) for every
                    // second j2 and they swap the foreign halves with a shuffle -- half as many
                    // store instructions, each filling whole 32-byte sectors.
                    const bool odd = (r & 1) != 0;
                    float2* dst = p.y + row * p.y_stride_row + (long long)n * p.y_stride_n + (odd ? R : 0) + (r & ~1);
#pragma unroll
                    for (int n2 = 0; n2 < 16; ++n2) {
                        const float2 a = v[slot32(2 * n2)], b = v[slot32(2 * n2 + 1)];
                        const float2 ev = INVERSE ? make_float2(a.y, a.x) : a;       // this lane's sample R*(2*n2) + r
                        const float2 od = INVERSE ? make_float2(b.y, b.x) : b;       // this lane's sample R*(2*n2+1) + r
                        const float2 send = odd ? ev : od;
                        float2 got;
                        got.x = __shfl_xor_sync(0xffffffffu, send.x, 1);
                        got.y = __shfl_xor_sync(0xffffffffu, send.y, 1);
                        float4 o4 = odd ? make_float4(got.x, got.y, od.x, od.y) : make_float4(ev.x, ev.y, got.x, got.y);
                        if (p.accumulate) {
                            const float4 prev = *reinterpret_cast<const float4*>(dst + 2 * R * n2);
                            o4.x += prev.x; o4.y += prev.y; o4.z += prev.z; o4.w += prev.w;
                        }
                        *reinterpret_cast<float4*>(dst + 2 * R * n2) = o4;
                    }
                } else {
                // Stage the warp's OUT_ROWS output rows in shared memory and hand each row to the
                // bulk-copy engine: the rows leave as full lines instead of 32-byte pieces through
                // the load/store unit.  The lanes that issue the copies first wait until their
                // previous copies have finished reading the staging buffer.
                unsigned char* ost = ((phase && is_fwd) ? ring : ostage) + qi * G::OUT_BYTES;
                if (lane < G::OUT_ROWS) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                __syncwarp();
                TFNO_TRACE_SINCE(2);
                // rows padded against bank conflicts, or dense as the tiled copy wants its box
                const int out_stride = (G::TENSOR_OUT && p.use_ymap) ? G::ROW_BYTES : G::OUT_STRIDE;
                float2* srow_out = reinterpret_cast<float2*>(ost + g * out_stride);
#pragma unroll
                for (int j2 = 0; j2 < 32; ++j2) {
                    const float2 o = v[slot32(j2)];
                    srow_out[R * j2 + r] = INVERSE ? make_float2(o.y, o.x) : o;
                }
                TFNO_TRACE_SINCE(3);
                fence_async_smem();
                __syncwarp();
                if (G::TENSOR_OUT && p.use_ymap) {
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];"
                                     ::"l"(reinterpret_cast<uint64_t>(&p.ymap)), "r"(0), "r"((int)row), "r"(t * GROUPS + qi * GPW),
                                       "r"(smem_u32(ost)) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                } else if (lane < G::OUT_ROWS) {
                    const int nn = t * GROUPS + qi * GPW + lane;
                    float2* dst = p.y + row * p.y_stride_row + (long long)nn * p.y_stride_n;
                    if (p.accumulate)
                        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                                     ::"l"(dst), "r"(smem_u32(ost + lane * G::OUT_STRIDE)), "r"(G::ROW_BYTES) : "memory");
                    else
                        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                     ::"l"(dst), "r"(smem_u32(ost + lane * G::OUT_STRIDE)), "r"(G::ROW_BYTES) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                }
                TFNO_TRACE_SINCE(9);
            }
        }
    }
    };   // run_tasks
    run_tasks(std::integral_constant<int, 0>{});
    if (drain_help && alive) {
        stagger_pending = false;
        // The forward warps wait for the planes of the last row on a barrier of their own: they have
        // not followed the phases of B_PFULL, and a parity wait cannot tell "not yet" from "two
        // phases on".  The inverse warps wait on B_PFULL as in every row.
        if (is_fwd) alive = __all_sync(0xffffffffu, mbar_wait(bar(B_HELP), 0, abort_flag, p.status, 44));
        if (alive) run_tasks(std::integral_constant<int, 1>{});
    }
    if (is_inv || drain_help) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all output rows have landed
    }   // forward / inverse warps

    // ---------------- teardown ----------------
    TFNO_TRACE_FLUSH();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

}  // namespace tc
}  // namespace tfno

// Host-side launch helpers shared by the C ABI: size dispatch (transform length -> lanes per
// signal R, output channels -> accumulator blocks NB), shared-memory sizing and persistent grids.
#pragma once
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include <mutex>
#ifdef TFNO_TC_TRACE
#include <vector>
#endif
#include "../../include/turbofno_b200.h"
#include "spectral_kernels.cuh"
#include "spectral_tc.cuh"
#include "cgemm_tc.cuh"
#include "cgemm_permode.cuh"
#include "spectral_image32.cuh"

namespace tfno {

struct DeviceInfo {
    int device = 0;
    int sms = 0;
    int max_smem_optin = 0;
    bool use_tensor_cores = true;   // tcgen05 fused kernel where its shape limits allow
    int* status = nullptr;          // device word written by kernels whose bounded waits ran out
    // Dry run: when set, every launcher appends the name of the kernel it would launch (separated
    // by ';') and launches nothing.  tfno_plan_kernels reports a plan's kernels this way, from
    // the same dispatch code tfno_exec runs.
    char* record = nullptr;
    size_t record_cap = 0;
};

inline int log2_exact(long long v) {
    int l = 0;
    while ((1LL << l) < v) ++l;
    return ((1LL << l) == v) ? l : -1;
}
inline bool supported_len(int len) { return len == 128 || len == 256 || len == 512 || len == 1024; }

// Appends "name" (printf-style) to the record buffer; true when the caller is a dry run.
inline bool record_launch(const DeviceInfo& dev, const char* fmt, int a = 0, int b = 0, int c = 0, int d = 0) {
    if (!dev.record) return false;
    const size_t used = std::strlen(dev.record);
    if (used + 2 < dev.record_cap) {
        int n = 0;
        if (used) n = std::snprintf(dev.record + used, dev.record_cap - used, ";");
        std::snprintf(dev.record + used + n, dev.record_cap - used - n, fmt, a, b, c, d);
    }
    return true;
}

// Per-kernel launch set-up, done once per (kernel, device, block size, shared-memory size) and
// remembered: the opt-in to more than 48 KB of dynamic shared memory and the resident blocks per
// SM.  A fixed table, no heap: the allocation-free entry point goes through here too.
struct KernelSetupEntry {
    const void* func;
    int device, threads;
    size_t smem;
    int occ;
};
constexpr int kKernelSetupSlots = 512;
inline KernelSetupEntry* kernel_setup_table() {
    static KernelSetupEntry table[kKernelSetupSlots];
    return table;
}
inline std::mutex& kernel_setup_mutex() {
    static std::mutex m;
    return m;
}
inline int kernel_setup_count(int add = 0) {
    static int n = 0;
    n += add;
    return n;
}

inline int prepare_kernel_cached(const void* func, int threads, size_t smem, const DeviceInfo& dev, int* blocks_per_sm) {
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lock(kernel_setup_mutex());
    KernelSetupEntry* table = kernel_setup_table();
    const int n = kernel_setup_count();
    size_t opted_in = 48 * 1024;        // largest dynamic shared-memory size this kernel has been opted in to so far
    for (int i = 0; i < n; ++i) {
        if (table[i].func != func || table[i].device != dev.device) continue;
        if (table[i].threads == threads && table[i].smem == smem) {
            *blocks_per_sm = table[i].occ;
            return TFNO_OK;
        }
        if (table[i].smem > opted_in) opted_in = table[i].smem;
    }
    // the attribute is one value per kernel: only ever raise it, or a launch that was set up
    // earlier with a larger size would be refused
    if (smem > opted_in) {
        if (cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return TFNO_ERR_CUDA;
        }
    }
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, func, threads, smem) != cudaSuccess || occ < 1) {
        cudaGetLastError();
        return TFNO_ERR_CUDA;
    }
    if (n < kKernelSetupSlots) {
        table[n] = KernelSetupEntry{func, dev.device, threads, smem, occ};
        kernel_setup_count(1);
    }
    *blocks_per_sm = occ;
    return TFNO_OK;
}

template <typename Kernel>
inline int prepare_kernel(Kernel kernel, size_t smem, const DeviceInfo& dev, int* blocks_per_sm, int threads = kThreads) {
    return prepare_kernel_cached(reinterpret_cast<const void*>(kernel), threads, smem, dev, blocks_per_sm);
}

#include "tc_trace.cuh"

inline int launch_status() { return cudaGetLastError() == cudaSuccess ? TFNO_OK : TFNO_ERR_CUDA; }

inline size_t tile_smem_bytes(int R, bool fwd, bool inv, int K, int N) {
    size_t elems = (size_t)K * kModes + (inv ? (size_t)N * kModes : 0) + 2 * (size_t)kSlabK * (N + kWPad) +
                   (fwd ? R * 64 : 0) + (inv ? R * 64 : 0);
    return elems * sizeof(float2);
}

template <int R, bool FWD, bool INV, int NB>
inline int launch_tile_inst(const DeviceInfo& dev, const TileParams& p, cudaStream_t st, int n_blocks = 1) {
    auto kernel = spectral_tile_kernel<R, FWD, INV, NB>;
    size_t smem = tile_smem_bytes(R, FWD, INV, p.K, p.N);
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    if (record_launch(dev, "spectral_tile_kernel<%d,%d,%d,%d>", R, FWD, INV, NB)) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(kernel, smem, dev, &occ);
    if (rc != TFNO_OK) return rc;
    long long grid = (long long)dev.sms * occ;
    if (grid > p.rows) grid = p.rows;
    kernel<<<dim3((unsigned)grid, (unsigned)n_blocks), kThreads, smem, st>>>(p);    // p.N channels per block of blockIdx.y
    return launch_status();
}

template <bool FWD, bool INV, int NB>
inline int launch_tile_r(const DeviceInfo& dev, int R, const TileParams& p, cudaStream_t st, int n_blocks = 1) {
    switch (R) {
        case 2: return launch_tile_inst<2, FWD, INV, NB>(dev, p, st, n_blocks);
        case 4: return launch_tile_inst<4, FWD, INV, NB>(dev, p, st, n_blocks);
        case 8: return launch_tile_inst<8, FWD, INV, NB>(dev, p, st, n_blocks);
        case 16: return launch_tile_inst<16, FWD, INV, NB>(dev, p, st, n_blocks);
    }
    return TFNO_ERR_UNSUPPORTED;
}

// Tensor-core fused kernel: N a multiple of 64 (64 per launch), K a multiple of the chunk size
// (4096 / DY channels: 32, 16, 8, 4 at DY = 128, 256, 512, 1024) up to 96 (tensor memory holds the
// weights, 4K columns, next to two accumulators), transform length 128 to 1024.
// Channels per launch of the fused tensor-core kernel: the weights of at most 96 channels fit tensor
// memory, so more channels (up to 192, a multiple of the chunk size) are split into two launches,
// the second adding its result to the first's (both halves multiples of the chunk size).
inline int tc_first_part(int K, int CH) {
    if (((K + CH - 1) / CH) * CH <= 96) return K;
    const int half = ((K / 2 + CH - 1) / CH) * CH;
    return half;
}
inline bool tc_eligible(const DeviceInfo& dev, int len, const TileParams& p) {
    if (!dev.use_tensor_cores || !dev.status) return false;
    if (p.N % 64 != 0 || !supported_len(len)) return false;
    const int CH = 128 / (len / 32);
    // K a multiple of 8; a last chunk of fewer than CH channels is padded with zero weights
    if (p.K < 8 || p.K > 192 || p.K % 8 != 0) return false;
    const int K1 = tc_first_part(p.K, CH), K2 = p.K - K1;
    if (K1 > 96 || ((K2 + CH - 1) / CH) * CH > 96) return false;
    const int launches = (p.N / 64) * (K2 ? 2 : 1);
    // several launches (one per 64 output channels and per part of the channels, each re-reading
    // its input): worth it only when the launches are long
    if (launches > 1 && p.rows < 2LL * dev.sms) return false;
    // a padded last chunk is wasted work: below one row per SM the FP32 kernel is as fast
    if (p.K % CH != 0 && p.rows < dev.sms) return false;
    return true;
}

// cuTensorMapEncodeTiled of the installed driver, looked up through the runtime (the library does
// not link libcuda); nullptr if the driver does not offer it.
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                      const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                      CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            f = nullptr;
        }
        return reinterpret_cast<TensorMapEncodeFn>(f);
    }();
    return fn;
}

// y as [channels][rows][len] complex (8-byte elements), box = {len, 1, box_channels}.  False when the
// layout does not meet the encoder's rules (16-byte aligned base and strides, box at most 256 wide).
inline bool encode_output_map(CUtensorMap* map, float2* y, int len, long long rows, int channels,
                              long long stride_row, long long stride_n, int box_channels) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc || len > 256 || rows <= 0 || rows > 0x7fffffffLL || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return false;
    if (stride_row <= 0 || stride_n <= 0 || (stride_row & 1) || (stride_n & 1)) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)len, (cuuint64_t)rows, (cuuint64_t)channels};
    const cuuint64_t strides[2] = {(cuuint64_t)stride_row * 8, (cuuint64_t)stride_n * 8};
    if (strides[0] >= (1ULL << 40) || strides[1] >= (1ULL << 40)) return false;
    const cuuint32_t box[3] = {(cuuint32_t)len, 1u, (cuuint32_t)box_channels};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 3, y, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Encoding a map costs the host several microseconds, which a launch of ~70 us that is issued
// back to back (eight ranks on one host) does not hide: keep the last maps, keyed by everything
// that goes into one.  A map holds an address and a geometry, nothing that can go stale.
inline bool cached_output_map(CUtensorMap* map, int device, float2* y, int len, long long rows, int channels,
                              long long stride_row, long long stride_n, int box_channels) {
    struct Entry { bool valid; int device, len, channels, box; const void* y; long long rows, sr, sn; CUtensorMap map; };
    constexpr int kEntries = 32;
    static std::mutex mu;
    static Entry table[kEntries] = {};
    static unsigned next = 0;
    std::lock_guard<std::mutex> lock(mu);
    for (const Entry& e : table)
        if (e.valid && e.device == device && e.y == y && e.len == len && e.rows == rows && e.channels == channels &&
            e.sr == stride_row && e.sn == stride_n && e.box == box_channels) {
            *map = e.map;
            return true;
        }
    CUtensorMap m;
    if (!encode_output_map(&m, y, len, rows, channels, stride_row, stride_n, box_channels)) return false;
    Entry& e = table[next++ % kEntries];
    e.valid = true; e.device = device; e.len = len; e.channels = channels; e.box = box_channels; e.y = y;
    e.rows = rows; e.sr = stride_row; e.sn = stride_n; e.map = m;
    *map = m;
    return true;
}

template <int R, bool INVERSE>
inline int launch_tc_inst(const DeviceInfo& dev, const TileParams& p, cudaStream_t st, bool accumulate = false) {
    auto kernel = tc::spectral_tc_kernel<R, INVERSE>;
    const size_t smem = tc::tc_smem_bytes<R>(p.K);
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    if (record_launch(dev, accumulate ? "spectral_tc_kernel<%d,%d>+=" : "spectral_tc_kernel<%d,%d>", R, INVERSE)) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(kernel, smem, dev, &occ, tc::kTcThreads);
    if (rc != TFNO_OK) return rc;
    {
        // The kernel redistributes registers between its warpgroups (setmaxnreg); the CTA's pool is
        // what it was launched with.  Refuse to launch a build whose pool is too small instead of
        // letting the register increase wait for ever.
        static int pool_ok = -1;
        if (pool_ok < 0) {
            cudaFuncAttributes fa{};
            pool_ok = (cudaFuncGetAttributes(&fa, kernel) == cudaSuccess &&
                       fa.numRegs * tc::kTcThreads >= 512 * tc::kComputeRegs + 256 * tc::kHelperRegs) ? 1 : 0;
        }
        if (!pool_ok) return TFNO_ERR_UNSUPPORTED;
    }
    tc::TcParams q{};
    q.rows = p.rows; q.K = p.K;
    q.x = p.x; q.x_stride_row = p.x_stride_row; q.x_stride_k = p.x_stride_k;
    q.w = p.w; q.w_stride_k = p.w_stride_k; q.w_stride_n = p.w_stride_n;
    q.y = p.y; q.y_stride_row = p.y_stride_row; q.y_stride_n = p.y_stride_n;
    q.inv_gain = p.inv_gain; q.conj_inverse = p.conj_inverse; q.status = dev.status;
    q.accumulate = accumulate ? 1 : 0;
#ifndef TFNO_NO_TENSOR_STORE
    if constexpr (tc::Geometry<R>::TENSOR_OUT)
        if (!accumulate) q.use_ymap = cached_output_map(&q.ymap, dev.device, p.y, 32 * R, p.rows, 64, p.y_stride_row, p.y_stride_n, tc::Geometry<R>::GPW) ? 1 : 0;
#endif
    long long grid = dev.sms;
    if (grid > p.rows) grid = p.rows;
#ifdef TFNO_TC_TRACE
    q.trace = tc_trace_buffer(dev, true);
#endif
#ifndef TFNO_NO_PDL
    {
        // launched so that its set-up may overlap the tail of the previous kernel in the stream
        // (the kernel orders itself behind that kernel with griddepcontrol.wait)
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = dim3((unsigned)grid);
        cfg.blockDim = dim3(tc::kTcThreads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, kernel, q) != cudaSuccess) {
            cudaGetLastError();
            return TFNO_ERR_CUDA;
        }
    }
#else
    kernel<<<(unsigned)grid, tc::kTcThreads, smem, st>>>(q);
#endif
#ifdef TFNO_TC_TRACE
    tc_trace_report(dev, (int)grid);
#endif
    return launch_status();
}

// Tensor-core contraction of compact spectra: N a multiple of 64 (64 per launch), K a multiple of 16 up to 64, beta = 0.
inline bool cgemm_tc_eligible(const DeviceInfo& dev, const TileParams& p) {
    if (!dev.use_tensor_cores || !dev.status) return false;
    // K a multiple of 8 (a last chunk of 8 channels is padded with zero weights), at most 96 per
    // launch (tensor memory) and 128 in two launches, the second adding to C
    if (p.N % 64 != 0 || p.K < 8 || p.K > 128 || p.K % 8 != 0) return false;
    // several launches (per block of 64 output channels, per half of K > 64), each re-reading its
    // spectra: worth it only when the launches are long
    if ((p.N > 64 || p.K > 64) && p.rows < 2LL * dev.sms) return false;

    if (p.beta.x != 0.f || p.beta.y != 0.f) return false;
    return ((reinterpret_cast<uintptr_t>(p.x) | reinterpret_cast<uintptr_t>(p.y)) & 15) == 0;
}
template <int TN>
inline int launch_cgemm_tc_inst(const DeviceInfo& dev, const TileParams& p, cudaStream_t st, bool accumulate) {
    auto kernel = tcg::cgemm_tc_kernel<TN>;
    const size_t smem = tcg::cgemm_tc_smem_bytes<TN>();
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    if (record_launch(dev, accumulate ? "cgemm_tc_kernel<%d>+=" : "cgemm_tc_kernel<%d>", TN)) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(kernel, smem, dev, &occ, tcg::kGemmThreads);
    if (rc != TFNO_OK) return rc;
    const long long M = p.rows * kModes;
    tcg::CgemmTcParams q{};
    q.tiles = M / TN; q.K = p.K;
    q.a = p.x; q.a_stride_k = M;
    q.w = p.w; q.w_stride_k = p.w_stride_k; q.w_stride_n = p.w_stride_n;
    q.c = p.y; q.c_stride_n = M;
    q.alpha = p.alpha; q.status = dev.status;
    q.accumulate = accumulate ? 1 : 0;
    long long grid = dev.sms;
    if (grid > q.tiles) grid = q.tiles;
    kernel<<<(unsigned)grid, tcg::kGemmThreads, smem, st>>>(q);
    return launch_status();
}
// 128-mode tiles when M allows it and there are enough of them to fill the device
inline int launch_cgemm_tc(const DeviceInfo& dev, const TileParams& p, cudaStream_t st) {
    const long long M = p.rows * kModes;
    // 65..96 channels: one launch on 64-mode tiles, whose smaller accumulators leave room for the
    // weights in tensor memory (4K + 2 TN <= 512 columns); more: two launches over the halves
    const bool narrow = p.K > 64 && p.K <= 96;
    const int K1 = p.K <= 96 ? p.K : ((p.K / 2 + tcg::kCH - 1) / tcg::kCH) * tcg::kCH;     // channels of the first launch
    for (int n0 = 0; n0 < p.N; n0 += 64) {
        for (int k0 = 0; k0 < p.K; k0 += K1) {
            TileParams q = p;
            q.N = 64;
            q.K = (k0 == 0) ? K1 : p.K - K1;
            q.x = p.x + (long long)k0 * M;                   // A[m + k*M]
            q.w = p.w + (long long)n0 * p.w_stride_n + (long long)k0 * p.w_stride_k;
            q.y = p.y + (long long)n0 * M;
            const bool acc = k0 != 0;
            const int rc = (!narrow && p.rows % 2 == 0 && p.rows / 2 >= dev.sms) ? launch_cgemm_tc_inst<128>(dev, q, st, acc) : launch_cgemm_tc_inst<64>(dev, q, st, acc);
            if (rc != TFNO_OK) return rc;
        }
    }
    return TFNO_OK;
}

// Row-tile kernel for any N that is a multiple of 64: output channels are processed in blocks of
// at most 128 (one launch per block; N <= 128, the whole reference grid, is a single launch).
template <bool FWD, bool INV>
inline int launch_tile(const DeviceInfo& dev, int len, TileParams p, cudaStream_t st) {
    if (p.rows <= 0) return TFNO_OK;
    if (p.K < kSlabK || p.K % kSlabK != 0 || p.N < 64 || p.N % 64 != 0) return TFNO_ERR_UNSUPPORTED;
    const int R = (FWD || INV) ? len / 64 : 2;      // the pure GEMM instance does not depend on R
    if ((FWD || INV) && !supported_len(len)) return TFNO_ERR_UNSUPPORTED;
    if constexpr (FWD && INV) {
        if (tc_eligible(dev, len, p)) {
            // The tensor-core kernel produces 64 output channels (its 128 accumulator rows); wider
            // layers run it once per block of 64, re-reading the input (still faster than the FP32
            // kernel: 1.0 against 1.7 ms at bs=8192, K=64, N=128, DY=256).
            const int K1 = tc_first_part(p.K, 128 / (len / 32));
            for (int n0 = 0; n0 < p.N; n0 += 64) {
                for (int k0 = 0; k0 < p.K; k0 += K1) {         // one or two parts of the channels
                    TileParams q = p;
                    q.N = 64;
                    q.K = (k0 == 0) ? K1 : p.K - K1;
                    q.x = p.x + (long long)k0 * p.x_stride_k;
                    q.w = p.w + (long long)n0 * p.w_stride_n + (long long)k0 * p.w_stride_k;
                    q.y = p.y + (long long)n0 * p.y_stride_n;
                    const bool acc = k0 != 0;
                    int rc = TFNO_ERR_UNSUPPORTED;
                    switch (len / 32) {            // lanes per signal
                        case 4: rc = q.conj_inverse ? launch_tc_inst<4, true>(dev, q, st, acc) : launch_tc_inst<4, false>(dev, q, st, acc); break;
                        case 8: rc = q.conj_inverse ? launch_tc_inst<8, true>(dev, q, st, acc) : launch_tc_inst<8, false>(dev, q, st, acc); break;
                        case 16: rc = q.conj_inverse ? launch_tc_inst<16, true>(dev, q, st, acc) : launch_tc_inst<16, false>(dev, q, st, acc); break;
                        case 32: rc = q.conj_inverse ? launch_tc_inst<32, true>(dev, q, st, acc) : launch_tc_inst<32, false>(dev, q, st, acc); break;
                    }
                    if (rc != TFNO_OK) return rc;
                }
            }
            return TFNO_OK;
        }
    }
    if constexpr (!FWD && !INV) {
        if (cgemm_tc_eligible(dev, p)) return launch_cgemm_tc(dev, p, st);
    }
    const int N = p.N;
    const long long M = p.rows * kModes;
    // A wide layer on a small batch: one launch whose grid also runs over blocks of 64 output
    // channels, so that the few rows are spread over N/64 times as many CTAs (a CTA that produces
    // all 128 channels of its row takes 47 us at K = N = 128; the latency, not the work, counts).
    if (N > 64 && p.rows * ((N + 127) / 128) * 2 <= dev.sms) {
        TileParams q = p;
        q.N = 64;
        return launch_tile_r<FWD, INV, 1>(dev, R, q, st, N / 64);
    }
    for (int n0 = 0; n0 < N; n0 += 128) {
        TileParams q = p;
        q.N = (N - n0 >= 128) ? 128 : 64;
        q.w = p.w + (long long)n0 * p.w_stride_n;
        q.y = p.y + (long long)n0 * (INV ? p.y_stride_n : M);
        int rc = (q.N == 128) ? launch_tile_r<FWD, INV, 2>(dev, R, q, st) : launch_tile_r<FWD, INV, 1>(dev, R, q, st);
        if (rc != TFNO_OK) return rc;
    }
    return TFNO_OK;
}

// Per-mode weights: persistent CTAs over (group of four modes, block of 64 outputs, split of the rows).
inline int launch_permode(const DeviceInfo& dev, PerModeParams p, cudaStream_t st) {
    if (p.rows <= 0) return TFNO_OK;
    if (p.K <= 0 || p.N % kPmNB != 0 || p.modes % kPmModes != 0) return TFNO_ERR_UNSUPPORTED;
    p.stage_a = pm_stage_a(p.K, dev.max_smem_optin) && (p.modes % 2 == 0) ? 1 : 0;
    const size_t smem = pm_smem_bytes(p.K, p.stage_a != 0);
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    if (record_launch(dev, "cgemm_permode_kernel")) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(cgemm_permode_kernel, smem, dev, &occ, kPmThreads);
    if (rc != TFNO_OK) return rc;
    // enough work items for two per SM, but never more splits than row tiles
    const long long groups = p.modes / kPmModes, passes = p.N / kPmNB, tiles = (p.rows + kPmRowTile - 1) / kPmRowTile;
    long long splits = (2LL * dev.sms + groups * passes - 1) / (groups * passes);
    if (splits > tiles) splits = tiles;
    if (splits < 1) splits = 1;
    p.splits = (int)splits;
    long long grid = groups * passes * splits;
    if (grid > (long long)dev.sms * occ) grid = (long long)dev.sms * occ;
    cgemm_permode_kernel<<<(unsigned)grid, kPmThreads, smem, st>>>(p);
    return launch_status();
}

template <typename Params, typename Kernel>
inline int launch_persistent(const DeviceInfo& dev, Kernel kernel, size_t smem, long long work_blocks,
                             const Params& p, cudaStream_t st, const char* name, int R) {
    if (work_blocks <= 0) return TFNO_OK;
    if (record_launch(dev, name, R)) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(kernel, smem, dev, &occ);
    if (rc != TFNO_OK) return rc;
    long long grid = (long long)dev.sms * occ;
    if (grid > work_blocks) grid = work_blocks;
    kernel<<<(unsigned)grid, kThreads, smem, st>>>(p);
    return launch_status();
}

inline int launch_fft_rows(const DeviceInfo& dev, int len, const RowsParams& p, cudaStream_t st) {
    const int R = len / 64;
    const long long blocks = (p.nsig + kThreads / R - 1) / (kThreads / R);
    switch (R) {
        case 2: return launch_persistent(dev, fft_rows_trunc_kernel<2>, 0, blocks, p, st, "fft_rows_trunc_kernel<%d>", 2);
        case 4: return launch_persistent(dev, fft_rows_trunc_kernel<4>, 0, blocks, p, st, "fft_rows_trunc_kernel<%d>", 4);
        case 8: return launch_persistent(dev, fft_rows_trunc_kernel<8>, 0, blocks, p, st, "fft_rows_trunc_kernel<%d>", 8);
        case 16: return launch_persistent(dev, fft_rows_trunc_kernel<16>, 0, blocks, p, st, "fft_rows_trunc_kernel<%d>", 16);
    }
    return TFNO_ERR_UNSUPPORTED;
}
inline int launch_ifft_rows(const DeviceInfo& dev, int len, const RowsParams& p, cudaStream_t st) {
    const int R = len / 64;
    const long long blocks = (p.nsig + kThreads / R - 1) / (kThreads / R);
    switch (R) {
        case 2: return launch_persistent(dev, ifft_rows_pad_kernel<2>, 0, blocks, p, st, "ifft_rows_pad_kernel<%d>", 2);
        case 4: return launch_persistent(dev, ifft_rows_pad_kernel<4>, 0, blocks, p, st, "ifft_rows_pad_kernel<%d>", 4);
        case 8: return launch_persistent(dev, ifft_rows_pad_kernel<8>, 0, blocks, p, st, "ifft_rows_pad_kernel<%d>", 8);
        case 16: return launch_persistent(dev, ifft_rows_pad_kernel<16>, 0, blocks, p, st, "ifft_rows_pad_kernel<%d>", 16);
    }
    return TFNO_ERR_UNSUPPORTED;
}
inline int launch_fft_cols(const DeviceInfo& dev, int len, const ColsParams& p, cudaStream_t st) {
    const int R = len / 64;
    const long long blocks = (p.nimg * p.DY + kThreads / R - 1) / (kThreads / R);
    switch (R) {
        case 2: return launch_persistent(dev, fft_cols_trunc_kernel<2>, 0, blocks, p, st, "fft_cols_trunc_kernel<%d>", 2);
        case 4: return launch_persistent(dev, fft_cols_trunc_kernel<4>, 0, blocks, p, st, "fft_cols_trunc_kernel<%d>", 4);
        case 8: return launch_persistent(dev, fft_cols_trunc_kernel<8>, 0, blocks, p, st, "fft_cols_trunc_kernel<%d>", 8);
        case 16: return launch_persistent(dev, fft_cols_trunc_kernel<16>, 0, blocks, p, st, "fft_cols_trunc_kernel<%d>", 16);
    }
    return TFNO_ERR_UNSUPPORTED;
}
inline int launch_ifft_cols(const DeviceInfo& dev, int len, const ColsParams& p, cudaStream_t st) {
    const int R = len / 64;
    const long long blocks = (p.nimg * p.DY + kThreads / R - 1) / (kThreads / R);
    switch (R) {
        case 2: return launch_persistent(dev, ifft_cols_pad_kernel<2>, 0, blocks, p, st, "ifft_cols_pad_kernel<%d>", 2);
        case 4: return launch_persistent(dev, ifft_cols_pad_kernel<4>, 0, blocks, p, st, "ifft_cols_pad_kernel<%d>", 4);
        case 8: return launch_persistent(dev, ifft_cols_pad_kernel<8>, 0, blocks, p, st, "ifft_cols_pad_kernel<%d>", 8);
        case 16: return launch_persistent(dev, ifft_cols_pad_kernel<16>, 0, blocks, p, st, "ifft_cols_pad_kernel<%d>", 16);
    }
    return TFNO_ERR_UNSUPPORTED;
}

inline size_t image_smem_bytes(int DX, int DY) {
    return ((size_t)DX * kModes + (DX / 64) * 64 + (DY / 64) * 64) * sizeof(float2);
}
// 16-byte loads and stores of sample pairs need 16-byte aligned rows
inline bool image_rows_aligned(const ImageParams& p, bool inverse) {
    const void* full = inverse ? (const void*)p.out : (const void*)p.in;
    return (reinterpret_cast<uintptr_t>(full) & 15) == 0 && (p.stride_b & 1) == 0 && (p.stride_k & 1) == 0;
}
// threads of the whole-image kernels: 8 warps at up to 255 registers; 12 warps at 168 registers were
// slower (2D layer bs=64, K=N=64, 256x256: 1.21 against 1.10 ms)
constexpr int kImageThreads = 256;
template <int THREADS, typename Kernel>
inline int launch_image(const DeviceInfo& dev, Kernel kernel, size_t smem, const ImageParams& p, cudaStream_t st,
                        const char* name, int RX, int RY) {
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    if (record_launch(dev, name, RX, RY, THREADS)) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(kernel, smem, dev, &occ, THREADS);
    if (rc != TFNO_OK) return rc;
    long long grid = (long long)dev.sms * occ;
    if (grid > p.nimg) grid = p.nimg;
    kernel<<<(unsigned)grid, THREADS, smem, st>>>(p);
    return launch_status();
}
// DX = 128: the 64 KB intermediate leaves room for two CTAs per SM if each has 4 warps (255
// registers per thread); the two then overlap one's X pass (half the warps idle) with the other's Y pass.
template <int RX> struct ImageThreads { static constexpr int value = (RX == 2) ? 128 : kImageThreads; };
template <int RX>
inline int launch_fft2d_rx(const DeviceInfo& dev, int RY, const ImageParams& p, bool inverse, cudaStream_t st) {
    const size_t smem = image_smem_bytes(64 * RX, 64 * RY);
    const bool paired = image_rows_aligned(p, inverse);
#define TFNO_IMG(RYV)                                                                                                  \
    case RYV:                                                                                                          \
        if (paired && inverse && p.centered_x)                                                                         \
            return launch_image<ImageThreads<RX>::value>(dev, ifft2d_pad_kernel<RX, RYV, true, ImageThreads<RX>::value, true>, smem, p, st, "ifft2d_pad_kernel<%d,%d,paired,%d,centered>", RX, RYV);  \
        if (paired)                                                                                                    \
            return inverse ? launch_image<ImageThreads<RX>::value>(dev, ifft2d_pad_kernel<RX, RYV, true, ImageThreads<RX>::value>, smem, p, st, "ifft2d_pad_kernel<%d,%d,paired,%d>", RX, RYV)   \
                           : launch_image<ImageThreads<RX>::value>(dev, fft2d_trunc_kernel<RX, RYV, true, ImageThreads<RX>::value>, smem, p, st, "fft2d_trunc_kernel<%d,%d,paired,%d>", RX, RYV); \
        if (p.centered_x) return TFNO_ERR_UNSUPPORTED;      /* centered modes only with 16-byte aligned rows */             \
        return inverse ? launch_image<kThreads>(dev, ifft2d_pad_kernel<RX, RYV, false, kThreads>, smem, p, st, "ifft2d_pad_kernel<%d,%d,scalar,%d>", RX, RYV)         \
                       : launch_image<kThreads>(dev, fft2d_trunc_kernel<RX, RYV, false, kThreads>, smem, p, st, "fft2d_trunc_kernel<%d,%d,scalar,%d>", RX, RYV);
    switch (RY) { TFNO_IMG(2) TFNO_IMG(4) }
#undef TFNO_IMG
    return TFNO_ERR_UNSUPPORTED;
}
// DX = 256: image kernels on the 32-point transform, 16 warps per CTA
template <typename Kernel>
inline int launch_image32(const DeviceInfo& dev, Kernel kernel, int DX, int DY, const ImageParams& p, cudaStream_t st, const char* name,
                          int a, int b, int c = 0) {
    const size_t smem = image32_smem_bytes(DX, DY);
    if ((long long)smem > dev.max_smem_optin) return TFNO_ERR_UNSUPPORTED;
    if (record_launch(dev, name, a, b, c)) return TFNO_OK;
    int occ = 0;
    int rc = prepare_kernel(kernel, smem, dev, &occ, kImage32Threads);
    if (rc != TFNO_OK) return rc;
    long long grid = (long long)dev.sms * occ;
    if (grid > p.nimg) grid = p.nimg;
    kernel<<<(unsigned)grid, kImage32Threads, smem, st>>>(p);
    return launch_status();
}
inline int launch_fft2d_32(const DeviceInfo& dev, int DY, const ImageParams& p, bool inverse, cudaStream_t st) {
    const bool conj = p.conj_inverse != 0;
    if (DY == 256) {
        if (!inverse) return launch_image32(dev, fft2d_trunc32_kernel<8, 8>, 256, 256, p, st, "fft2d_trunc32_kernel<%d,%d>", 8, 8);
        return conj ? launch_image32(dev, ifft2d_pad32_kernel<8, 8, true>, 256, 256, p, st, "ifft2d_pad32_kernel<%d,%d,%d>", 8, 8, 1)
                    : launch_image32(dev, ifft2d_pad32_kernel<8, 8, false>, 256, 256, p, st, "ifft2d_pad32_kernel<%d,%d,%d>", 8, 8, 0);
    }
    if (!inverse) return launch_image32(dev, fft2d_trunc32_kernel<8, 4>, 256, 128, p, st, "fft2d_trunc32_kernel<%d,%d>", 8, 4);
    return conj ? launch_image32(dev, ifft2d_pad32_kernel<8, 4, true>, 256, 128, p, st, "ifft2d_pad32_kernel<%d,%d,%d>", 8, 4, 1)
                : launch_image32(dev, ifft2d_pad32_kernel<8, 4, false>, 256, 128, p, st, "ifft2d_pad32_kernel<%d,%d,%d>", 8, 4, 0);
}

// whole-image kernels exist for DX, DY in {128, 256} (a 512-row intermediate would need 256 KB)
inline int launch_fft2d(const DeviceInfo& dev, int DX, int DY, const ImageParams& p, bool inverse, cudaStream_t st) {
    if (p.nimg <= 0) return TFNO_OK;
    // DX = 256: the forward image kernel on the 32-point transform (16 warps) is faster at both row
    // lengths (bs=64 K=N=64 256x256: 0.528 -> 0.480 ms), the inverse one only at DY = 128 (at
    // DY = 256 it takes 0.596 ms against 0.528 for the 64-point kernel) -- measured, kernel by kernel.
    if (DX == 256 && (DY == 128 || (DY == 256 && !inverse))) return launch_fft2d_32(dev, DY, p, inverse, st);
    switch (DX / 64) {
        case 2: return launch_fft2d_rx<2>(dev, DY / 64, p, inverse, st);
        case 4: return launch_fft2d_rx<4>(dev, DY / 64, p, inverse, st);
    }
    return TFNO_ERR_UNSUPPORTED;
}

}  // namespace tfno

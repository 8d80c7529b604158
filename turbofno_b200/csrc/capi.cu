// C ABI of turbofno_b200: handle / plan / exec and the stage-level entry points.
// Declarations and the reference interfaces they replace: include/turbofno_b200.h.
#include <cublas_v2.h>
#include <cufft.h>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <new>

#include "launch.cuh"

using namespace tfno;

struct tfno_handle_s {
    DeviceInfo dev;
};

struct HostStaging {
    bool ready = false;
    long long chunk_rows = 0;           // batch items per pipeline chunk
    long long chunk_override = 0;       // set by tfno_plan_set_host_chunk before the first host call
    float2* dx[2] = {nullptr, nullptr};
    float2* dy[2] = {nullptr, nullptr};
    void* dws[2] = {nullptr, nullptr};
    float2* dw[2] = {nullptr, nullptr}; // one copy of the weights per stream: no ordering between the two needed
    cudaStream_t stream[2] = {nullptr, nullptr};
    tfno_plan_s* chunk_plan = nullptr;  // plan for chunk_rows batch items
    tfno_plan_s* tail_plan = nullptr;   // plan for the last, shorter chunk (if any)
    long long tail_rows = 0;
};

struct tfno_plan_s {
    tfno_handle_s* h = nullptr;
    tfno_problem p{};
    long long B = 0;                    // 1D: bs*dimX rows; 2D: bs images per channel
    size_t ws_bytes = 0;
    bool default_layout = true;
    bool per_mode = false;              // per-mode weights (w_stride_m != 0)
    // variant E
    cufftHandle fft_fwd = 0, fft_inv = 0;
    bool have_fft = false;
    cublasHandle_t blas = nullptr;
    HostStaging host;
};

namespace {

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline float2 f2(float a, float b) { return make_float2(a, b); }
inline float2 cscale(float2 a, float s) { return make_float2(a.x * s, a.y * s); }
inline size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

long long image_elems(const tfno_problem& p) { return (long long)p.DX * p.DY; }

// workspace carving: A/S (spectrum of x), C (spectrum of y), T1/T2 (X-transformed 64-row images),
// F (full-size transform buffer of the library path)
struct Workspace {
    size_t offA = 0, offC = 0, offT1 = 0, offT2 = 0, offF = 0, total = 0;
};

size_t weight_bytes(const tfno_plan_s& pl) {
    const tfno_problem& p = pl.p;
    const size_t nmodes = !pl.per_mode ? 1 : (p.rank == 1 ? (size_t)kModes : (size_t)kModes * kModes);
    return sizeof(float2) * (size_t)p.K * p.N * nmodes;
}

Workspace carve(const tfno_plan_s& pl) {
    const tfno_problem& p = pl.p;
    Workspace w;
    const long long per_row = (p.rank == 1) ? kModes : (long long)kModes * kModes;
    const size_t szA = align_up(sizeof(float2) * (size_t)(p.K * pl.B * per_row));
    const size_t szC = align_up(sizeof(float2) * (size_t)(p.N * pl.B * per_row));
    size_t off = 0;
    auto take = [&](size_t& slot, size_t sz) { slot = off; off += sz; };
    int v = p.variant;
    if (p.w_stride_m != 0 && p.rank == 1) v = TFNO_VARIANT_A;      // per-mode weights: three kernels, spectra A and C in the workspace
    if (p.rank == 1) {
        if (v == TFNO_VARIANT_A || v == TFNO_VARIANT_C || v == TFNO_VARIANT_E) take(w.offA, szA);
        if (v == TFNO_VARIANT_A || v == TFNO_VARIANT_B || v == TFNO_VARIANT_E) take(w.offC, szC);
        if (v == TFNO_VARIANT_E) take(w.offF, align_up(sizeof(float2) * (size_t)(p.K * pl.B * p.DY)));
    } else {
        const size_t szT1 = align_up(sizeof(float2) * (size_t)(p.K * pl.B * kModes * p.DY));
        const size_t szT2 = align_up(sizeof(float2) * (size_t)(p.N * pl.B * kModes * p.DY));
        if (v == TFNO_VARIANT_A || v == TFNO_VARIANT_C || v == TFNO_VARIANT_D || v == TFNO_VARIANT_E) take(w.offA, szA);
        if (v == TFNO_VARIANT_A || v == TFNO_VARIANT_B || v == TFNO_VARIANT_D || v == TFNO_VARIANT_E) take(w.offC, szC);
        if (v == TFNO_VARIANT_A || v == TFNO_VARIANT_B || v == TFNO_VARIANT_C) { take(w.offT1, szT1); take(w.offT2, szT2); }
        if (v == TFNO_VARIANT_E) take(w.offF, align_up(sizeof(float2) * (size_t)(p.K * pl.B * image_elems(p))));
    }
    w.total = off;
    return w;
}

int validate(const tfno_problem& p) {
    if (p.rank != 1 && p.rank != 2) return TFNO_ERR_INVALID_ARG;
    if (p.bs <= 0 || p.K <= 0 || p.N <= 0) return TFNO_ERR_INVALID_ARG;
    if (p.rank == 1 && p.dimX <= 0) return TFNO_ERR_INVALID_ARG;
    if (p.variant < TFNO_VARIANT_A || p.variant > TFNO_VARIANT_E) return TFNO_ERR_INVALID_ARG;
    if (p.modes != kModes) return TFNO_ERR_UNSUPPORTED;
    if (!supported_len(p.DY)) return TFNO_ERR_UNSUPPORTED;
    if (p.rank == 2 && !supported_len(p.DX)) return TFNO_ERR_UNSUPPORTED;
    if (p.K % kSlabK != 0 || p.N % 64 != 0) return TFNO_ERR_UNSUPPORTED;
    if (p.rank == 2 && p.variant == TFNO_VARIANT_D && (p.DX > 256 || p.DY > 256)) return TFNO_ERR_UNSUPPORTED;
    // centered X modes: the whole-image kernels of the 2D variant D, true inverse only
    if (p.x_modes_centered && (p.rank != 2 || p.variant != TFNO_VARIANT_D || p.second_transform_forward)) return TFNO_ERR_UNSUPPORTED;
    if (p.w_stride_m != 0) {
        // per-mode weights: transform ; per-mode contraction ; transform
        const bool ok_variant = (p.rank == 1) ? (p.variant == TFNO_VARIANT_A || p.variant == TFNO_VARIANT_D) : (p.variant == TFNO_VARIANT_D);
        if (!ok_variant || p.K > 96 || p.beta_re != 0.f || p.beta_im != 0.f) return TFNO_ERR_UNSUPPORTED;
        if (p.rank == 2 && (p.DX > 256 || p.DY > 256)) return TFNO_ERR_UNSUPPORTED;
    }
    return TFNO_OK;
}

void host_staging_free(HostStaging& hs) {
    for (int i = 0; i < 2; ++i) {
        if (hs.dx[i]) cudaFree(hs.dx[i]);
        if (hs.dy[i]) cudaFree(hs.dy[i]);
        if (hs.dws[i]) cudaFree(hs.dws[i]);
        if (hs.dw[i]) cudaFree(hs.dw[i]);
        if (hs.stream[i]) cudaStreamDestroy(hs.stream[i]);
        hs.dx[i] = hs.dy[i] = hs.dw[i] = nullptr;
        hs.dws[i] = nullptr;
        hs.stream[i] = nullptr;
    }
    if (hs.chunk_plan) tfno_plan_destroy(hs.chunk_plan);
    if (hs.tail_plan) tfno_plan_destroy(hs.tail_plan);
    hs.chunk_plan = hs.tail_plan = nullptr;
    hs.ready = false;
}

}  // namespace

extern "C" {

const char* tfno_status_string(int status) {
    switch (status) {
        case TFNO_OK: return "ok";
        case TFNO_ERR_INVALID_ARG: return "invalid argument (null or misaligned pointer, non-positive size)";
        case TFNO_ERR_UNSUPPORTED: return "unsupported size (need DY,DX in {128,256,512,1024}, K%8==0, N%64==0, modes==64)";
        case TFNO_ERR_CUDA: return "CUDA runtime call or kernel launch failed";
        case TFNO_ERR_ALLOC: return "allocation failed";
        case TFNO_ERR_LIBRARY: return "cuFFT or cuBLAS call failed";
        case TFNO_ERR_WORKSPACE: return "workspace pointer missing";
        case TFNO_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the library's static 64 MiB array holds";
        case TFNO_ERR_KERNEL_WAIT: return "a kernel-side wait ran out; the output is incomplete (see tfno_device_status)";
    }
    return "unknown status";
}

int tfno_problem_init(tfno_problem* p, int rank) {
    if (!p || (rank != 1 && rank != 2)) return TFNO_ERR_INVALID_ARG;
    std::memset(p, 0, sizeof(*p));
    p->rank = rank;
    p->bs = 1;
    p->dimX = 1;
    p->DX = rank == 2 ? 256 : 1;
    p->DY = 256;
    p->K = 64;
    p->N = 64;
    p->modes = kModes;
    p->variant = TFNO_VARIANT_D;
    p->alpha_re = 1.f;
    p->scale_inverse = 1;
    return TFNO_OK;
}

int tfno_create(tfno_handle** out, int device) {
    if (!out) return TFNO_ERR_INVALID_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count <= 0) { cudaGetLastError(); return TFNO_ERR_CUDA; }
    if (device < 0 || device >= count) return TFNO_ERR_INVALID_ARG;
    tfno_handle_s* h = new (std::nothrow) tfno_handle_s();
    if (!h) return TFNO_ERR_ALLOC;
    h->dev.device = device;
    if (cudaDeviceGetAttribute(&h->dev.sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&h->dev.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) {
        cudaGetLastError();
        delete h;
        return TFNO_ERR_CUDA;
    }
    {
        DeviceGuard guard(device);
        if (!guard.ok || cudaMalloc(&h->dev.status, sizeof(int)) != cudaSuccess ||
            cudaMemset(h->dev.status, 0, sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            delete h;
            return TFNO_ERR_ALLOC;
        }
    }
    const char* no_tc = std::getenv("TFNO_DISABLE_TENSOR_CORES");
    h->dev.use_tensor_cores = !(no_tc && no_tc[0] == '1');
    *out = h;
    return TFNO_OK;
}

int tfno_destroy(tfno_handle* h) {
    if (!h) return TFNO_OK;
    if (h->dev.status) {
        DeviceGuard guard(h->dev.device);
        cudaFree(h->dev.status);
    }
    delete h;
    return TFNO_OK;
}

int tfno_device_status(tfno_handle* h, int* out) {
    if (!h || !out) return TFNO_ERR_INVALID_ARG;
    DeviceGuard guard(h->dev.device);
    // every stream of the device, non-blocking ones included, before the word is read
    if (!guard.ok || cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(out, h->dev.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return TFNO_ERR_CUDA;
    }
    return TFNO_OK;
}

int tfno_device_status_reset(tfno_handle* h) {
    if (!h) return TFNO_ERR_INVALID_ARG;
    DeviceGuard guard(h->dev.device);
    if (!guard.ok || cudaMemset(h->dev.status, 0, sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        return TFNO_ERR_CUDA;
    }
    return TFNO_OK;
}

// One warp waits on a barrier that nothing ever completes.  The wait gives up after its limit (one
// second), records code 99 in the status word and the kernel returns normally: the error path of
// every kernel-side wait of this library, made to happen without any fault.
__global__ void bounded_wait_selftest_kernel(int* status) {
    __shared__ uint64_t bar_storage;
    __shared__ int abort_storage;
    const uint32_t bar = tc::smem_u32(&bar_storage);
    if (threadIdx.x == 0) {
        tc::mbar_init(bar, 1);
        abort_storage = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    tc::mbar_wait(bar, 0, &abort_storage, status, 99, tc::kHelperIdleNs);
}

int tfno_selftest_bounded_wait(tfno_handle* h, void* stream) {
    if (!h) return TFNO_ERR_INVALID_ARG;
    DeviceGuard guard(h->dev.device);
    if (!guard.ok) return TFNO_ERR_CUDA;
    bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(h->dev.status);
    return launch_status();
}

int tfno_sm_count(const tfno_handle* h, int* out) {
    if (!h || !out) return TFNO_ERR_INVALID_ARG;
    *out = h->dev.sms;
    return TFNO_OK;
}

int tfno_plan_destroy(tfno_plan* plan) {
    if (!plan) return TFNO_OK;
    DeviceGuard guard(plan->h->dev.device);
    if (plan->have_fft) { cufftDestroy(plan->fft_fwd); cufftDestroy(plan->fft_inv); }
    if (plan->blas) cublasDestroy(plan->blas);
    host_staging_free(plan->host);
    delete plan;
    return TFNO_OK;
}

int tfno_plan_create(tfno_handle* h, const tfno_problem* problem, tfno_plan** out) {
    if (!h || !problem || !out) return TFNO_ERR_INVALID_ARG;
    *out = nullptr;
    int rc = validate(*problem);
    if (rc != TFNO_OK) return rc;
    tfno_plan_s* pl = new (std::nothrow) tfno_plan_s();
    if (!pl) return TFNO_ERR_ALLOC;
    pl->h = h;
    pl->p = *problem;
    tfno_problem& p = pl->p;
    pl->B = (p.rank == 1) ? p.bs * p.dimX : p.bs;
    const long long unit = (p.rank == 1) ? p.DY : image_elems(p);
    const long long nmodes = (p.rank == 1) ? kModes : (long long)kModes * kModes;
    pl->per_mode = p.w_stride_m != 0;
    const bool w_default = pl->per_mode ? (p.w_stride_k == 0 || (p.w_stride_m == 1 && p.w_stride_k == nmodes && p.w_stride_n == p.K * nmodes))
                                        : (p.w_stride_k == 0 || (p.w_stride_k == 1 && p.w_stride_n == p.K));
    pl->default_layout = (p.x_stride_b == 0 || (p.x_stride_b == unit && p.x_stride_k == pl->B * unit)) &&
                         (p.y_stride_b == 0 || (p.y_stride_b == unit && p.y_stride_n == pl->B * unit)) && w_default;
    if (p.x_stride_b == 0) { p.x_stride_b = unit; p.x_stride_k = pl->B * unit; }
    if (p.y_stride_b == 0) { p.y_stride_b = unit; p.y_stride_n = pl->B * unit; }
    if (pl->per_mode && p.w_stride_k == 0) { p.w_stride_m = 1; p.w_stride_k = nmodes; p.w_stride_n = p.K * nmodes; }
    if (p.w_stride_k == 0) { p.w_stride_k = 1; p.w_stride_n = p.K; }
    if ((p.x_stride_b | p.x_stride_k | p.y_stride_b | p.y_stride_n) & 1) {   // 16-byte alignment of rows
        delete pl;
        return TFNO_ERR_INVALID_ARG;
    }
    pl->ws_bytes = carve(*pl).total;

    if (p.variant == TFNO_VARIANT_E) {
        if (!pl->default_layout) { delete pl; return TFNO_ERR_UNSUPPORTED; }
        DeviceGuard guard(h->dev.device);
        if (!guard.ok) { delete pl; return TFNO_ERR_CUDA; }
        // handles per plan, as the reference creates them per configuration
        // (fusion_variants/1D_E_baseline/fused.cu:171-179); unlike the reference they are destroyed.
        if (cublasCreate(&pl->blas) != CUBLAS_STATUS_SUCCESS) { pl->blas = nullptr; tfno_plan_destroy(pl); return TFNO_ERR_LIBRARY; }
        cufftResult r1, r2;
        if (p.rank == 1) {
            r1 = cufftPlan1d(&pl->fft_fwd, p.DY, CUFFT_C2C, (int)(p.K * pl->B));
            r2 = (r1 == CUFFT_SUCCESS) ? cufftPlan1d(&pl->fft_inv, p.DY, CUFFT_C2C, (int)(p.N * pl->B)) : r1;
        } else {
            int n[2] = {p.DX, p.DY};
            r1 = cufftPlanMany(&pl->fft_fwd, 2, n, nullptr, 1, p.DX * p.DY, nullptr, 1, p.DX * p.DY, CUFFT_C2C, (int)(p.K * pl->B));
            r2 = (r1 == CUFFT_SUCCESS)
                     ? cufftPlanMany(&pl->fft_inv, 2, n, nullptr, 1, p.DX * p.DY, nullptr, 1, p.DX * p.DY, CUFFT_C2C, (int)(p.N * pl->B))
                     : r1;
        }
        if (r1 != CUFFT_SUCCESS || r2 != CUFFT_SUCCESS) {
            if (r1 == CUFFT_SUCCESS) cufftDestroy(pl->fft_fwd);
            tfno_plan_destroy(pl);
            return TFNO_ERR_LIBRARY;
        }
        pl->have_fft = true;
    }
    *out = pl;
    return TFNO_OK;
}

size_t tfno_workspace_bytes(const tfno_plan* plan) { return plan ? plan->ws_bytes : 0; }

}  // extern "C"

// The dispatch of one layer.  With dev.record set it is a dry run: every launcher appends the
// name of the kernel it would launch and nothing touches the device.
static int exec_impl(const tfno_plan* plan, const DeviceInfo& dev, const void* x, const void* w, void* y, void* workspace,
                     void* stream) {
    const tfno_problem& p = plan->p;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const Workspace ws = carve(*plan);
    char* wsb = static_cast<char*>(workspace);
    float2* A = reinterpret_cast<float2*>(wsb + ws.offA);
    float2* C = reinterpret_cast<float2*>(wsb + ws.offC);
    float2* T1 = reinterpret_cast<float2*>(wsb + ws.offT1);
    float2* T2 = reinterpret_cast<float2*>(wsb + ws.offT2);
    float2* F = reinterpret_cast<float2*>(wsb + ws.offF);

    const float2 alpha = f2(p.alpha_re, p.alpha_im), beta = f2(p.beta_re, p.beta_im);
    const int conj = p.second_transform_forward ? 0 : 1;
    const float scale = p.scale_inverse ? 1.0f / (p.rank == 1 ? (float)p.DY : (float)p.DX * (float)p.DY) : 1.0f;
    const long long B = plan->B;
    const float2* xin = static_cast<const float2*>(x);
    const float2* win = static_cast<const float2*>(w);
    float2* yout = static_cast<float2*>(y);
    int rc = TFNO_OK;

    // operand descriptions reused below
    TileParams t{};
    t.K = p.K; t.N = p.N;
    t.w = win; t.w_stride_k = p.w_stride_k; t.w_stride_n = p.w_stride_n;
    t.alpha = alpha; t.beta = beta; t.conj_inverse = conj;

    if (p.rank == 1) {
        const long long M = B * kModes;
        (void)M;
        RowsParams fr{};   // x -> A
        fr.nsig = p.K * B; fr.per_k = B; fr.in = xin; fr.out = A; fr.stride_row = p.x_stride_b; fr.stride_k = p.x_stride_k;
        RowsParams ir{};   // C -> y
        ir.nsig = p.N * B; ir.per_k = B; ir.in = C; ir.out = yout; ir.stride_row = p.y_stride_b; ir.stride_k = p.y_stride_n;
        ir.gain = f2(scale, 0.f); ir.conj_inverse = conj;
        t.rows = B;
        if (plan->per_mode) {
            rc = launch_fft_rows(dev, p.DY, fr, st);
            if (rc) return rc;
            PerModeParams pm{};
            pm.rows = B; pm.modes = kModes; pm.K = p.K; pm.N = p.N;
            pm.a = A; pm.w = win; pm.w_sk = p.w_stride_k; pm.w_sn = p.w_stride_n; pm.w_sm = p.w_stride_m;
            pm.c = C; pm.alpha = alpha;
            rc = launch_permode(dev, pm, st);
            if (rc) return rc;
            return launch_ifft_rows(dev, p.DY, ir, st);
        }
        switch (p.variant) {
            case TFNO_VARIANT_A:
                rc = launch_fft_rows(dev, p.DY, fr, st);
                if (rc) return rc;
                t.x = A; t.y = C;
                rc = launch_tile<false, false>(dev, p.DY, t, st);
                if (rc) return rc;
                return launch_ifft_rows(dev, p.DY, ir, st);
            case TFNO_VARIANT_B:
                t.x = xin; t.x_stride_row = p.x_stride_b; t.x_stride_k = p.x_stride_k; t.y = C;
                rc = launch_tile<true, false>(dev, p.DY, t, st);
                if (rc) return rc;
                return launch_ifft_rows(dev, p.DY, ir, st);
            case TFNO_VARIANT_C:
                rc = launch_fft_rows(dev, p.DY, fr, st);
                if (rc) return rc;
                t.x = A; t.y = yout; t.y_stride_row = p.y_stride_b; t.y_stride_n = p.y_stride_n;
                t.inv_gain = cscale(alpha, scale);
                return launch_tile<false, true>(dev, p.DY, t, st);
            case TFNO_VARIANT_D:
                t.x = xin; t.x_stride_row = p.x_stride_b; t.x_stride_k = p.x_stride_k;
                t.y = yout; t.y_stride_row = p.y_stride_b; t.y_stride_n = p.y_stride_n;
                t.inv_gain = cscale(alpha, scale);
                return launch_tile<true, true>(dev, p.DY, t, st);
            default: break;
        }
    } else {
        const long long rows = B * kModes;       // 64-mode row tiles: one per (batch, kx)
        ImageParams fi{};  // x -> A
        fi.nimg = p.K * B; fi.per_k = B; fi.in = xin; fi.out = A; fi.stride_b = p.x_stride_b; fi.stride_k = p.x_stride_k;
        ImageParams ii{};  // C -> y
        ii.nimg = p.N * B; ii.per_k = B; ii.in = C; ii.out = yout; ii.stride_b = p.y_stride_b; ii.stride_k = p.y_stride_n;
        ii.gain = f2(scale, 0.f); ii.conj_inverse = conj;
        fi.centered_x = ii.centered_x = p.x_modes_centered ? 1 : 0;
        ColsParams fc{};   // x -> T1  [K*B][64][DY]
        fc.nimg = p.K * B; fc.per_k = B; fc.DY = p.DY; fc.in = xin; fc.out = T1; fc.stride_b = p.x_stride_b; fc.stride_k = p.x_stride_k;
        ColsParams ic{};   // T2 -> y
        ic.nimg = p.N * B; ic.per_k = B; ic.DY = p.DY; ic.in = T2; ic.out = yout; ic.stride_b = p.y_stride_b; ic.stride_k = p.y_stride_n;
        ic.gain = f2(scale, 0.f); ic.conj_inverse = conj;
        RowsParams fr{};   // T1 -> A   (compact both sides)
        fr.nsig = p.K * rows; fr.per_k = p.K * rows; fr.in = T1; fr.out = A; fr.stride_row = p.DY; fr.stride_k = 0;
        RowsParams ir{};   // C -> T2
        ir.nsig = p.N * rows; ir.per_k = p.N * rows; ir.in = C; ir.out = T2; ir.stride_row = p.DY; ir.stride_k = 0;
        ir.gain = f2(1.f, 0.f); ir.conj_inverse = conj;
        t.rows = rows;
        if (plan->per_mode) {
            rc = launch_fft2d(dev, p.DX, p.DY, fi, false, st);
            if (rc) return rc;
            PerModeParams pm{};
            pm.rows = B; pm.modes = (long long)kModes * kModes; pm.K = p.K; pm.N = p.N;
            pm.a = A; pm.w = win; pm.w_sk = p.w_stride_k; pm.w_sn = p.w_stride_n; pm.w_sm = p.w_stride_m;
            pm.c = C; pm.alpha = alpha;
            rc = launch_permode(dev, pm, st);
            if (rc) return rc;
            return launch_fft2d(dev, p.DX, p.DY, ii, true, st);
        }
        switch (p.variant) {
            case TFNO_VARIANT_D:
                rc = launch_fft2d(dev, p.DX, p.DY, fi, false, st);
                if (rc) return rc;
                t.x = A; t.y = C;
                t.beta = f2(0.f, 0.f);      // D ignores beta in both ranks (the spectrum buffer C is scratch)
                rc = launch_tile<false, false>(dev, p.DY, t, st);
                if (rc) return rc;
                return launch_fft2d(dev, p.DX, p.DY, ii, true, st);
            case TFNO_VARIANT_A:
                rc = launch_fft_cols(dev, p.DX, fc, st);
                if (rc) return rc;
                rc = launch_fft_rows(dev, p.DY, fr, st);
                if (rc) return rc;
                t.x = A; t.y = C;
                rc = launch_tile<false, false>(dev, p.DY, t, st);
                if (rc) return rc;
                rc = launch_ifft_rows(dev, p.DY, ir, st);
                if (rc) return rc;
                return launch_ifft_cols(dev, p.DX, ic, st);
            case TFNO_VARIANT_B:
                rc = launch_fft_cols(dev, p.DX, fc, st);
                if (rc) return rc;
                t.x = T1; t.x_stride_row = p.DY; t.x_stride_k = rows * p.DY; t.y = C;
                rc = launch_tile<true, false>(dev, p.DY, t, st);
                if (rc) return rc;
                rc = launch_ifft_rows(dev, p.DY, ir, st);
                if (rc) return rc;
                return launch_ifft_cols(dev, p.DX, ic, st);
            case TFNO_VARIANT_C:
                rc = launch_fft_cols(dev, p.DX, fc, st);
                if (rc) return rc;
                rc = launch_fft_rows(dev, p.DY, fr, st);
                if (rc) return rc;
                t.x = A; t.y = T2; t.y_stride_row = p.DY; t.y_stride_n = rows * p.DY;
                t.inv_gain = alpha;
                rc = launch_tile<false, true>(dev, p.DY, t, st);
                if (rc) return rc;
                return launch_ifft_cols(dev, p.DX, ic, st);
            default: break;
        }
    }

    // ---- variant E: cuFFT -> truncate -> cuBLAS CGEMM -> zero-pad -> cuFFT ----------------------
    // call sequence of fusion_variants/1D_E_baseline/fused.cu:200-216 and
    // fusion_variants/2D_E_baseline/fused_trunc_2D.cu:238-253, stream-ordered, without the host
    // synchronisation after every step.  The 1/len scale rides on alpha (beta must then be 0 for
    // FNO semantics; with scale_inverse = 0 any beta behaves as in the reference).
    if (dev.record) {
        record_launch(dev, "cufftExecC2C");
        record_launch(dev, p.rank == 1 ? "truncate_rows_kernel" : "truncate_corner_kernel");
        record_launch(dev, "cublasCgemm");
        record_launch(dev, p.rank == 1 ? "zero_pad_rows_kernel" : "zero_pad_corner_kernel");
        record_launch(dev, "cufftExecC2C");
        return TFNO_OK;
    }
    if (cufftSetStream(plan->fft_fwd, st) != CUFFT_SUCCESS || cufftSetStream(plan->fft_inv, st) != CUFFT_SUCCESS ||
        cublasSetStream(plan->blas, st) != CUBLAS_STATUS_SUCCESS)
        return TFNO_ERR_LIBRARY;
    if (cufftExecC2C(plan->fft_fwd, (cufftComplex*)xin, (cufftComplex*)F, CUFFT_FORWARD) != CUFFT_SUCCESS)
        return TFNO_ERR_LIBRARY;
    const int copy_blocks = dev.sms * 8;
    const long long per_row = (p.rank == 1) ? kModes : (long long)kModes * kModes;
    const long long Mlib = B * per_row;
    if (p.rank == 1)
        truncate_rows_kernel<<<copy_blocks, 256, 0, st>>>((const float4*)F, (float4*)A, p.K * B, p.DY);
    else
        truncate_corner_kernel<<<copy_blocks, 256, 0, st>>>((const float4*)F, (float4*)A, p.K * B, p.DX, p.DY);
    if ((rc = launch_status())) return rc;
    const float2 a2 = cscale(alpha, scale);
    if (cublasCgemm(plan->blas, CUBLAS_OP_N, CUBLAS_OP_N, (int)Mlib, p.N, p.K, (const cuComplex*)&a2, (const cuComplex*)A,
                    (int)Mlib, (const cuComplex*)win, p.K, (const cuComplex*)&beta, (cuComplex*)C, (int)Mlib) !=
        CUBLAS_STATUS_SUCCESS)
        return TFNO_ERR_LIBRARY;
    if (p.rank == 1)
        zero_pad_rows_kernel<<<copy_blocks, 256, 0, st>>>((const float4*)C, (float4*)yout, p.N * B, p.DY);
    else
        zero_pad_corner_kernel<<<copy_blocks, 256, 0, st>>>((const float4*)C, (float4*)yout, p.N * B, p.DX, p.DY);
    if ((rc = launch_status())) return rc;
    if (cufftExecC2C(plan->fft_inv, (cufftComplex*)yout, (cufftComplex*)yout, conj ? CUFFT_INVERSE : CUFFT_FORWARD) !=
        CUFFT_SUCCESS)
        return TFNO_ERR_LIBRARY;
    return TFNO_OK;
}

extern "C" {

int tfno_exec(const tfno_plan* plan, const void* x, const void* w, void* y, void* workspace, void* stream) {
    if (!plan || !x || !w || !y) return TFNO_ERR_INVALID_ARG;
    if (!aligned16(x) || !aligned16(y) || !aligned16(w) || !aligned16(workspace)) return TFNO_ERR_INVALID_ARG;
    if (plan->ws_bytes > 0 && !workspace) return TFNO_ERR_WORKSPACE;
    const DeviceInfo& dev = plan->h->dev;
    DeviceGuard guard(dev.device);
    if (!guard.ok) return TFNO_ERR_CUDA;
    return exec_impl(plan, dev, x, w, y, workspace, stream);
}

int tfno_plan_kernels(const tfno_plan* plan, char* buf, size_t cap) {
    if (!plan || !buf || cap < 2) return TFNO_ERR_INVALID_ARG;
    buf[0] = 0;
    DeviceInfo dev = plan->h->dev;
    dev.record = buf;
    dev.record_cap = cap;
    // dry run over stand-in operands: 256-byte aligned, never dereferenced
    char* fake = reinterpret_cast<char*>(static_cast<uintptr_t>(1) << 20);
    return exec_impl(plan, dev, fake, fake, fake, fake, nullptr);
}

// ------------------------------------------------------------------------------------------------
// Host-buffer execution: batch chunks pipelined over two streams (copy-in, layer, copy-out each
// stream-ordered; the two streams overlap one another's copies and kernels).
// ------------------------------------------------------------------------------------------------
static int host_staging_init(tfno_plan_s* plan) {
    HostStaging& hs = plan->host;
    if (hs.ready) return TFNO_OK;
    const tfno_problem& p = plan->p;
    const long long unit = (p.rank == 1) ? (long long)p.dimX * p.DY : image_elems(p);   // elements per batch item and channel
    // Chunk size: about 64 MiB of input, but at least eight chunks per call when the batch allows
    // it, so that copy-in, layer and copy-out of neighbouring chunks overlap on the two streams
    // also for a small batch (a shard of a multi-GPU job).
    long long chunk = (64LL << 20) / (long long)(sizeof(float2) * unit * p.K);
    if (chunk > (p.bs + 7) / 8) chunk = (p.bs + 7) / 8;
    if (hs.chunk_override > 0) chunk = hs.chunk_override;
    if (chunk < 1) chunk = 1;
    if (chunk > p.bs) chunk = p.bs;
    hs.chunk_rows = chunk;
    hs.tail_rows = p.bs % chunk;
    tfno_problem cp = p;
    cp.bs = chunk;
    cp.x_stride_b = cp.x_stride_k = cp.y_stride_b = cp.y_stride_n = 0;
    int rc = tfno_plan_create(plan->h, &cp, &hs.chunk_plan);
    if (rc == TFNO_OK && hs.tail_rows) {
        cp.bs = hs.tail_rows;
        rc = tfno_plan_create(plan->h, &cp, &hs.tail_plan);
    }
    if (rc == TFNO_OK) {
        const size_t xin = sizeof(float2) * (size_t)(unit * p.K * chunk), yout = sizeof(float2) * (size_t)(unit * p.N * chunk);
        const size_t wsz = hs.chunk_plan->ws_bytes;
        for (int i = 0; i < 2 && rc == TFNO_OK; ++i) {
            if (cudaMalloc(&hs.dx[i], xin) != cudaSuccess || cudaMalloc(&hs.dy[i], yout) != cudaSuccess ||
                (wsz && cudaMalloc(&hs.dws[i], wsz) != cudaSuccess) ||
                cudaMalloc(&hs.dw[i], weight_bytes(*plan)) != cudaSuccess ||
                cudaStreamCreateWithFlags(&hs.stream[i], cudaStreamNonBlocking) != cudaSuccess) {
                cudaGetLastError();
                rc = TFNO_ERR_ALLOC;
            }
        }
    }
    if (rc != TFNO_OK) {
        host_staging_free(hs);          // nothing half-built survives a failed set-up
        return rc;
    }
    hs.ready = true;
    return TFNO_OK;
}

int tfno_plan_set_host_chunk(tfno_plan* plan, long long batch_items) {
    if (!plan || batch_items < 0) return TFNO_ERR_INVALID_ARG;
    if (plan->host.ready) return TFNO_ERR_INVALID_ARG;      // staging already sized
    plan->host.chunk_override = batch_items;
    return TFNO_OK;
}

int tfno_exec_host(tfno_plan* plan, const void* x_host, const void* w_host, void* y_host) {
    if (!plan || !x_host || !w_host || !y_host) return TFNO_ERR_INVALID_ARG;
    if (!plan->default_layout) return TFNO_ERR_UNSUPPORTED;
    DeviceGuard guard(plan->h->dev.device);
    if (!guard.ok) return TFNO_ERR_CUDA;
    int rc = host_staging_init(plan);
    if (rc) return rc;
    HostStaging& hs = plan->host;
    const tfno_problem& p = plan->p;
    const long long unit = (p.rank == 1) ? (long long)p.dimX * p.DY : image_elems(p);
    const size_t full_pitch = sizeof(float2) * (size_t)(unit * p.bs);   // bytes between channels on the host
    // On any failure: wait for what is already in flight (the copies read and write caller-owned
    // host buffers) before returning.
    auto fail = [&](int code) {
        cudaStreamSynchronize(hs.stream[0]);
        cudaStreamSynchronize(hs.stream[1]);
        cudaGetLastError();
        return code;
    };
    int slot = 0;
    long long chunk_index = 0;
    for (long long b0 = 0; b0 < p.bs; b0 += hs.chunk_rows, slot ^= 1, ++chunk_index) {
        const long long nb = (p.bs - b0 < hs.chunk_rows) ? p.bs - b0 : hs.chunk_rows;
        tfno_plan_s* cp = (nb == hs.chunk_rows) ? hs.chunk_plan : hs.tail_plan;
        const size_t width = sizeof(float2) * (size_t)(unit * nb);
        cudaStream_t st = hs.stream[slot];
        // each stream brings its own copy of the weights with its first chunk (stream-ordered
        // before that chunk's kernels; no host synchronisation, no ordering between the streams)
        if (chunk_index < 2 &&
            cudaMemcpyAsync(hs.dw[slot], w_host, weight_bytes(*plan), cudaMemcpyHostToDevice, st) != cudaSuccess)
            return fail(TFNO_ERR_CUDA);
        // [K][bs][unit] on the host -> compact [K][nb][unit] on the device
        if (cudaMemcpy2DAsync(hs.dx[slot], width, static_cast<const char*>(x_host) + sizeof(float2) * (size_t)(unit * b0),
                              full_pitch, width, (size_t)p.K, cudaMemcpyHostToDevice, st) != cudaSuccess)
            return fail(TFNO_ERR_CUDA);
        rc = tfno_exec(cp, hs.dx[slot], hs.dw[slot], hs.dy[slot], hs.dws[slot], st);
        if (rc) return fail(rc);
        if (cudaMemcpy2DAsync(static_cast<char*>(y_host) + sizeof(float2) * (size_t)(unit * b0), full_pitch, hs.dy[slot], width,
                              width, (size_t)p.N, cudaMemcpyDeviceToHost, st) != cudaSuccess)
            return fail(TFNO_ERR_CUDA);
    }
    if (cudaStreamSynchronize(hs.stream[0]) != cudaSuccess || cudaStreamSynchronize(hs.stream[1]) != cudaSuccess) {
        cudaGetLastError();
        return TFNO_ERR_CUDA;
    }
    // y is complete only if no kernel-side wait ran out
    int word = 0;
    if (plan->h->dev.status &&
        cudaMemcpy(&word, plan->h->dev.status, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return TFNO_ERR_CUDA;
    }
    return word == 0 ? TFNO_OK : TFNO_ERR_KERNEL_WAIT;
}

// ------------------------------------------------------------------------------------------------
// Stage-level entry points
// ------------------------------------------------------------------------------------------------
static int check_stage(tfno_handle* h, const void* a, const void* b, const void* c) {
    if (!h || !a || !b || !c) return TFNO_ERR_INVALID_ARG;
    if (!aligned16(a) || !aligned16(b) || !aligned16(c)) return TFNO_ERR_INVALID_ARG;
    return TFNO_OK;
}

static TileParams stage_tile(long long M, int N, int K, const void* in, const void* B, void* out, float ar, float ai,
                             float br, float bi) {
    TileParams t{};
    t.rows = M / kModes; t.K = K; t.N = N;
    t.x = static_cast<const float2*>(in);
    t.w = static_cast<const float2*>(B); t.w_stride_k = 1; t.w_stride_n = K;
    t.y = static_cast<float2*>(out);
    t.alpha = f2(ar, ai); t.beta = f2(br, bi);
    t.inv_gain = t.alpha; t.conj_inverse = 1;
    return t;
}

int tfno_fused_fft_cgemm_ifft(tfno_handle* h, int log2_len, long long M, int N, int K, const void* in, const void* B,
                              void* C, void* out, float ar, float ai, float br, float bi, void* stream) {
    (void)C;
    int rc = check_stage(h, in, B, out);
    if (rc) return rc;
    if (M <= 0 || M % kModes) return TFNO_ERR_INVALID_ARG;
    if (log2_len < 7 || log2_len > 10) return TFNO_ERR_UNSUPPORTED;
    DeviceGuard guard(h->dev.device);
    const int len = 1 << log2_len;
    TileParams t = stage_tile(M, N, K, in, B, out, ar, ai, br, bi);
    t.x_stride_row = len; t.x_stride_k = t.rows * len;
    t.y_stride_row = len; t.y_stride_n = t.rows * len;
    return launch_tile<true, true>(h->dev, len, t, static_cast<cudaStream_t>(stream));
}

int tfno_fused_fft_cgemm(tfno_handle* h, int log2_len, long long M, int N, int K, const void* in, const void* B, void* C,
                         float ar, float ai, float br, float bi, void* stream) {
    int rc = check_stage(h, in, B, C);
    if (rc) return rc;
    if (M <= 0 || M % kModes) return TFNO_ERR_INVALID_ARG;
    if (log2_len < 7 || log2_len > 10) return TFNO_ERR_UNSUPPORTED;
    DeviceGuard guard(h->dev.device);
    const int len = 1 << log2_len;
    TileParams t = stage_tile(M, N, K, in, B, C, ar, ai, br, bi);
    t.x_stride_row = len; t.x_stride_k = t.rows * len;
    return launch_tile<true, false>(h->dev, len, t, static_cast<cudaStream_t>(stream));
}

int tfno_fused_cgemm_ifft(tfno_handle* h, int log2_len, long long M, int N, int K, const void* A, const void* B, void* C,
                          void* out, float ar, float ai, float br, float bi, void* stream) {
    (void)C;
    int rc = check_stage(h, A, B, out);
    if (rc) return rc;
    if (M <= 0 || M % kModes) return TFNO_ERR_INVALID_ARG;
    if (log2_len < 7 || log2_len > 10) return TFNO_ERR_UNSUPPORTED;
    DeviceGuard guard(h->dev.device);
    const int len = 1 << log2_len;
    TileParams t = stage_tile(M, N, K, A, B, out, ar, ai, br, bi);
    t.y_stride_row = len; t.y_stride_n = t.rows * len;
    return launch_tile<false, true>(h->dev, len, t, static_cast<cudaStream_t>(stream));
}

int tfno_cgemm(tfno_handle* h, long long M, int N, int K, const void* A, const void* B, void* C, float ar, float ai,
               float br, float bi, void* stream) {
    int rc = check_stage(h, A, B, C);
    if (rc) return rc;
    if (M <= 0 || M % kModes) return TFNO_ERR_INVALID_ARG;
    DeviceGuard guard(h->dev.device);
    TileParams t = stage_tile(M, N, K, A, B, C, ar, ai, br, bi);
    return launch_tile<false, false>(h->dev, 128, t, static_cast<cudaStream_t>(stream));
}

static RowsParams stage_rows(int len, const void* in, void* out, long long total, bool forward) {
    RowsParams r{};
    r.nsig = total; r.per_k = total > 0 ? total : 1;
    r.in = static_cast<const float2*>(in); r.out = static_cast<float2*>(out);
    r.stride_row = len; r.stride_k = 0;
    r.gain = f2(1.f, 0.f); r.conj_inverse = 1;
    (void)forward;
    return r;
}

int tfno_fft_stride_DY(tfno_handle* h, int log2_len, const void* in, void* out, long long total, void* stream) {
    int rc = check_stage(h, in, out, out);
    if (rc) return rc;
    if (total < 0) return TFNO_ERR_INVALID_ARG;
    if (log2_len < 7 || log2_len > 10) return TFNO_ERR_UNSUPPORTED;
    if (total == 0) return TFNO_OK;
    DeviceGuard guard(h->dev.device);
    return launch_fft_rows(h->dev, 1 << log2_len, stage_rows(1 << log2_len, in, out, total, true), static_cast<cudaStream_t>(stream));
}

int tfno_ifft_stride_DY(tfno_handle* h, int log2_len, const void* in, void* out, long long total, void* stream) {
    int rc = check_stage(h, in, out, out);
    if (rc) return rc;
    if (total < 0) return TFNO_ERR_INVALID_ARG;
    if (log2_len < 7 || log2_len > 10) return TFNO_ERR_UNSUPPORTED;
    if (total == 0) return TFNO_OK;
    DeviceGuard guard(h->dev.device);
    return launch_ifft_rows(h->dev, 1 << log2_len, stage_rows(1 << log2_len, in, out, total, false), static_cast<cudaStream_t>(stream));
}

static int stage_cols(tfno_handle* h, int log2_len, const void* in, void* out, int DY, long long total_columns, bool fwd,
                      void* stream) {
    int rc = check_stage(h, in, out, out);
    if (rc) return rc;
    if (DY <= 0 || (DY & 1) || total_columns < 0 || total_columns % DY) return TFNO_ERR_INVALID_ARG;
    if (log2_len < 7 || log2_len > 10) return TFNO_ERR_UNSUPPORTED;
    if (total_columns == 0) return TFNO_OK;
    DeviceGuard guard(h->dev.device);
    const int len = 1 << log2_len;
    ColsParams c{};
    c.nimg = total_columns / DY; c.per_k = c.nimg; c.DY = DY;
    c.in = static_cast<const float2*>(in); c.out = static_cast<float2*>(out);
    c.stride_b = (long long)len * DY; c.stride_k = 0;
    c.gain = f2(1.f, 0.f); c.conj_inverse = 1;
    return fwd ? launch_fft_cols(h->dev, len, c, static_cast<cudaStream_t>(stream))
               : launch_ifft_cols(h->dev, len, c, static_cast<cudaStream_t>(stream));
}

int tfno_fft_stride(tfno_handle* h, int log2_len, const void* in, void* out, int DY, long long total_columns, void* stream) {
    return stage_cols(h, log2_len, in, out, DY, total_columns, true, stream);
}
int tfno_ifft_stride(tfno_handle* h, int log2_len, const void* in, void* out, int DY, long long total_columns, void* stream) {
    return stage_cols(h, log2_len, in, out, DY, total_columns, false, stream);
}


// ------------------------------------------------------------------------------------------------
// Allocation-free 2D layer
//
// Some hosts of this library may not allocate device memory at the point where they run a layer:
// code inside a memory-pool or arena scheme that owns every byte of the device and hands none
// back, real-time / safety-reviewed pipelines that forbid allocation after start-up, and callers
// that sit between another framework's allocator calls where an extra cudaMalloc would
// synchronise the device.  tfno_exec already allocates nothing, but the 2D path needs two
// spectrum-sized scratch buffers that those callers cannot provide.  This entry point keeps the
// scratch in a fixed device array that is part of the library image.
// ------------------------------------------------------------------------------------------------
namespace {

constexpr size_t kStaticScratchBytes = (size_t)64 << 20;     // 64 MiB per GPU that loads the library
static __device__ __align__(256) unsigned char tfno_static_scratch[kStaticScratchBytes];

constexpr int kMaxStaticDevices = 64;
struct StaticDevice {
    bool ready;
    unsigned char* scratch;     // device address of tfno_static_scratch on this device
    DeviceInfo dev;
};
StaticDevice g_static_devices[kMaxStaticDevices];   // zero-initialised, no heap

// once per device, with that device current: resolve the array's DEVICE address (the symbol's
// name in host code is only a host-side handle) and read the launch limits
int static_device_setup(int device, StaticDevice** out) {
    if (device < 0 || device >= kMaxStaticDevices) return TFNO_ERR_INVALID_ARG;
    StaticDevice& sd = g_static_devices[device];
    if (!sd.ready) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, tfno_static_scratch) != cudaSuccess || ptr == nullptr) {
            cudaGetLastError();
            return TFNO_ERR_CUDA;
        }
        sd.scratch = static_cast<unsigned char*>(ptr);
        sd.dev = DeviceInfo();
        sd.dev.device = device;
        sd.dev.use_tensor_cores = false;
        if (cudaDeviceGetAttribute(&sd.dev.sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sd.dev.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device) != cudaSuccess) {
            cudaGetLastError();
            return TFNO_ERR_CUDA;
        }
        sd.ready = true;
    }
    *out = &sd;
    return TFNO_OK;
}

}  // namespace

size_t tfno_static_scratch_bytes(void) { return kStaticScratchBytes; }

int tfno_spectral_conv2d_static(long long bs, int DX, int DY, int K, int N, const void* x, const void* w, void* y,
                                float alpha_re, float alpha_im, void* stream) {
    if (!x || !w || !y || bs <= 0 || K <= 0 || N <= 0) return TFNO_ERR_INVALID_ARG;
    if (!aligned16(x) || !aligned16(w) || !aligned16(y)) return TFNO_ERR_INVALID_ARG;
    if ((DX != 128 && DX != 256) || (DY != 128 && DY != 256) || K % kSlabK != 0 || N % 64 != 0) return TFNO_ERR_UNSUPPORTED;
    // size check by division: no product of caller-given sizes is formed before it is known to fit
    constexpr size_t kPerChannelImage = sizeof(float2) * (size_t)kModes * kModes;      // 32 KiB of spectrum
    const size_t max_units = kStaticScratchBytes / kPerChannelImage;                     // (K + N) * bs may not exceed this
    if ((size_t)K > max_units || (size_t)N > max_units || (size_t)bs > max_units / ((size_t)K + (size_t)N))
        return TFNO_ERR_SCRATCH_LIMIT;
    const size_t spec_in = align_up(kPerChannelImage * (size_t)K * (size_t)bs);
    const size_t spec_out = align_up(kPerChannelImage * (size_t)N * (size_t)bs);
    if (spec_in + spec_out > kStaticScratchBytes) return TFNO_ERR_SCRATCH_LIMIT;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); return TFNO_ERR_CUDA; }
    StaticDevice* sd = nullptr;
    int rc = static_device_setup(device, &sd);
    if (rc != TFNO_OK) return rc;
    // every launch of this call must fit before the first one is enqueued: a refused call does nothing
    if ((long long)image_smem_bytes(DX, DY) > sd->dev.max_smem_optin ||
        (long long)tile_smem_bytes(2, false, false, K, N > 128 ? 128 : N) > sd->dev.max_smem_optin)
        return TFNO_ERR_UNSUPPORTED;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    float2* S = reinterpret_cast<float2*>(sd->scratch);
    float2* C = reinterpret_cast<float2*>(sd->scratch + spec_in);
    const long long img = (long long)DX * DY;

    // image transform, channel contraction, image inverse: the kernel sequence of a 2D variant-D
    // plan, except that the contraction always runs on the FP32 row-tile kernel (the tensor-core
    // contraction reports through a handle's status word, and this entry point has no handle).
    // Every scratch element that is read has been written by the preceding kernel of this call
    // (beta = 0), so nothing has to start at zero.
    ImageParams fi{};
    fi.nimg = K * bs; fi.per_k = bs; fi.in = static_cast<const float2*>(x); fi.out = S; fi.stride_b = img; fi.stride_k = bs * img;
    rc = launch_fft2d(sd->dev, DX, DY, fi, false, st);
    if (rc != TFNO_OK) return rc;
    TileParams t{};
    t.rows = bs * kModes; t.K = K; t.N = N;
    t.x = S; t.w = static_cast<const float2*>(w); t.w_stride_k = 1; t.w_stride_n = K; t.y = C;
    t.alpha = f2(alpha_re, alpha_im); t.beta = f2(0.f, 0.f); t.conj_inverse = 1;
    rc = launch_tile<false, false>(sd->dev, DY, t, st);
    if (rc != TFNO_OK) return rc;
    ImageParams ii{};
    ii.nimg = N * bs; ii.per_k = bs; ii.in = C; ii.out = static_cast<float2*>(y); ii.stride_b = img; ii.stride_k = bs * img;
    ii.gain = f2(1.0f / ((float)DX * (float)DY), 0.f); ii.conj_inverse = 1;
    return launch_fft2d(sd->dev, DX, DY, ii, true, st);
}

}  // extern "C"

// TurboFNO_{1D,2D}_{A,B,C,D,E}: one source, compiled once per (rank, variant) with
//   -DTFNO_RANK=1|2 -DTFNO_VARIANT=TFNO_VARIANT_x -DTFNO_TAG="1D_D" -DDEFAULT_CONFIG_PATH="..."
//
// Command line (superset of the reference's two driver flavours):
//   (no arguments)                 sweep the grid in DEFAULT_CONFIG_PATH
//                                  (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:79-103)
//   <bs> <dimX|DX> <DY> <N> <K>    one configuration
//                                  (fusion_variants_benchmark/1D_D_exp_fused_fft_cgemm_ifft/fused.cu:32-48)
//   --config <file>                sweep the grid in <file>
//   --stream                       time 20 back-to-back launches without host synchronisation
//                                  (default: 5 launches with a device synchronisation after each,
//                                  as the reference times them, fused.cu:135-139)
//   --as-shipped                   alpha=(1,-1), beta=(-1,1), second transform forward, unscaled:
//                                  the arithmetic the reference drivers run (fused.cu:76)
//   --json                         one JSON object per configuration instead of the text line
// Output line (fused.cu:146):  "1D_D, bs=%-4d, dimX=%-4d, DY=%-4d, N=%-4d, K=%-4d, TIME=%8.3fms"
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <fstream>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

#include "TurboFNO.h"
#include "driver_config.h"

#ifndef TFNO_RANK
#define TFNO_RANK 1
#endif
#ifndef TFNO_VARIANT
#define TFNO_VARIANT TFNO_VARIANT_D
#endif
#ifndef TFNO_TAG
#define TFNO_TAG "1D_D"
#endif
#ifndef DEFAULT_CONFIG_PATH
#define DEFAULT_CONFIG_PATH "benchmark_config/problem_size_1d.txt"
#endif

namespace {

struct Config { long long bs; int d1; int DY; int N; int K; };   // d1 = dimX (1D) or DX (2D)

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    fprintf(stderr, "%s: CUDA error: %s\n", what, cudaGetErrorString(e));
    return false;
}

// counter-based fill: value i depends only on (seed, i)
void fill_uniform(std::vector<float>& v, uint64_t seed) {
    for (size_t i = 0; i < v.size(); ++i) {
        uint64_t z = seed + 0x9E3779B97F4A7C15ull * (i + 1);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        v[i] = (float)((double)(z >> 11) * (2.0 / 9007199254740992.0) - 1.0);
    }
}

long long in_elems(const Config& c) { return TFNO_RANK == 1 ? c.bs * c.d1 * c.DY * c.K : c.bs * (long long)c.d1 * c.DY * c.K; }
long long out_elems(const Config& c) { return TFNO_RANK == 1 ? c.bs * c.d1 * c.DY * c.N : c.bs * (long long)c.d1 * c.DY * c.N; }

}  // namespace

int main(int argc, char** argv) {
    std::string config_path = DEFAULT_CONFIG_PATH;
    bool stream_mode = false, as_shipped = false, json = false;
    std::vector<long long> positional;
    for (int i = 1; i < argc; ++i) {
        std::string a = argv[i];
        if (a == "--stream") stream_mode = true;
        else if (a == "--as-shipped") as_shipped = true;
        else if (a == "--json") json = true;
        else if (a == "--config" && i + 1 < argc) config_path = argv[++i];
        else if (!a.empty() && (isdigit((unsigned char)a[0]))) positional.push_back(atoll(a.c_str()));
        else {
            fprintf(stderr, "Usage: %s [<bs> <%s> <DY> <N> <K>] [--config file] [--stream] [--as-shipped] [--json]\n", argv[0],
                    TFNO_RANK == 1 ? "dimX" : "DX");
            return 2;
        }
    }
    std::vector<Config> configs;
    if (!positional.empty()) {
        if (positional.size() != 5) {
            fprintf(stderr, "Usage: %s <bs> <%s> <DY> <N> <K>\n", argv[0], TFNO_RANK == 1 ? "dimX" : "DX");
            return 2;
        }
        configs.push_back({positional[0], (int)positional[1], (int)positional[2], (int)positional[3], (int)positional[4]});
    } else {
        std::ifstream f(config_path);
        if (!f) { fprintf(stderr, "cannot open config file %s\n", config_path.c_str()); return 2; }
        std::stringstream ss; ss << f.rdbuf();
        auto grid = tfno_driver::parse_config(ss.str());
        const char* k1 = TFNO_RANK == 1 ? "dimX_list" : "DX_list";
        for (int bs : grid["bs_list"]) for (int d1 : grid[k1]) for (int DY : grid["DY_list"])
            for (int N : grid["N_list"]) for (int K : grid["K_list"]) configs.push_back({bs, d1, DY, N, K});
        if (configs.empty()) { fprintf(stderr, "config file %s defines an empty grid\n", config_path.c_str()); return 2; }
    }

    tfno_handle* h = nullptr;
    int rc = tfno_create(&h, 0);
    if (rc) { fprintf(stderr, "tfno_create: %s\n", tfno_status_string(rc)); return 1; }

    // one allocation sized for the largest configuration that fits in free memory
    size_t free_b = 0, total_b = 0;
    if (!cuda_ok(cudaMemGetInfo(&free_b, &total_b), "cudaMemGetInfo")) return 1;
    int failures = 0;
    for (const Config& c : configs) {
        tfno_problem p;
        tfno_problem_init(&p, TFNO_RANK);
        p.bs = c.bs; p.DY = c.DY; p.N = c.N; p.K = c.K; p.variant = TFNO_VARIANT;
        if (TFNO_RANK == 1) p.dimX = c.d1; else p.DX = c.d1;
        if (as_shipped) { p.alpha_re = 1.f; p.alpha_im = -1.f; p.beta_re = -1.f; p.beta_im = 1.f; p.second_transform_forward = 1; p.scale_inverse = 0; }
        tfno_plan* plan = nullptr;
        rc = tfno_plan_create(h, &p, &plan);
        if (rc) {
            fprintf(stderr, "%s, bs=%lld d=%d DY=%d N=%d K=%d: %s\n", TFNO_TAG, c.bs, c.d1, c.DY, c.N, c.K, tfno_status_string(rc));
            ++failures;
            continue;
        }
        const size_t xb = sizeof(float2) * (size_t)in_elems(c), yb = sizeof(float2) * (size_t)out_elems(c);
        const size_t wb = sizeof(float2) * (size_t)c.K * c.N, wsb = tfno_workspace_bytes(plan);
        if (xb + yb + wb + wsb + (256u << 20) > free_b) {
            fprintf(stderr, "%s, bs=%lld d=%d DY=%d N=%d K=%d: skipped, needs %.1f GB of device memory\n", TFNO_TAG, c.bs, c.d1, c.DY,
                    c.N, c.K, (xb + yb + wb + wsb) / 1e9);
            tfno_plan_destroy(plan);
            continue;
        }
        float2 *dx = nullptr, *dy = nullptr, *dw = nullptr; void* dws = nullptr;
        bool ok = cuda_ok(cudaMalloc(&dx, xb), "cudaMalloc x") && cuda_ok(cudaMalloc(&dy, yb), "cudaMalloc y") &&
                  cuda_ok(cudaMalloc(&dw, wb), "cudaMalloc w") && (wsb == 0 || cuda_ok(cudaMalloc(&dws, wsb), "cudaMalloc workspace"));
        if (ok) {
            // host fill in slices of at most 64 Mi floats
            const size_t slice = 64u << 20;
            std::vector<float> hbuf(std::min(slice, (size_t)in_elems(c) * 2));
            for (size_t off = 0; off < (size_t)in_elems(c) * 2 && ok; off += slice) {
                size_t n = std::min(slice, (size_t)in_elems(c) * 2 - off);
                hbuf.resize(n);
                fill_uniform(hbuf, 1234 + off);
                ok = cuda_ok(cudaMemcpy((float*)dx + off, hbuf.data(), n * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy x");
            }
            std::vector<float> hw((size_t)c.K * c.N * 2);
            fill_uniform(hw, 4321);
            const float s = 1.0f / std::sqrt((float)c.K);
            for (float& v : hw) v *= s;
            ok = ok && cuda_ok(cudaMemcpy(dw, hw.data(), wb, cudaMemcpyHostToDevice), "cudaMemcpy w");
            if (wsb) ok = ok && cuda_ok(cudaMemset(dws, 0, wsb), "cudaMemset workspace");
        }
        float ms = 0.f;
        if (ok) {
            rc = tfno_exec(plan, dx, dw, dy, dws, nullptr);          // warm-up, checked
            ok = (rc == TFNO_OK) && cuda_ok(cudaDeviceSynchronize(), "warm-up");
            if (rc) fprintf(stderr, "tfno_exec: %s\n", tfno_status_string(rc));
        }
        if (ok) {
            cudaEvent_t e0, e1;
            cudaEventCreate(&e0); cudaEventCreate(&e1);
            const int reps = stream_mode ? 20 : ntest;
            cudaEventRecord(e0);
            for (int i = 0; i < reps && rc == TFNO_OK; ++i) {
                rc = tfno_exec(plan, dx, dw, dy, dws, nullptr);
                if (!stream_mode) cudaDeviceSynchronize();
            }
            cudaEventRecord(e1);
            ok = cuda_ok(cudaEventSynchronize(e1), "timed loop") && rc == TFNO_OK;
            cudaEventElapsedTime(&ms, e0, e1);
            ms /= reps;
            cudaEventDestroy(e0); cudaEventDestroy(e1);
        }
        if (ok) {
            if (json) {
                const double bytes = 8.0 * (double)(TFNO_RANK == 1 ? c.bs * c.d1 * c.DY : c.bs * (long long)c.d1 * c.DY) * (c.K + c.N);
                printf("{\"tag\": \"%s\", \"bs\": %lld, \"%s\": %d, \"DY\": %d, \"N\": %d, \"K\": %d, \"time_ms\": %.4f, "
                       "\"layers_per_s\": %.2f, \"algorithmic_GBps\": %.1f}\n",
                       TFNO_TAG, c.bs, TFNO_RANK == 1 ? "dimX" : "DX", c.d1, c.DY, c.N, c.K, ms, 1000.0 / ms, bytes / ms * 1e-6);
            } else if (TFNO_RANK == 1) {
                printf("%s, bs=%-4d, dimX=%-4d, DY=%-4d, N=%-4d, K=%-4d, TIME=%8.3fms\n", TFNO_TAG, (int)c.bs, c.d1, c.DY, c.N, c.K, ms);
            } else {
                printf("%s, bs=%-4d, DX=%-4d, DY=%-4d, N=%-4d, K=%-4d, TIME=%8.3fms\n", TFNO_TAG, (int)c.bs, c.d1, c.DY, c.N, c.K, ms);
            }
            fflush(stdout);
        } else {
            ++failures;
        }
        cudaFree(dx); cudaFree(dy); cudaFree(dw); cudaFree(dws);
        tfno_plan_destroy(plan);
    }
    // a kernel-side wait that ran out leaves outputs incomplete without failing any call: read the
    // device's status word once, after everything has been timed
    int status_word = 0;
    if (tfno_device_status(h, &status_word) != TFNO_OK || status_word != 0) {
        fprintf(stderr, "%s: device status word %d after the run (a kernel-side wait ran out)\n", TFNO_TAG, status_word);
        ++failures;
    }
    tfno_destroy(h);
    return failures ? 1 : 0;
}

/* CPU oracle for the FNO spectral-convolution path, plain C + OpenMP.
 *
 * TEST INFRASTRUCTURE ONLY: linked or loaded by tests/, __graft_entry__.smoke() and
 * bench.py's cpu_baseline / --impl reference legs; never by the shipped library.
 *
 * PARITY UNPINNED BY THE REFERENCE: TurboFNO has no tests, golden vectors or fixtures and no
 * driver of it copies a result back to the host.  This restatement is pinned against analytic
 * known-answer cases and against an independent numpy (pocketfft) restatement in
 * oracle/oracle_np.py; tests/test_oracle.py holds both checks.
 *
 * The reference ships no CPU implementation of this path.  The float instantiation
 * (oracle_spectral_conv{1d,2d}_f32) therefore doubles as the timed CPU baseline ("port"):
 * same math, all host threads, single precision like the GPU path.
 *
 * Build: gcc -O3 -march=native -fopenmp -shared -fPIC spectral_oracle.c -o liboracle.so -lm  */
#include <math.h>
#include <omp.h>
#include <stdlib.h>

/* tw[2j], tw[2j+1] = cos, -sin of 2 pi j / n for j < n/2 (forward-transform twiddles). */
static double* twiddles(int n) {
    double* tw = (double*)malloc(sizeof(double) * (size_t)n);
    if (!tw) return 0;
    for (int j = 0; j < n / 2; ++j) {
        double a = -2.0 * M_PI * (double)j / (double)n;
        tw[2 * j] = cos(a);
        tw[2 * j + 1] = sin(a);
    }
    return tw;
}

#define CAT2(a, b) a##b
#define CAT(a, b) CAT2(a, b)

#define REAL double
#define FN(name) CAT(name, _f64)
#include "spectral_oracle_impl.inc"
#undef REAL
#undef FN

#define REAL float
#define FN(name) CAT(name, _f32)
#include "spectral_oracle_impl.inc"
#undef REAL
#undef FN

int oracle_max_threads(void) { return omp_get_max_threads(); }

// Host-side check of the register FFT arithmetic in turbofno_b200/csrc/fft64.cuh.
// The lane-local functions are compiled for the CPU; the xor-shuffle exchange of
// forward_trunc() is replayed over an array of R emulated lanes.  Prints the maximum absolute
// error against a direct double-precision DFT for every supported group size.
#include <complex>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "../../turbofno_b200/csrc/fft64.cuh"

using cd = std::complex<double>;
using namespace tfno;

static double urand() { return 2.0 * rand() / RAND_MAX - 1.0; }

template <int R>
static double check_forward() {
    constexpr int DY = 64 * R;
    std::vector<cd> x(DY);
    for (auto& e : x) e = cd(urand(), urand());
    std::vector<float2> twF(R * 64);
    fill_forward_table<R>(twF.data(), 0, 1);
    static float2 v[R][64];
    for (int r = 0; r < R; ++r) {
        for (int n = 0; n < 64; ++n) v[r][n] = make_float2((float)x[R * n + r].real(), (float)x[R * n + r].imag());
        forward_local<R>(v[r], twF.data(), r);
    }
    // exchange rounds, as in forward_trunc()
    float2 t[R][64];
    for (int r = 0; r < R; ++r) for (int j = 0; j < 32; ++j) t[r][j] = cadd(v[r][slot(j)], v[r ^ (R >> 1)][slot(32 + j)]);
    for (int r = 0; r < R; ++r) for (int j = 0; j < 32; ++j) v[r][slot(j)] = t[r][j];
    for (int h = R >> 2, len = 16; h >= 1; h >>= 1, len >>= 1) {
        float2 send[R][32];
        for (int r = 0; r < R; ++r) for (int j = 0; j < len; ++j) send[r][j] = (r & h) ? v[r][slot(j)] : v[r][slot(len + j)];
        for (int r = 0; r < R; ++r) for (int j = 0; j < len; ++j) {
            float2 keep = (r & h) ? v[r][slot(len + j)] : v[r][slot(j)];
            v[r][slot(j)] = cadd(keep, send[r ^ h][j]);
        }
    }
    double err = 0;
    for (int r = 0; r < R; ++r) for (int j = 0; j < 64 / R; ++j) {
        int k = 64 / R * r + j;
        cd ref = 0;
        for (int n = 0; n < DY; ++n) ref += x[n] * std::polar(1.0, -2.0 * kPi * (double)((long)n * k % DY) / DY);
        cd got(v[r][slot(j)].x, v[r][slot(j)].y);
        err = std::max(err, std::abs(got - ref));
    }
    return err;
}

template <int R>
static double check_inverse(bool conj) {
    constexpr int DY = 64 * R;
    std::vector<cd> c(64);
    for (auto& e : c) e = cd(urand(), urand());
    float2 g = make_float2(0.5f, -0.25f);
    std::vector<float2> twI(R * 64);
    fill_inverse_table<R>(twI.data(), 0, 1, g, conj);
    double err = 0;
    for (int j1 = 0; j1 < R; ++j1) {
        float2 v[64];
        for (int m = 0; m < 64; ++m) v[m] = make_float2((float)c[m].real(), (float)c[m].imag());
        if (conj) inverse_pad_lane<+1, R>(v, twI.data(), j1); else inverse_pad_lane<-1, R>(v, twI.data(), j1);
        for (int j2 = 0; j2 < 64; ++j2) {
            int j = R * j2 + j1;
            cd ref = 0;
            for (int m = 0; m < 64; ++m) ref += c[m] * std::polar(1.0, (conj ? 2.0 : -2.0) * kPi * (double)((long)j * m % DY) / DY);
            ref *= cd(g.x, g.y);
            cd got(v[slot(j2)].x, v[slot(j2)].y);
            err = std::max(err, std::abs(got - ref));
        }
    }
    return err;
}

int main() {
    srand(7);
    printf("fwd2 %.3e\nfwd4 %.3e\nfwd8 %.3e\nfwd16 %.3e\n", check_forward<2>(), check_forward<4>(), check_forward<8>(), check_forward<16>());
    printf("inv2 %.3e\ninv4 %.3e\ninv8 %.3e\ninv16 %.3e\n", check_inverse<2>(true), check_inverse<4>(true), check_inverse<8>(true), check_inverse<16>(true));
    printf("fwdagain4 %.3e\n", check_inverse<4>(false));
    return 0;
}

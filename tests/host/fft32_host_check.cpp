// Host-side check of the register FFT arithmetic in turbofno_b200/csrc/fft32.cuh.
// The lane-local functions are compiled for the CPU; the xor-shuffle exchange rounds of
// forward_trunc32() are replayed over an array of R emulated lanes.  Prints the maximum absolute
// error against a direct double-precision DFT for every supported group size.
#include <complex>
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "../../turbofno_b200/csrc/fft32.cuh"

using cd = std::complex<double>;
using namespace tfno;

static double urand() { return 2.0 * rand() / RAND_MAX - 1.0; }

static double check_fft32(float s) {
    std::vector<cd> x(32);
    for (auto& e : x) e = cd(urand(), urand());
    float2 v[32];
    for (int n = 0; n < 32; ++n) v[n] = make_float2((float)x[n].real(), (float)x[n].imag());
    fft32<-1>(v, s);
    double err = 0;
    for (int k = 0; k < 32; ++k) {
        const int kk = s < 0 ? (k + 16) & 31 : k;
        cd ref = 0;
        for (int n = 0; n < 32; ++n) ref += x[n] * std::polar(1.0, -2.0 * kPi * (double)(n * kk % 32) / 32);
        err = std::max(err, std::abs(cd(v[slot32(k)].x, v[slot32(k)].y) - ref));
    }
    return err;
}

template <int R>
static double check_forward() {
    constexpr int DY = 32 * R;
    std::vector<cd> x(DY);
    for (auto& e : x) e = cd(urand(), urand());
    std::vector<float2> twF(R * 32);
    fill_forward_table32<R>(twF.data(), 0, 1);
    static float2 v[R][32];
    for (int r = 0; r < R; ++r) {
        for (int n = 0; n < 32; ++n) v[r][n] = make_float2((float)x[R * n + r].real(), (float)x[R * n + r].imag());
        forward_local32<R>(v[r], twF.data(), r);
    }
    // round 1: every value crosses, own + coef * received
    {
        static float2 t[R][32];
        for (int r = 0; r < R; ++r)
            for (int j = 0; j < 32; ++j) t[r][j] = cmadd(v[r][j], round1_coef32<R>(r), v[r ^ (R >> 1)][j]);
        for (int r = 0; r < R; ++r) for (int j = 0; j < 32; ++j) v[r][j] = t[r][j];
    }
    // round 2: slots 16..31 go to the partner, no selects
    {
        static float2 t[R][16];
        const int h = R >> 2;
        for (int r = 0; r < R; ++r) for (int j = 0; j < 16; ++j) t[r][j] = cadd(v[r][slot32(j)], v[r ^ h][slot32(16 + j)]);
        for (int r = 0; r < R; ++r) for (int j = 0; j < 16; ++j) v[r][slot32(j)] = t[r][j];
    }
    for (int h = R >> 3, len = 8; h >= 1; h >>= 1, len >>= 1) {
        static float2 send[R][16];
        for (int r = 0; r < R; ++r) for (int j = 0; j < len; ++j) send[r][j] = (r & h) ? v[r][slot32(j)] : v[r][slot32(len + j)];
        for (int r = 0; r < R; ++r) for (int j = 0; j < len; ++j) {
            float2 keep = (r & h) ? v[r][slot32(len + j)] : v[r][slot32(j)];
            v[r][slot32(j)] = cadd(keep, send[r ^ h][j]);
        }
    }
    double err = 0;
    for (int r = 0; r < R; ++r) for (int j = 0; j < 64 / R; ++j) {
        int k = 64 / R * r + j;
        cd ref = 0;
        for (int n = 0; n < DY; ++n) ref += x[n] * std::polar(1.0, -2.0 * kPi * (double)((long)n * k % DY) / DY);
        cd got(v[r][slot32(j)].x, v[r][slot32(j)].y);
        err = std::max(err, std::abs(got - ref));
    }
    return err;
}

template <int R>
static double check_inverse(bool conj) {
    constexpr int DY = 32 * R;
    std::vector<cd> c(64);
    for (auto& e : c) e = cd(urand(), urand());
    float2 g = make_float2(0.5f, -0.25f);
    std::vector<float2> twI(R * 64);
    fill_inverse_table32<R>(twI.data(), 0, 1, g, conj);
    double err = 0;
    for (int j1 = 0; j1 < R; ++j1) {
        float2 v[32];
        auto mode = [&](int m) { return make_float2((float)c[m].real(), (float)c[m].imag()); };
        if (conj) inverse_pad_lane32<+1, R>(v, twI.data(), j1, mode); else inverse_pad_lane32<-1, R>(v, twI.data(), j1, mode);
        for (int j2 = 0; j2 < 32; ++j2) {
            int j = R * j2 + j1;
            cd ref = 0;
            for (int m = 0; m < 64; ++m) ref += c[m] * std::polar(1.0, (conj ? 2.0 : -2.0) * kPi * (double)((long)j * m % DY) / DY);
            ref *= cd(g.x, g.y);
            cd got(v[slot32(j2)].x, v[slot32(j2)].y);
            err = std::max(err, std::abs(got - ref));
        }
    }
    return err;
}

// the folded form used by the fused kernel: 32 table entries per lane plus one constant
template <int R>
static double check_inverse_folded(bool conj) {
    constexpr int DY = 32 * R;
    std::vector<cd> c(64);
    for (auto& e : c) e = cd(urand(), urand());
    float2 g = make_float2(0.75f, 0.5f);
    std::vector<float2> twI(R * 32);
    fill_inverse_table32_folded<R>(twI.data(), 0, 1, g, conj);
    double err = 0;
    for (int j1 = 0; j1 < R; ++j1) {
        const float2 coef = inverse_fold_coef32<R>(j1, conj);
        float2 v[32];
        for (int m = 0; m < 32; ++m) {
            const float2 lo = make_float2((float)c[m].real(), (float)c[m].imag());
            const float2 hi = make_float2((float)c[m + 32].real(), (float)c[m + 32].imag());
            v[m] = cmul(cmadd(lo, coef, hi), twI[tw_index<R>(j1, m)]);
        }
        if (conj) fft32<+1>(v); else fft32<-1>(v);
        for (int j2 = 0; j2 < 32; ++j2) {
            int j = R * j2 + j1;
            cd ref = 0;
            for (int m = 0; m < 64; ++m) ref += c[m] * std::polar(1.0, (conj ? 2.0 : -2.0) * kPi * (double)((long)j * m % DY) / DY);
            ref *= cd(g.x, g.y);
            err = std::max(err, std::abs(cd(v[slot32(j2)].x, v[slot32(j2)].y) - ref));
        }
    }
    return err;
}

int main() {
    srand(11);
    printf("fft32 %.3e\nfft32rot %.3e\n", check_fft32(1.0f), check_fft32(-1.0f));
    printf("fwd4 %.3e\nfwd8 %.3e\nfwd16 %.3e\nfwd32 %.3e\n", check_forward<4>(), check_forward<8>(), check_forward<16>(), check_forward<32>());
    printf("inv4 %.3e\ninv8 %.3e\ninv16 %.3e\ninv32 %.3e\n", check_inverse<4>(true), check_inverse<8>(true), check_inverse<16>(true), check_inverse<32>(true));
    printf("fwdagain8 %.3e\n", check_inverse<8>(false));
    printf("invfold4 %.3e\ninvfold8 %.3e\nfwdagainfold8 %.3e\n", check_inverse_folded<4>(true), check_inverse_folded<8>(true), check_inverse_folded<8>(false));
    return 0;
}

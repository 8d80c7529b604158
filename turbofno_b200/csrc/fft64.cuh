// Register-resident 64-point complex FFT and the multi-lane truncated / zero-padded transforms
// built on it.
//
// Every transform of the spectral-convolution path keeps (forward) or starts from (inverse)
// exactly 64 modes, so one fully unrolled 64-point kernel with compile-time twiddles serves
// every signal length DY = 64*R, R in {2,4,8,16}:
//
//   forward, keep modes k<64 (role of the reference's fft_N_fused / fft_N_stride_DY device
//   code, whose sources are not in the reference tree; call sites
//   fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused_fft_cgemm_ifft_7.cuh:46,114):
//       X[k] = sum_{r<R} W_DY^{rk} F_r[k],   F_r = FFT64( x[R*n + r] )            (DIT, radix R last)
//     lane r of a group of R adjacent lanes owns F_r; the sum over r is a reduce-scatter over
//     the R lanes with xor-shuffles, after which lane r holds modes [64/R*r, 64/R*(r+1)).
//
//   inverse from 64 non-zero modes (role of fft_N_fused_output / ifft_N_stride_DY, call site
//   fused_fft_cgemm_ifft_7.cuh:218):
//       y[R*j2 + j1] = IFFT64_{m->j2}( C[m] * W_DY^{-j1*m} )                       (DIF, radix R first)
//     lane j1 owns residue class j1; every lane reads the same 64 modes, no exchange at all.
//
// The 64-point kernel is 8x8: eight radix-8 butterflies, 49 non-trivial constant twiddles,
// eight radix-8 butterflies.  Outputs stay in place, i.e. mode k = k1 + 8*k2 is found in
// register slot 8*k1 + k2 (see slot()).
#pragma once
#include <cuda_runtime.h>
#include <math.h>

#if defined(__CUDACC__)
#define TFNO_HD __host__ __device__ __forceinline__
#define TFNO_D __device__ __forceinline__
#else
#define TFNO_HD inline
#define TFNO_D inline
#endif

namespace tfno {

// ------------------------------------------------------------------------------------------
// compile-time sine / cosine (Taylor series in double on a reduced argument)
// ------------------------------------------------------------------------------------------
constexpr double kPi = 3.14159265358979323846264338327950288;

constexpr double cx_sin_small(double x) {   // |x| <= pi/4
    double term = x, sum = x;
    for (int i = 1; i < 12; ++i) { term *= -x * x / ((2.0 * i) * (2.0 * i + 1.0)); sum += term; }
    return sum;
}
constexpr double cx_cos_small(double x) {   // |x| <= pi/4
    double term = 1.0, sum = 1.0;
    for (int i = 1; i < 12; ++i) { term *= -x * x / ((2.0 * i - 1.0) * (2.0 * i)); sum += term; }
    return sum;
}
// cos and sin of 2*pi*num/den for integer num, den (den a multiple of 8), exact symmetries.
constexpr double cx_cos2pi(int num, int den) {
    num %= den; if (num < 0) num += den;
    if (num * 2 > den) return cx_cos2pi(den - num, den);            // cos(2pi - a) = cos a
    if (num * 4 > den) return -cx_cos2pi(den / 2 - num, den);       // cos(pi - a) = -cos a
    if (num * 8 > den) return cx_sin_small(2.0 * kPi * (den / 4 - num) / den);  // cos a = sin(pi/2 - a)
    return cx_cos_small(2.0 * kPi * num / den);
}
constexpr double cx_sin2pi(int num, int den) { return cx_cos2pi(num - den / 4, den); }

// ------------------------------------------------------------------------------------------
// tiny complex helpers on float2.  On sm_100 a complex add / subtract / real-scaled accumulate
// is ONE packed instruction (add.f32x2 / fma.rn.f32x2 on an aligned register pair); the host
// build and older targets fall back to two scalar operations.
// ------------------------------------------------------------------------------------------
#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ >= 1000)
#define TFNO_PACKED_F32X2 1
#endif

TFNO_HD float2 cadd(float2 a, float2 b) {
#ifdef TFNO_PACKED_F32X2
    return __fadd2_rn(a, b);
#else
    return make_float2(a.x + b.x, a.y + b.y);
#endif
}
TFNO_HD float2 csub(float2 a, float2 b) {
#ifdef TFNO_PACKED_F32X2
    return __ffma2_rn(b, make_float2(-1.0f, -1.0f), a);
#else
    return make_float2(a.x - b.x, a.y - b.y);
#endif
}
TFNO_HD float2 cmul(float2 a, float2 b) {
    return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
// a * (S*i): S=-1 gives -i*a (forward transform), S=+1 gives +i*a (inverse transform)
template <int S> TFNO_HD float2 mul_si(float2 a) {
    return S < 0 ? make_float2(a.y, -a.x) : make_float2(-a.y, a.x);
}
// e + s*t for a real factor held twice in s2 = (s, s)
TFNO_HD float2 cfma_s(float2 s2, float2 t, float2 e) {
#ifdef TFNO_PACKED_F32X2
    return __ffma2_rn(s2, t, e);
#else
    return make_float2(fmaf(s2.x, t.x, e.x), fmaf(s2.y, t.y, e.y));
#endif
}

// register slot holding mode k after fft64()
TFNO_HD constexpr int slot(int k) { return 8 * (k & 7) + (k >> 3); }

// ------------------------------------------------------------------------------------------
// 4-point and 8-point butterflies.  S = -1: e^{-2 pi i jk/n} (forward); S = +1: inverse.
// ------------------------------------------------------------------------------------------
template <int S>
TFNO_HD void dft4(float2& b0, float2& b1, float2& b2, float2& b3) {
    const float2 p0 = cadd(b0, b2), p1 = csub(b0, b2), p2 = cadd(b1, b3);
    // p3 = (S*i) * (b1 - b3), written component-wise so that the rotation costs no moves
    const float2 p3 = S < 0 ? make_float2(b1.y - b3.y, b3.x - b1.x) : make_float2(b3.y - b1.y, b1.x - b3.x);
    b0 = cadd(p0, p2); b2 = csub(p0, p2); b1 = cadd(p1, p3); b3 = csub(p1, p3);
}

// Real sign s = +-1 of the odd-indexed inputs of fft8(), in the forms its last stage consumes.
struct OddSign {
    float s, ns;          // s, -s
    float2 s2, ns2;       // (s, s), (-s, -s)
    float2 sh2, nsh2;     // (s*h, s*h), (-s*h, -s*h), h = sqrt(1/2)
};
TFNO_HD OddSign make_odd_sign(float s) {
    constexpr float h = 0.70710678118654752440f;
    OddSign o;
    o.s = s; o.ns = -s;
    o.s2 = make_float2(s, s); o.ns2 = make_float2(-s, -s);
    o.sh2 = make_float2(s * h, s * h); o.nsh2 = make_float2(-s * h, -s * h);
    return o;
}

// Decimation-in-time radix-8.  Inputs a[j] at a0..a7, outputs X[k] returned in place (a_k = X[k]).
// The odd-indexed inputs are taken as s*a[j] with a run-time s = +-1: negating the odd inputs
// rotates the output by four places, which the forward transform uses to make each lane's
// "keep" half land in fixed registers.  The sign rides on the multiply-accumulates of the last
// stage and costs nothing.
template <int S>
TFNO_HD void fft8(float2& a0, float2& a1, float2& a2, float2& a3, float2& a4, float2& a5, float2& a6,
                  float2& a7, const OddSign& sg) {
    float2 e0 = a0, e1 = a2, e2 = a4, e3 = a6;
    float2 o0 = a1, o1 = a3, o2 = a5, o3 = a7;
    dft4<S>(e0, e1, e2, e3);
    dft4<S>(o0, o1, o2, o3);
    // T[k] = O[k] * W8^k, W8 = e^{S*2 pi i/8}; the factor h of T1, T3 is folded into sh2 / nsh2,
    // the rotation T2 = (S*i)*O2 into the operand order of four scalar multiply-accumulates
    const float2 w1 = make_float2(o1.x - S * o1.y, o1.y + S * o1.x);
    const float2 w3 = make_float2(-o3.x - S * o3.y, -o3.y + S * o3.x);
    a0 = cfma_s(sg.s2, o0, e0);  a4 = cfma_s(sg.ns2, o0, e0);
    a1 = cfma_s(sg.sh2, w1, e1); a5 = cfma_s(sg.nsh2, w1, e1);
    a3 = cfma_s(sg.sh2, w3, e3); a7 = cfma_s(sg.nsh2, w3, e3);
    if (S < 0) {
        a2 = make_float2(fmaf(sg.s, o2.y, e2.x), fmaf(sg.ns, o2.x, e2.y));
        a6 = make_float2(fmaf(sg.ns, o2.y, e2.x), fmaf(sg.s, o2.x, e2.y));
    } else {
        a2 = make_float2(fmaf(sg.ns, o2.y, e2.x), fmaf(sg.s, o2.x, e2.y));
        a6 = make_float2(fmaf(sg.s, o2.y, e2.x), fmaf(sg.ns, o2.x, e2.y));
    }
}

template <int S, int N2, int K1>
TFNO_HD float2 twiddle64(float2 a) {   // a * e^{S*2 pi i*N2*K1/64}, constants folded at compile time
    constexpr int e = (N2 * K1) & 63;
    if constexpr (e == 0) return a;
    else if constexpr (e == 16) return mul_si<S>(a);
    else if constexpr (e == 32) return make_float2(-a.x, -a.y);
    else if constexpr (e == 48) return mul_si<-S>(a);
    else {
        constexpr float c = (float)cx_cos2pi(e, 64);
        constexpr float sn = (float)(S * cx_sin2pi(e, 64));
        return make_float2(a.x * c - a.y * sn, a.x * sn + a.y * c);
    }
}

template <int S, int K1>
TFNO_HD void twiddle_row(float2* v) {   // v[8*K1 + n2] *= W64^{n2*K1}, n2 = 1..7
    v[8 * K1 + 1] = twiddle64<S, 1, K1>(v[8 * K1 + 1]);
    v[8 * K1 + 2] = twiddle64<S, 2, K1>(v[8 * K1 + 2]);
    v[8 * K1 + 3] = twiddle64<S, 3, K1>(v[8 * K1 + 3]);
    v[8 * K1 + 4] = twiddle64<S, 4, K1>(v[8 * K1 + 4]);
    v[8 * K1 + 5] = twiddle64<S, 5, K1>(v[8 * K1 + 5]);
    v[8 * K1 + 6] = twiddle64<S, 6, K1>(v[8 * K1 + 6]);
    v[8 * K1 + 7] = twiddle64<S, 7, K1>(v[8 * K1 + 7]);
}

// 64-point transform, in registers.  In: v[n] = sample n.  Out: mode k in v[slot(k)].
// With s = -1 the odd samples are negated, i.e. the output is rotated by 32:
// v[slot(k)] then holds mode (k + 32) mod 64.
template <int S>
TFNO_HD void fft64(float2 (&v)[64], float s = 1.0f) {
    const OddSign plus = make_odd_sign(1.0f), sg = make_odd_sign(s);
    // step 1: for every n2, radix-8 over n1 on v[8*n1 + n2]; result k1 stored at v[8*k1 + n2]
#pragma unroll
    for (int n2 = 0; n2 < 8; ++n2)
        fft8<S>(v[n2], v[8 + n2], v[16 + n2], v[24 + n2], v[32 + n2], v[40 + n2], v[48 + n2], v[56 + n2], plus);
    // step 2: twiddles W64^{n2*k1}
    twiddle_row<S, 1>(v); twiddle_row<S, 2>(v); twiddle_row<S, 3>(v); twiddle_row<S, 4>(v);
    twiddle_row<S, 5>(v); twiddle_row<S, 6>(v); twiddle_row<S, 7>(v);
    // step 3: for every k1, radix-8 over n2 on v[8*k1 + n2]; result k2 stored at v[8*k1 + k2].
    // Sample parity equals the parity of n2, so the run-time sign enters here.
#pragma unroll
    for (int k1 = 0; k1 < 8; ++k1)
        fft8<S>(v[8 * k1], v[8 * k1 + 1], v[8 * k1 + 2], v[8 * k1 + 3], v[8 * k1 + 4], v[8 * k1 + 5],
                v[8 * k1 + 6], v[8 * k1 + 7], sg);
}

// ------------------------------------------------------------------------------------------
// Twiddle tables (shared memory), one row of 64 complex per lane of a group.
//
// forward:  twF[r][j] = W_DY^{r*k},  k = (j + 32*hi(r)) mod 64, hi(r) = top bit of r.
//           Lane r multiplies register slot(j) by twF[r][j]; the rotation by 32 matches the
//           s = -1 trick in fft64(), so that slots j<32 always hold the half the lane keeps in
//           the first exchange round.
// inverse:  twI[j1][m] = g * W_DY^{-j1*m} (conjugate), g = alpha * scale folded in.
// For an "inverse" that is really a second forward transform (the reference's variant E as
// shipped, fusion_variants/1D_E_baseline/fused.cu:190) conj = false.
// ------------------------------------------------------------------------------------------
// e^{sign * 2 pi i * e / n} for 0 <= e < n (n a power of two, so e/n is exact in float)
TFNO_HD float2 unit_root(int e, int n, float sign) {
    float sn, cs;
#if defined(__CUDA_ARCH__)
    sincospif(sign * 2.0f * (float)e / (float)n, &sn, &cs);
#else
    sn = (float)sin((double)sign * 2.0 * kPi * e / n);
    cs = (float)cos((double)sign * 2.0 * kPi * e / n);
#endif
    return make_float2(cs, sn);
}

// Table layout: the entries of mode pair (j, j+1) of the R lanes are adjacent -- element (r, j)
// sits at ((j/2)*R + r)*2 + (j&1) -- so that the R lanes of a group, which read the same pair in
// the same instruction, fetch one contiguous R*16-byte piece instead of R pieces in one bank.
template <int R>
TFNO_HD constexpr int tw_index(int r, int j) { return ((j >> 1) * R + r) * 2 + (j & 1); }

// `centered`: the kept modes are -32..31 instead of 0..63 (mode k of the result is k - 32 of the
// signal).  That is the transform of the signal times e^{+2 pi i 32 n / DY}, and for sample
// n = R*i + r this factor is (-1)^i * e^{+2 pi i 32 r / DY}: a sign on the lane's odd samples,
// which the 64-point transform applies for free (forward_local), and a constant per lane, which
// goes into the lane's row of this table.
template <int R>
TFNO_HD void fill_forward_table(float2* twF, int tid, int nthreads, bool centered = false) {
    constexpr int DY = 64 * R;
    for (int i = tid; i < R * 64; i += nthreads) {
        int r = i >> 6, j = i & 63;
        int k = (j + ((r & (R >> 1)) ? 32 : 0)) & 63;
        const int e = centered ? (r * k - 32 * r) & (DY - 1) : (r * k) & (DY - 1);
        twF[tw_index<R>(r, j)] = unit_root(e, DY, -1.0f);
    }
}

// `centered` (true inverse only): the 64 given modes are -32..31.  Sample R*j2 + j1 of the result
// is the ordinary one times e^{-2 pi i 32 (R*j2 + j1) / DY} = (-1)^j2 * e^{-2 pi i 32 j1 / DY}: the
// constant per lane goes into this table, the sign is a rotation of the transform's input by 32
// (inverse_pad_lane<CONJ, R, true>).
template <int R>
TFNO_HD void fill_inverse_table(float2* twI, int tid, int nthreads, float2 g, bool conj, bool centered = false) {
    constexpr int DY = 64 * R;
    for (int i = tid; i < R * 64; i += nthreads) {
        int j1 = i >> 6, m = i & 63;
        const int e = centered ? (j1 * m - 32 * j1) & (DY - 1) : (j1 * m) & (DY - 1);
        twI[tw_index<R>(j1, m)] = cmul(g, unit_root(e, DY, conj ? 1.0f : -1.0f));
    }
}

// Lane-local part of the forward transform: 64-point transform of the lane's decimated
// samples (rotated by 32 on the upper half of the group) and the W_DY^{rk} twiddles.
template <int R>
TFNO_HD void forward_local(float2 (&v)[64], const float2* __restrict__ twF, int r, bool centered = false) {
    const bool hi = (r & (R >> 1)) != 0;
    fft64<-1>(v, (hi != centered) ? -1.0f : 1.0f);
#pragma unroll
    for (int j = 0; j < 64; j += 2) {
        float4 t = *reinterpret_cast<const float4*>(twF + tw_index<R>(r, j));
        v[slot(j)] = cmul(v[slot(j)], make_float2(t.x, t.y));
        v[slot(j + 1)] = cmul(v[slot(j + 1)], make_float2(t.z, t.w));
    }
}

#if defined(__CUDACC__)
TFNO_D float2 shfl_xor2(float2 a, int mask) {
    return make_float2(__shfl_xor_sync(0xffffffffu, a.x, mask), __shfl_xor_sync(0xffffffffu, a.y, mask));
}

// One reduce-scatter round over 2*LEN live entries: lanes with `up` keep entries LEN..2*LEN-1,
// the others keep 0..LEN-1; the other half goes to the partner lane (lane ^ mask).
// Written as three passes over the registers -- arrange, shuffle IN PLACE, add -- so that all
// shuffles of a round are independent and in flight together; fused into one loop the compiler,
// short of registers, serialises shuffle and add and every element pays the full shuffle latency.
template <int LEN>
TFNO_D void exchange_round(float2 (&v)[64], int mask, bool up) {
#pragma unroll
    for (int j = 0; j < LEN; ++j) {
        const float2 lo = v[slot(j)], hi = v[slot(LEN + j)];
        v[slot(j)] = up ? hi : lo;            // keep
        v[slot(LEN + j)] = up ? lo : hi;      // send
    }
#pragma unroll
    for (int j = 0; j < LEN; ++j) v[slot(LEN + j)] = shfl_xor2(v[slot(LEN + j)], mask);
#pragma unroll
    for (int j = 0; j < LEN; ++j) v[slot(j)] = cadd(v[slot(j)], v[slot(LEN + j)]);
}

// First round (partner differs in the top lane bit): the rotation by 32 done inside fft64 has
// already put the kept half into slots 0..31 and the half to send into slots 32..63.
TFNO_D void exchange_round_top(float2 (&v)[64], int mask) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[slot(32 + j)] = shfl_xor2(v[slot(32 + j)], mask);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[slot(j)] = cadd(v[slot(j)], v[slot(32 + j)]);
}

// Forward transform of one signal by R adjacent lanes, truncated to 64 modes.
//   v[n]   : sample R*n + r of the signal (r = lane index within the group)
//   twF    : the forward table (fill_forward_table<R>)
// On return lane r holds modes 64/R*r + j, j < 64/R, in v[slot(j)].
template <int R>
TFNO_D void forward_trunc(float2 (&v)[64], const float2* __restrict__ twF, int r, bool centered = false) {
    forward_local<R>(v, twF, r, centered);
    // round 1 (partner R/2): slots j<32 keep, slots 32+j go to the partner
    exchange_round_top(v, R >> 1);
    // further rounds: conditional swap so that the kept half sits in the low slots
    if constexpr (R >= 4) exchange_round<16>(v, R >> 2, (r & (R >> 2)) != 0);
    if constexpr (R >= 8) exchange_round<8>(v, R >> 3, (r & (R >> 3)) != 0);
    if constexpr (R >= 16) exchange_round<4>(v, R >> 4, (r & (R >> 4)) != 0);
}
#endif

// Inverse transform by one lane of a group of R: in v[m] = mode m (m<64); out: sample
// R*j2 + j1 in v[slot(j2)].  twI = the inverse table (fill_inverse_table<R>).
// CONJ = +1 for a true inverse, -1 for a second forward transform.
// ROT32: the result is multiplied by (-1)^j2, done as a rotation of the transform's input by 32
// (a renaming of registers), for the centered mode set of fill_inverse_table.
template <int CONJ, int R, bool ROT32 = false>
TFNO_HD void inverse_pad_lane(float2 (&v)[64], const float2* __restrict__ twI, int j1) {
#pragma unroll
    for (int m = 0; m < 64; m += 2) {
        float4 t = *reinterpret_cast<const float4*>(twI + tw_index<R>(j1, m));
        v[m] = cmul(v[m], make_float2(t.x, t.y));
        v[m + 1] = cmul(v[m + 1], make_float2(t.z, t.w));
    }
    if constexpr (ROT32) {
#pragma unroll
        for (int m = 0; m < 32; ++m) {
            const float2 t = v[m];
            v[m] = v[m + 32];
            v[m + 32] = t;
        }
    }
    fft64<CONJ>(v);
}

}  // namespace tfno

// Register-resident 32-point complex FFT and the multi-lane truncated / zero-padded transforms
// built on it: the same operators as fft64.cuh (forward transform of a signal of length DY that
// keeps modes 0..63, inverse transform from 64 modes to DY samples; roles of the reference's
// fft_N_fused / fft_N_fused_output device code, call sites
// fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/fused_fft_cgemm_ifft_7.cuh:46,114,218), with HALF the
// per-lane state: a lane holds 32 samples (64 registers) instead of 64, a signal is spread over
// R = DY/32 lanes instead of DY/64.  A thread then fits in ~100 registers, so twice as many warps
// are resident per scheduler to hide shared-memory, shuffle and barrier latency -- which is what
// bounds the kernels built on the 64-point transform.
//
//   forward, keep modes k < 64.  Lane r owns x[R*n + r], n < 32, and F_r = FFT32 of them:
//       X[k]      = sum_r W_DY^{r k}            F_r[k]          k < 32
//       X[k + 32] = sum_r W_DY^{r k} W_R^{r}    F_r[k]          (W_R = e^{-2 pi i / R})
//     Round 1 pairs lane a < R/2 with b = a + R/2 (W_R^{b} = -W_R^{a}): a keeps the k < 32 half,
//     b the k + 32 half, each as  own * table + coef * received  -- one complex multiply-add per
//     value, the pair's common factor W_R^{a} folded into b's table and undone by a's coef.
//     The remaining log2(R) - 1 rounds are a reduce-scatter of partial sums (adds only).
//     Lane r ends with modes 64/R*r + j, j < 64/R.
//
//   inverse from 64 modes.  Lane j1 owns samples R*j2 + j1, j2 < 32:
//       y[R*j2 + j1] = IFFT32_{m'->j2}( C[m'] T[j1][m'] + C[m'+32] T[j1][m'+32] ),  T[j1][m] = g W_DY^{-j1 m}
//     every lane reads the same 64 modes; no exchange.
//
// The 32-point kernel is 4 x 8: eight radix-4 butterflies, 21 non-trivial constant twiddles,
// four radix-8 butterflies.  Outputs stay in place: mode k = k1 + 4*k2 is in register slot
// 8*k1 + k2 (slot32()).
#pragma once
#include "fft64.cuh"

namespace tfno {

TFNO_HD constexpr int slot32(int k) { return 8 * (k & 3) + (k >> 2); }

template <int S, int N2, int K1>
TFNO_HD float2 twiddle32(float2 a) {   // a * e^{S*2 pi i*N2*K1/32}
    constexpr int e = (N2 * K1) & 31;
    if constexpr (e == 0) return a;
    else if constexpr (e == 8) return mul_si<S>(a);
    else if constexpr (e == 16) return make_float2(-a.x, -a.y);
    else if constexpr (e == 24) return mul_si<-S>(a);
    else {
        constexpr float c = (float)cx_cos2pi(e, 32);
        constexpr float sn = (float)(S * cx_sin2pi(e, 32));
        return make_float2(a.x * c - a.y * sn, a.x * sn + a.y * c);
    }
}
template <int S, int K1>
TFNO_HD void twiddle_row32(float2* v) {   // v[8*K1 + n2] *= W32^{n2*K1}, n2 = 1..7
    v[8 * K1 + 1] = twiddle32<S, 1, K1>(v[8 * K1 + 1]);
    v[8 * K1 + 2] = twiddle32<S, 2, K1>(v[8 * K1 + 2]);
    v[8 * K1 + 3] = twiddle32<S, 3, K1>(v[8 * K1 + 3]);
    v[8 * K1 + 4] = twiddle32<S, 4, K1>(v[8 * K1 + 4]);
    v[8 * K1 + 5] = twiddle32<S, 5, K1>(v[8 * K1 + 5]);
    v[8 * K1 + 6] = twiddle32<S, 6, K1>(v[8 * K1 + 6]);
    v[8 * K1 + 7] = twiddle32<S, 7, K1>(v[8 * K1 + 7]);
}

// 32-point transform, in registers.  In: v[n] = sample n.  Out: mode k in v[slot32(k)].
// With s = -1 the odd samples are negated, i.e. the output is rotated by 16:
// v[slot32(k)] then holds mode (k + 16) mod 32.
template <int S>
TFNO_HD void fft32(float2 (&v)[32], float s = 1.0f) {
    const OddSign sg = make_odd_sign(s);
    // step 1: for every n2, radix-4 over n1 on v[8*n1 + n2]; result k1 stored at v[8*k1 + n2]
#pragma unroll
    for (int n2 = 0; n2 < 8; ++n2) dft4<S>(v[n2], v[8 + n2], v[16 + n2], v[24 + n2]);
    // step 2: twiddles W32^{n2*k1}
    twiddle_row32<S, 1>(v); twiddle_row32<S, 2>(v); twiddle_row32<S, 3>(v);
    // step 3: for every k1, radix-8 over n2 on v[8*k1 + n2]; result k2 stored at v[8*k1 + k2].
    // Sample parity equals the parity of n2, so the run-time sign enters here.
#pragma unroll
    for (int k1 = 0; k1 < 4; ++k1)
        fft8<S>(v[8 * k1], v[8 * k1 + 1], v[8 * k1 + 2], v[8 * k1 + 3], v[8 * k1 + 4], v[8 * k1 + 5],
                v[8 * k1 + 6], v[8 * k1 + 7], sg);
}

// ------------------------------------------------------------------------------------------
// Tables (shared memory).  Layout as in fft64.cuh: the entries of slot pair (j, j+1) of the R
// lanes are adjacent, so the R lanes of a group fetch one contiguous R*16-byte piece.
// ------------------------------------------------------------------------------------------
// Lanes whose bit R/4 is set run the 32-point transform with negated odd samples (output rotated
// by 16), so that the half a lane keeps in round 2 always sits in slots 0..15.
template <int R> TFNO_HD bool lane_rotated32(int r) { return (r & (R >> 2)) != 0; }

// forward: twF[r][j] = t_r * W_DY^{r k},  k = (j + 16*rotated(r)) mod 32,  t_r = 1 for the lanes
// r < R/2 (which keep modes < 32) and -W_R^{a} for r = a + R/2 (which keep modes 32..63).
// `centered`: the kept modes are -32..31 instead of 0..63 (mode k of the result is k - 32 of the
// signal): the transform of the signal times e^{+2 pi i 32 n / DY}, which for sample n = R*i + r is
// the per-lane constant e^{+2 pi i r / R} = W_DY^{-32 r} -- it goes into the lane's row of the table.
template <int R>
TFNO_HD void fill_forward_table32(float2* twF, int tid, int nthreads, bool centered = false) {
    constexpr int DY = 32 * R;
    for (int i = tid; i < R * 32; i += nthreads) {
        const int r = i >> 5, j = i & 31;
        const int k = (j + (lane_rotated32<R>(r) ? 16 : 0)) & 31;
        int e = (r * k) & (DY - 1);
        const bool hi = r >= (R >> 1);
        if (hi) e = (e + 32 * (r - (R >> 1)) + DY / 2) & (DY - 1);      // times -W_R^{a} = W_DY^{32 a + DY/2}
        if (centered) e = (e - 32 * r) & (DY - 1);
        twF[tw_index<R>(r, j)] = unit_root(e, DY, -1.0f);
    }
}
// coefficient applied to the values received in round 1: lane a < R/2 gets b's values, which carry
// -W_R^{a}, and undoes that factor; lane b gets a's plain values and applies W_R^{a}
template <int R>
TFNO_HD float2 round1_coef32(int r) {
    constexpr int DY = 32 * R;
    const bool hi = r >= (R >> 1);
    const int a = hi ? r - (R >> 1) : r;
    // hi: W_R^{a} = W_DY^{32 a};   lo: -conj(W_R^{a}) = W_DY^{-32 a + DY/2}
    const int e = hi ? (32 * a) & (DY - 1) : (DY / 2 - 32 * a) & (DY - 1);
    return unit_root(e, DY, -1.0f);
}

// inverse: twI[j1][m] = g * W_DY^{-j1 m} (conj) for m < 64
template <int R>
TFNO_HD void fill_inverse_table32(float2* twI, int tid, int nthreads, float2 g, bool conj) {
    constexpr int DY = 32 * R;
    for (int i = tid; i < R * 64; i += nthreads) {
        const int j1 = i >> 6, m = i & 63;
        twI[tw_index<R>(j1, m)] = cmul(g, unit_root((j1 * m) & (DY - 1), DY, conj ? 1.0f : -1.0f));
    }
}

// Folded form of the inverse table: W_DY^{-j1 (m'+32)} = W_DY^{-j1 m'} W_R^{-j1}, so
//     C[m'] T[m'] + C[m'+32] T[m'+32] = T[m'] ( C[m'] + c C[m'+32] ),   c = inverse_fold_coef32(j1)
// and a lane needs 32 table entries (m' < 32) plus one constant.
// `centered` (true inverse only): the 64 given modes are -32..31; sample R*j2 + j1 of the result is
// the ordinary one times e^{-2 pi i 32 (R*j2 + j1) / DY} = e^{-2 pi i j1 / R}, a per-lane constant.
template <int R>
TFNO_HD void fill_inverse_table32_folded(float2* twI, int tid, int nthreads, float2 g, bool conj, bool centered = false) {
    constexpr int DY = 32 * R;
    for (int i = tid; i < R * 32; i += nthreads) {
        const int j1 = i >> 5, m = i & 31;
        const int e = centered ? (j1 * m - 32 * j1) & (DY - 1) : (j1 * m) & (DY - 1);
        twI[tw_index<R>(j1, m)] = cmul(g, unit_root(e, DY, conj ? 1.0f : -1.0f));
    }
}
template <int R>
TFNO_HD float2 inverse_fold_coef32(int j1, bool conj) {
    constexpr int DY = 32 * R;
    return unit_root((32 * j1) & (DY - 1), DY, conj ? 1.0f : -1.0f);
}

// Lane-local part of the forward transform: 32-point transform of the lane's decimated samples
// and the table multiply.
template <int R>
TFNO_HD void forward_local32(float2 (&v)[32], const float2* __restrict__ twF, int r) {
    fft32<-1>(v, lane_rotated32<R>(r) ? -1.0f : 1.0f);
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
        const float4 t = *reinterpret_cast<const float4*>(twF + tw_index<R>(r, j));
        v[slot32(j)] = cmul(v[slot32(j)], make_float2(t.x, t.y));
        v[slot32(j + 1)] = cmul(v[slot32(j + 1)], make_float2(t.z, t.w));
    }
}

// own + coef * received
TFNO_HD float2 cmadd(float2 own, float2 coef, float2 got) {
    return make_float2(fmaf(coef.x, got.x, fmaf(-coef.y, got.y, own.x)), fmaf(coef.x, got.y, fmaf(coef.y, got.x, own.y)));
}

#if defined(__CUDACC__)
// Exchange rounds over lanes that are `stride` apart per unit of r (lane = g + stride * r).
// Round 1: all 32 values cross; shuffles are issued in batches of 8 so that few extra registers
// are live.
TFNO_D void exchange_round1_32(float2 (&v)[32], int mask, float2 coef) {
#pragma unroll
    for (int j0 = 0; j0 < 32; j0 += 8) {
        float2 got[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) got[j] = shfl_xor2(v[j0 + j], mask);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j0 + j] = cmadd(v[j0 + j], coef, got[j]);
    }
}
// Round 2: slots 0..15 stay, slots 16..31 go to the partner (the rotation inside fft32 has put
// the kept half into the low slots on both sides).
TFNO_D void exchange_round2_32(float2 (&v)[32], int mask) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[slot32(16 + j)] = shfl_xor2(v[slot32(16 + j)], mask);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[slot32(j)] = cadd(v[slot32(j)], v[slot32(16 + j)]);
}
// Further rounds over 2*LEN live entries: lanes with `up` keep entries LEN..2*LEN-1.
template <int LEN>
TFNO_D void exchange_round_32(float2 (&v)[32], int mask, bool up) {
#pragma unroll
    for (int j = 0; j < LEN; ++j) {
        const float2 lo = v[slot32(j)], hi = v[slot32(LEN + j)];
        v[slot32(j)] = up ? hi : lo;
        v[slot32(LEN + j)] = up ? lo : hi;
    }
#pragma unroll
    for (int j = 0; j < LEN; ++j) v[slot32(LEN + j)] = shfl_xor2(v[slot32(LEN + j)], mask);
#pragma unroll
    for (int j = 0; j < LEN; ++j) v[slot32(j)] = cadd(v[slot32(j)], v[slot32(LEN + j)]);
}

// Forward transform of one signal by R lanes that are `stride` lanes apart, truncated to 64 modes.
//   v[n]   : sample R*n + r of the signal
// On return lane r holds modes 64/R*r + j, j < 64/R, in v[slot32(j)].
template <int R>
TFNO_D void forward_trunc32(float2 (&v)[32], const float2* __restrict__ twF, int r, int stride, float2 coef) {
    forward_local32<R>(v, twF, r);
    exchange_round1_32(v, (R >> 1) * stride, coef);
    exchange_round2_32(v, (R >> 2) * stride);
    if constexpr (R >= 8) exchange_round_32<8>(v, (R >> 3) * stride, (r & (R >> 3)) != 0);
    if constexpr (R >= 16) exchange_round_32<4>(v, (R >> 4) * stride, (r & (R >> 4)) != 0);
    if constexpr (R >= 32) exchange_round_32<2>(v, (R >> 5) * stride, (r & (R >> 5)) != 0);
}
#endif

// Inverse transform by one lane of a group of R: `mode(m)` returns mode m < 64 of the signal;
// out: sample R*j2 + j1 in v[slot32(j2)].  CONJ = +1 for a true inverse, -1 for a second forward
// transform (the table must have been filled with the matching `conj`).
template <int CONJ, int R, typename ModeFn>
TFNO_HD void inverse_pad_lane32(float2 (&v)[32], const float2* __restrict__ twI, int j1, ModeFn mode) {
#pragma unroll
    for (int m = 0; m < 32; m += 2) {
        const float4 t0 = *reinterpret_cast<const float4*>(twI + tw_index<R>(j1, m));
        const float4 t1 = *reinterpret_cast<const float4*>(twI + tw_index<R>(j1, m + 32));
        v[m] = cmadd(cmul(mode(m), make_float2(t0.x, t0.y)), make_float2(t1.x, t1.y), mode(m + 32));
        v[m + 1] = cmadd(cmul(mode(m + 1), make_float2(t0.z, t0.w)), make_float2(t1.z, t1.w), mode(m + 33));
    }
    fft32<CONJ>(v);
}

}  // namespace tfno

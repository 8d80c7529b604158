"""CPU oracle (numpy, complex128) for the FNO spectral-convolution path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package may import this file; it is the
checker used by tests/, by __graft_entry__.smoke() and by bench.py's cpu_baseline leg.

PARITY UNPINNED BY THE REFERENCE: TurboFNO ships no tests, golden vectors or fixtures, and its
drivers never copy a result back to the host (fusion_variants/1D_E_baseline/fused.cu:200-216 only
times).  This oracle is therefore pinned against (a) analytic known-answer cases, (b) an independent
double-precision C restatement (oracle/spectral_oracle.c) with its own FFT, and (c) on a GPU box,
against the reference's own truncation / zero-padding / cgemm kernels compiled from the reference
sources (oracle/ref_harness.cu -> oracle/_ref/).

Pipeline restated here (reference: fusion_variants/1D_E_baseline/fused.cu:180-190 and
fusion_variants/2D_E_baseline/fused_trunc_2D.cu:200-227), with FNO semantics
(alpha=1, beta=0, true inverse transform, 1/DY or 1/(DX*DY) scale):

  1D:  X = FFT_DY(x)                 forward, e^{-2 pi i jk/DY}, unnormalised (cuFFT C2C convention)
       A[m] = X[m], m < modes        direct_copy_colmajor_float4_truncation, fused.cu:13-37
       C[b,n,m] = sum_k A[b,k,m] W[k,n]     cublasCgemm NN, lda=M, ldb=K, fused.cu:186
       P[m] = C[m] (m<modes) else 0  direct_copy_colmajor_float4_zero_padding, fused.cu:39-63
       y = alpha * iFFT_DY(P) / DY
  2D:  same with a 2-D transform over (DX, DY) and the corner block [0,modes) x [0,modes)
       (fused_trunc_2D.cu:13-41 truncation, :44-71 zero padding).

Logical tensor shapes used by every oracle entry point (layout-independent):
  1D:  x[B, K, DY]        w[K, N]   ->  y[B, N, DY]        with B = bs*dimX
  2D:  x[B, K, DX, DY]    w[K, N]   ->  y[B, N, DX, DY]

Per-mode weights (an extension, not reference behaviour: the reference's GEMM shares one K x N
matrix between all modes, cgemm.cuh:42-43): w[K, N, modes] (1D) or w[K, N, modes, modes] (2D),
C[b,n,m] = sum_k A[b,k,m] W[k,n,m].
"""
import numpy as np

MODES = 64


def spectral_conv_1d(x, w, modes=MODES, alpha=1.0, inverse=True, scale=True):
    x = np.asarray(x, dtype=np.complex128)
    w = np.asarray(w, dtype=np.complex128)
    B, K, DY = x.shape
    N = w.shape[1]
    X = np.fft.fft(x, axis=-1)[..., :modes]                  # [B,K,modes]
    C = (np.einsum("bkm,knm->bnm", X, w) if w.ndim == 3 else np.einsum("bkm,kn->bnm", X, w)) * alpha   # [B,N,modes]
    P = np.zeros((B, N, DY), dtype=np.complex128)
    P[..., :modes] = C
    if inverse:
        y = np.fft.ifft(P, axis=-1)
        if not scale:
            y = y * DY
    else:  # "as shipped": second transform is forward again, fused.cu:190
        y = np.fft.fft(P, axis=-1)
    return y


def spectrum_1d(x, modes=MODES):
    """Forward transform + truncation only: [B,K,DY] -> [B,K,modes]."""
    return np.fft.fft(np.asarray(x, dtype=np.complex128), axis=-1)[..., :modes]


def cgemm_modes(a, w, alpha=1.0, beta=0.0, c=None):
    """a[B,K,m], w[K,N] -> alpha*sum_k a w + beta*c  (cgemm.cuh:178-200)."""
    out = np.einsum("bkm,kn->bnm", np.asarray(a, np.complex128), np.asarray(w, np.complex128)) * alpha
    if c is not None:
        out = out + beta * np.asarray(c, np.complex128)
    return out


def ifft_pad_1d(c, DY, scale=True):
    """[B,N,modes] -> zero-pad to DY -> inverse transform."""
    c = np.asarray(c, np.complex128)
    P = np.zeros(c.shape[:-1] + (DY,), dtype=np.complex128)
    P[..., : c.shape[-1]] = c
    y = np.fft.ifft(P, axis=-1)
    return y if scale else y * DY


def spectral_conv_2d(x, w, modes=MODES, alpha=1.0, inverse=True, scale=True, x_modes_centered=False):
    """x_modes_centered: keep X modes -modes/2 .. modes/2-1 (both low-frequency blocks of a
    non-last axis, as an FNO layer does) instead of the reference's corner 0 .. modes-1
    (fusion_variants/2D_E_baseline/fused_trunc_2D.cu:30-39); an extension, not reference behaviour."""
    x = np.asarray(x, dtype=np.complex128)
    w = np.asarray(w, dtype=np.complex128)
    B, K, DX, DY = x.shape
    N = w.shape[1]
    kx = (np.arange(-modes // 2, modes // 2) % DX) if x_modes_centered else np.arange(modes)
    X = np.fft.fft2(x, axes=(-2, -1))[..., kx, :][..., :modes]   # [B,K,modes,modes]
    C = (np.einsum("bkxy,knxy->bnxy", X, w) if w.ndim == 4 else np.einsum("bkxy,kn->bnxy", X, w)) * alpha
    P = np.zeros((B, N, DX, DY), dtype=np.complex128)
    P[..., kx, :modes] = C
    if inverse:
        y = np.fft.ifft2(P, axes=(-2, -1))
        if not scale:
            y = y * (DX * DY)
    else:
        y = np.fft.fft2(P, axes=(-2, -1))
    return y


def spectrum_2d(x, modes=MODES):
    return np.fft.fft2(np.asarray(x, np.complex128), axes=(-2, -1))[..., :modes, :modes]


def ifft_pad_2d(c, DX, DY, scale=True):
    c = np.asarray(c, np.complex128)
    P = np.zeros(c.shape[:-2] + (DX, DY), dtype=np.complex128)
    P[..., : c.shape[-2], : c.shape[-1]] = c
    y = np.fft.ifft2(P, axes=(-2, -1))
    return y if scale else y * (DX * DY)


def fft_cols_trunc(x, modes=MODES):
    """X-axis (strided) forward transform with row truncation: [I,DX,DY] -> [I,modes,DY]
    (interface of fft_N_stride, fusion_variants/2D_D_exp_fused_fft_cgemm_ifft/fused_trunc_2D.cu:153-160)."""
    return np.fft.fft(np.asarray(x, np.complex128), axis=-2)[..., :modes, :]


def ifft_cols_pad(c, DX, scale=True):
    """[I,modes,DY] -> zero-pad rows to DX -> inverse along X -> [I,DX,DY]."""
    c = np.asarray(c, np.complex128)
    P = np.zeros(c.shape[:-2] + (DX, c.shape[-1]), dtype=np.complex128)
    P[..., : c.shape[-2], :] = c
    y = np.fft.ifft(P, axis=-2)
    return y if scale else y * DX


# ---------------------------------------------------------------------------------------------
# Seeded synthetic inputs (function of the LOGICAL index, so every memory layout holds the same
# tensor): x re/im ~ U[-1,1], W re/im ~ N(0, 1/K).
# ---------------------------------------------------------------------------------------------
def make_inputs_1d(B, K, N, DY, seed=1234, wseed=4321):
    rx = np.random.default_rng(seed)
    x = rx.uniform(-1, 1, (B, K, DY)) + 1j * rx.uniform(-1, 1, (B, K, DY))
    rw = np.random.default_rng(wseed)
    s = 1.0 / np.sqrt(K)
    w = rw.normal(0, s, (K, N)) + 1j * rw.normal(0, s, (K, N))
    return x.astype(np.complex64), w.astype(np.complex64)


def make_inputs_2d(B, K, N, DX, DY, seed=1234, wseed=4321):
    rx = np.random.default_rng(seed)
    x = rx.uniform(-1, 1, (B, K, DX, DY)) + 1j * rx.uniform(-1, 1, (B, K, DX, DY))
    rw = np.random.default_rng(wseed)
    s = 1.0 / np.sqrt(K)
    w = rw.normal(0, s, (K, N)) + 1j * rw.normal(0, s, (K, N))
    return x.astype(np.complex64), w.astype(np.complex64)


def errors(test, ref):
    """(max_rel, rel_l2): max|a-b|/max|ref| and ||a-b||_2/||ref||_2 (per-element relative error
    is ill-conditioned near zero crossings of the output)."""
    test = np.asarray(test, np.complex128)
    ref = np.asarray(ref, np.complex128)
    d = np.abs(test - ref)
    den = max(np.abs(ref).max(), 1e-30)
    l2 = np.sqrt((d ** 2).sum()) / max(np.sqrt((np.abs(ref) ** 2).sum()), 1e-30)
    return float(d.max() / den), float(l2)


def make_per_mode_weights(K, N, mode_shape, wseed=4321):
    """w[K, N, *mode_shape], re/im ~ N(0, 1/K), seeded."""
    rw = np.random.default_rng(wseed)
    s = 1.0 / np.sqrt(K)
    shape = (K, N) + tuple(mode_shape)
    return (rw.normal(0, s, shape) + 1j * rw.normal(0, s, shape)).astype(np.complex64)

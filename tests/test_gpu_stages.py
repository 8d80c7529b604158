"""GPU tests of the stage-level entry points (the reference's kernel tables) against the oracle."""
import numpy as np
import pytest

from util import assert_close, oracle_np

pytestmark = pytest.mark.gpu


def _dev(cuda, a):
    import torch

    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


@pytest.mark.parametrize("DY", [128, 256, 512, 1024])
def test_fft_and_ifft_stride_DY(cuda, DY):
    import torch
    import turbofno_b200 as t

    S = 150                                   # not a multiple of the signals-per-CTA
    x, _ = oracle_np.make_inputs_1d(S, 1, 64, DY, seed=DY)
    x = x[:, 0, :]
    out = torch.empty((S, 64), dtype=torch.complex64, device=cuda)
    t.fft_stride_DY(_dev(cuda, x), out, S, DY)
    spec = np.fft.fft(x.astype(np.complex128), axis=-1)[:, :64]
    assert_close(out.cpu().numpy(), spec, "fft_stride_DY %d" % DY)
    back = torch.empty((S, DY), dtype=torch.complex64, device=cuda)
    t.ifft_stride_DY(_dev(cuda, spec.astype(np.complex64)), back, S, DY)
    assert_close(back.cpu().numpy(), oracle_np.ifft_pad_1d(spec.astype(np.complex64), DY, scale=False), "ifft_stride_DY %d" % DY)


@pytest.mark.parametrize("DX,DY", [(128, 128), (256, 128), (128, 256), (512, 64 * 3)])
def test_fft_and_ifft_stride_X(cuda, DX, DY):
    import torch
    import turbofno_b200 as t

    I = 3
    rng = np.random.default_rng(DX + DY)
    x = (rng.uniform(-1, 1, (I, DX, DY)) + 1j * rng.uniform(-1, 1, (I, DX, DY))).astype(np.complex64)
    out = torch.empty((I, 64, DY), dtype=torch.complex64, device=cuda)
    t.fft_stride(_dev(cuda, x), out, DY, I * DY, DX)
    ref = oracle_np.fft_cols_trunc(x)
    assert_close(out.cpu().numpy(), ref, "fft_stride")
    back = torch.empty((I, DX, DY), dtype=torch.complex64, device=cuda)
    t.ifft_stride(_dev(cuda, ref.astype(np.complex64)), back, DY, I * DY, DX)
    assert_close(back.cpu().numpy(), oracle_np.ifft_cols_pad(ref.astype(np.complex64), DX, scale=False), "ifft_stride")


@pytest.mark.parametrize("rows,K,N", [(1, 8, 64), (5, 24, 128), (300, 64, 64), (3, 128, 192)])
def test_cgemm(cuda, rows, K, N):
    import torch
    import turbofno_b200 as t

    M = rows * 64
    rng = np.random.default_rng(rows + K)
    A = (rng.standard_normal((K, M)) + 1j * rng.standard_normal((K, M))).astype(np.complex64)      # A[m + k*M]
    Bm = (rng.standard_normal((N, K)) + 1j * rng.standard_normal((N, K))).astype(np.complex64)     # B[k + n*K]
    C0 = (rng.standard_normal((N, M)) + 1j * rng.standard_normal((N, M))).astype(np.complex64)
    alpha, beta = 1 - 1j, -1 + 1j             # the reference drivers' constants
    C = _dev(cuda, C0)
    t.cgemm(M, N, K, _dev(cuda, A), _dev(cuda, Bm), C, alpha, beta)
    ref = alpha * (Bm.astype(np.complex128) @ A.astype(np.complex128)) + beta * C0
    assert_close(C.cpu().numpy(), ref, "cgemm")


@pytest.mark.parametrize("rows,K", [(1, 16), (7, 32), (149, 48), (600, 64), (296, 16), (1000, 48),
                                     # a padded last chunk (8 of 16 channels), and two launches over the halves of K > 64
                                     (5, 8), (301, 24), (600, 56), (600, 72), (297, 96), (600, 104), (298, 128), (1001, 120)])
def test_cgemm_beta_zero_takes_the_tensor_core_kernel(cuda, rows, K):
    """beta = 0, K a multiple of 8 up to 128: the contraction runs on tcgen05 (cgemm_tc_kernel; K > 64
    needs two rows of tiles per SM), every other case on the FP32 kernel; both must agree with the
    float64 product. Even row counts of at
    least two per SM use 128-mode tiles, the others 64-mode tiles. 149 and 600 tiles give
    the CTAs of a 148-SM device one, two and five tiles (double-buffered accumulators, both ring
    stages of a half-team); C starts as NaN to show that every element is written."""
    import torch
    import turbofno_b200 as t

    N, M = 64, rows * 64
    rng = np.random.default_rng(100 * rows + K)
    A = (rng.uniform(-1, 1, (K, M)) + 1j * rng.uniform(-1, 1, (K, M))).astype(np.complex64)
    Bm = ((rng.standard_normal((N, K)) + 1j * rng.standard_normal((N, K))) / np.sqrt(K)).astype(np.complex64)
    alpha = 0.75 - 0.5j
    C = torch.full((N, M), float("nan"), dtype=torch.complex64, device=cuda)
    t.cgemm(M, N, K, _dev(cuda, A), _dev(cuda, Bm), C, alpha, 0.0)
    ref = alpha * (Bm.astype(np.complex128) @ A.astype(np.complex128))
    got = C.cpu().numpy()
    assert np.isfinite(got.view(np.float32)).all()
    assert_close(got, ref, "cgemm (tensor cores)")
    assert t.Handle.get(0).device_status == 0
    # same inputs with a non-zero beta (FP32 kernel) differ from it by rounding only
    C2 = torch.zeros((N, M), dtype=torch.complex64, device=cuda)
    t.cgemm(M, N, K, _dev(cuda, A), _dev(cuda, Bm), C2, alpha, 1.0)
    assert_close(C2.cpu().numpy(), ref, "cgemm (FP32 kernel)")


def test_cgemm_wide_layer_runs_the_tensor_core_kernel_per_block_of_64_outputs(cuda):
    import torch
    import turbofno_b200 as t

    rows, K, N = 600, 32, 192
    M = rows * 64
    rng = np.random.default_rng(77)
    A = (rng.uniform(-1, 1, (K, M)) + 1j * rng.uniform(-1, 1, (K, M))).astype(np.complex64)
    Bm = ((rng.standard_normal((N, K)) + 1j * rng.standard_normal((N, K))) / np.sqrt(K)).astype(np.complex64)
    C = torch.full((N, M), float("nan"), dtype=torch.complex64, device=cuda)
    t.cgemm(M, N, K, _dev(cuda, A), _dev(cuda, Bm), C, 1.0, 0.0)
    assert_close(C.cpu().numpy(), Bm.astype(np.complex128) @ A.astype(np.complex128), "cgemm N=192 (tensor cores)")
    # the 2D layer with 128 output channels: the plan reports two launches of the contraction
    plan = t.SpectralConv(2, 8, 128, 32, 128, DX=128, variant="D")
    assert plan.kernels().count("cgemm_tc_kernel<128>") == 2
    plan.close()


@pytest.mark.parametrize("DY", [128, 256])
def test_partial_fusions(cuda, DY):
    import torch
    import turbofno_b200 as t

    B, K, N = 9, 16, 128
    M = B * 64
    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=DY + 1)
    xd = _dev(cuda, np.swapaxes(x, 0, 1))     # [K][B][DY]
    wd = _dev(cuda, w.T)                      # [N][K]
    spec = oracle_np.spectrum_1d(x)           # [B,K,64]
    cref = oracle_np.cgemm_modes(spec, w)     # [B,N,64]
    # fused FFT + CGEMM -> compact C[n][M]
    C = torch.zeros((N, M), dtype=torch.complex64, device=cuda)
    t.fused_fft_cgemm(M, N, K, xd, wd, C, DY=DY)
    assert_close(C.cpu().numpy().reshape(N, B, 64), np.swapaxes(cref, 0, 1), "fused_fft_cgemm")
    # fused CGEMM + iFFT from compact A[k][M]
    A = _dev(cuda, np.swapaxes(spec, 0, 1).astype(np.complex64).reshape(K, M))
    out = torch.empty((N, B, DY), dtype=torch.complex64, device=cuda)
    t.fused_cgemm_ifft(M, N, K, A, wd, None, out, DY=DY)
    yref = oracle_np.spectral_conv_1d(x, w, scale=False)
    assert_close(np.swapaxes(out.cpu().numpy(), 0, 1), yref, "fused_cgemm_ifft")
    # fully fused, kernel-table signature
    out2 = torch.empty((N, B, DY), dtype=torch.complex64, device=cuda)
    t.fused_fft_cgemm_ifft(M, N, K, xd, wd, None, out2, DY=DY)
    assert_close(np.swapaxes(out2.cpu().numpy(), 0, 1), yref, "fused_fft_cgemm_ifft")


def test_a_kernel_side_wait_that_runs_out_reports_a_status_and_leaves_the_device_usable(cuda):
    """Every wait inside the kernels is bounded; this makes one run out on purpose (a barrier that
    nothing completes) without any fault: the kernel returns, the status word carries the code, and
    the next layer on the same context is right."""
    import time

    import torch
    import turbofno_b200 as t

    h = t.Handle.get(0)
    assert h.device_status == 0
    t0 = time.perf_counter()
    h.selftest_bounded_wait()
    assert h.device_status == 99                      # reading the status synchronises
    assert 0.5 < time.perf_counter() - t0 < 30.0      # the one-second limit, not the spin-count backstop
    h.reset_device_status()
    assert h.device_status == 0
    x, w = oracle_np.make_inputs_1d(3, 16, 64, 256, seed=2)
    plan = t.SpectralConv(1, 3, 256, 16, 64, variant="D")
    y = plan(_dev(cuda, np.swapaxes(x, 0, 1)), _dev(cuda, w.T))
    assert_close(np.swapaxes(y.cpu().numpy(), 0, 1), oracle_np.spectral_conv_1d(x, w), "layer after a timed-out wait")
    assert h.device_status == 0

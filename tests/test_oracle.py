"""CPU tests of the oracles themselves: numpy restatement vs C restatement vs analytic
known-answer cases vs the committed golden fixtures."""
import glob
import os

import numpy as np
import pytest

from util import oracle_c, oracle_np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("B,K,N,DY", [(1, 8, 64, 128), (3, 16, 128, 256), (2, 8, 64, 512), (1, 8, 64, 1024)])
def test_c_oracle_matches_numpy_1d(B, K, N, DY):
    x, w = oracle_np.make_inputs_1d(B, K, N, DY)
    ref = oracle_np.spectral_conv_1d(x, w)
    mr, l2 = oracle_np.errors(oracle_c.spectral_conv_1d(x, w, double=True), ref)
    assert mr < 1e-12 and l2 < 1e-12
    mr, l2 = oracle_np.errors(oracle_c.spectral_conv_1d(x, w, double=False), ref)
    assert mr < 2e-6 and l2 < 2e-6


@pytest.mark.parametrize("B,K,N,DX,DY", [(1, 8, 64, 128, 128), (2, 8, 64, 128, 256), (1, 16, 128, 256, 128)])
def test_c_oracle_matches_numpy_2d(B, K, N, DX, DY):
    x, w = oracle_np.make_inputs_2d(B, K, N, DX, DY)
    ref = oracle_np.spectral_conv_2d(x, w)
    mr, l2 = oracle_np.errors(oracle_c.spectral_conv_2d(x, w, double=True), ref)
    assert mr < 1e-12 and l2 < 1e-12
    mr, l2 = oracle_np.errors(oracle_c.spectral_conv_2d(x, w, double=False), ref)
    assert mr < 2e-6 and l2 < 2e-6


def test_as_shipped_semantics_differ_only_by_second_transform():
    # second transform forward and unscaled (reference drivers) == DY * conj-inverse relation:
    # FFT(P)[j] = DY * iFFT(P)[(-j) mod DY]
    x, w = oracle_np.make_inputs_1d(2, 8, 64, 128)
    inv = oracle_np.spectral_conv_1d(x, w)
    fwd = oracle_np.spectral_conv_1d(x, w, inverse=False)
    idx = (-np.arange(128)) % 128
    assert np.allclose(fwd, 128 * inv[..., idx], rtol=1e-12, atol=1e-12)
    fwd_c = oracle_c.spectral_conv_1d(x, w, inverse=False, scale=False)
    assert oracle_np.errors(fwd_c, fwd)[0] < 1e-12


# ---- analytic known-answer cases ------------------------------------------------------------
def test_delta_input_gives_flat_spectrum_and_dirichlet_kernel():
    DY, K, N = 256, 8, 64
    x = np.zeros((1, K, DY), np.complex64)
    x[0, 0, 0] = 1.0                       # delta in channel 0
    w = np.zeros((K, N), np.complex64)
    w[0, :] = 1.0
    y = oracle_c.spectral_conv_1d(x, w)
    j = np.arange(DY)
    expect = np.exp(2j * np.pi * np.outer(np.arange(64), j) / DY).sum(0) / DY    # sum of the 64 kept modes
    assert np.allclose(y[0, 5], expect, atol=1e-12)


@pytest.mark.parametrize("mode,passes", [(3, True), (63, True), (64, False), (200, False)])
def test_single_exponential_passes_only_below_64(mode, passes):
    DY, K, N = 256, 8, 64
    j = np.arange(DY)
    x = np.zeros((1, K, DY), np.complex64)
    x[0, 2] = np.exp(2j * np.pi * mode * j / DY)
    w = np.zeros((K, N), np.complex64)
    w[2, 7] = 2.0
    y = oracle_c.spectral_conv_1d(x, w)
    if passes:
        assert np.allclose(y[0, 7], 2.0 * x[0, 2], atol=1e-5)
    else:
        assert np.abs(y).max() < 1e-5
    assert np.abs(np.delete(y[0], 7, axis=0)).max() < 1e-5


def test_identity_weights_low_pass():
    x, _ = oracle_np.make_inputs_1d(2, 64, 64, 128)
    w = np.eye(64, dtype=np.complex64)
    y = oracle_c.spectral_conv_1d(x, w)
    X = np.fft.fft(x.astype(np.complex128), axis=-1)
    X[..., 64:] = 0
    assert np.allclose(y, np.fft.ifft(X, axis=-1), atol=1e-12)


def test_linearity_and_alpha():
    x1, w = oracle_np.make_inputs_1d(2, 8, 64, 128, seed=1)
    x2, _ = oracle_np.make_inputs_1d(2, 8, 64, 128, seed=2)
    a = 0.5 - 2j
    lhs = oracle_c.spectral_conv_1d((x1 + x2).astype(np.complex64), w, alpha=a)
    rhs = a * (oracle_c.spectral_conv_1d(x1, w) + oracle_c.spectral_conv_1d(x2, w))
    assert oracle_np.errors(lhs, rhs)[0] < 1e-6     # inputs are rounded to complex64 before the sum


def test_2d_corner_truncation_has_no_negative_frequency_block():
    DX = DY = 128
    ix, iy = np.meshgrid(np.arange(DX), np.arange(DY), indexing="ij")
    x = np.zeros((1, 8, DX, DY), np.complex64)
    x[0, 0] = np.exp(2j * np.pi * (5 * ix + 9 * iy) / 128)          # mode (5, 9): kept
    x[0, 1] = np.exp(2j * np.pi * (-5 * ix + 9 * iy) / 128)         # mode (123, 9): dropped
    w = np.zeros((8, 64), np.complex64)
    w[0, 0] = 1
    w[1, 1] = 1
    y = oracle_c.spectral_conv_2d(x, w)
    assert np.allclose(y[0, 0], x[0, 0], atol=1e-5)
    assert np.abs(y[0, 1]).max() < 1e-5


# ---- golden fixtures ---------------------------------------------------------------------------
def test_golden_fixtures_present():
    assert len(glob.glob(os.path.join(GOLDEN, "*.npz"))) == 3


def test_c_oracle_against_golden():
    g = np.load(os.path.join(GOLDEN, "c0_1d_bs1_dy128_k8_n64.npz"))
    assert oracle_np.errors(oracle_c.spectral_conv_1d(g["x"], g["w"]), g["y"])[0] < 1e-12
    g = np.load(os.path.join(GOLDEN, "c1_1d_bs4_dy256_k24_n128.npz"))
    assert oracle_np.errors(oracle_c.spectral_conv_1d(g["x"], g["w"])[:, ::8, :], g["y"])[0] < 1e-12
    g = np.load(os.path.join(GOLDEN, "c2_2d_bs1_k8_n64_128x256.npz"))
    assert oracle_np.errors(oracle_c.spectral_conv_2d(g["x"], g["w"])[:, ::8, ::8, ::8], g["y"])[0] < 1e-12


def test_centered_x_modes_keep_negative_frequencies():
    """A plane wave with X frequency -5 passes a layer with identity weights when the centered X
    mode set (-32..31) is kept, and is removed by the reference's corner set (0..63)."""
    DX = DY = 128
    xx, yy = np.meshgrid(np.arange(DX), np.arange(DY), indexing="ij")
    wave = np.exp(2j * np.pi * (-5 * xx / DX + 3 * yy / DY))
    x = np.zeros((1, 8, DX, DY), np.complex128)
    x[0, 2] = wave
    w = np.zeros((8, 64), np.complex128)
    w[2, 7] = 1.0
    y_c = oracle_np.spectral_conv_2d(x, w, x_modes_centered=True)
    y_0 = oracle_np.spectral_conv_2d(x, w)
    assert np.abs(y_c[0, 7] - wave).max() < 1e-9
    assert np.abs(y_0).max() < 1e-9
    # a positive frequency inside both sets passes both
    x[0, 2] = np.exp(2j * np.pi * (9 * xx / DX + 3 * yy / DY))
    assert np.abs(oracle_np.spectral_conv_2d(x, w, x_modes_centered=True) - oracle_np.spectral_conv_2d(x, w)).max() < 1e-9


def test_per_mode_weights_extension_of_the_oracle():
    """Per-mode weights W[k,n,m]: with weights that do not depend on the mode the result is the
    shared-weight layer; a weight tensor that is non-zero for one mode only passes that mode."""
    x, w = oracle_np.make_inputs_1d(3, 8, 64, 128, seed=5)
    wm = np.repeat(w[:, :, None], 64, axis=2)
    assert np.abs(oracle_np.spectral_conv_1d(x, wm) - oracle_np.spectral_conv_1d(x, w)).max() < 1e-12
    one = np.zeros((8, 64, 64), np.complex64)
    one[2, 5, 9] = 3.0                      # channel 2 -> output 5, mode 9 only
    y = oracle_np.spectral_conv_1d(x, one)
    X = np.fft.fft(x.astype(np.complex128), axis=-1)
    expect = 3.0 * X[:, 2, 9, None] * np.exp(2j * np.pi * 9 * np.arange(128) / 128) / 128
    assert np.abs(y[:, 5] - expect).max() < 1e-12 and np.abs(np.delete(y, 5, axis=1)).max() < 1e-12
    x2, w2 = oracle_np.make_inputs_2d(2, 8, 64, 128, 128, seed=6)
    wm2 = np.broadcast_to(w2[:, :, None, None], (8, 64, 64, 64))
    assert np.abs(oracle_np.spectral_conv_2d(x2, wm2) - oracle_np.spectral_conv_2d(x2, w2)).max() < 1e-12

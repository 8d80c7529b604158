"""torch.ops.turbofno_b200.spectral_conv{1,2}d: registration and shape function on CPU, results on GPU."""
import numpy as np
import pytest

from util import assert_close, oracle_np


def test_operators_are_registered_with_a_shape_function():
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import turbofno_b200.torch_op  # noqa: F401  (registers the operators; loads no CUDA code)

    assert hasattr(torch.ops.turbofno_b200, "spectral_conv1d") and hasattr(torch.ops.turbofno_b200, "spectral_conv2d")
    with FakeTensorMode():
        x = torch.empty((3, 16, 256), dtype=torch.complex64)
        w = torch.empty((16, 64), dtype=torch.complex64)
        y = torch.ops.turbofno_b200.spectral_conv1d(x, w)
        assert tuple(y.shape) == (3, 64, 256) and y.dtype == torch.complex64
        x2 = torch.empty((2, 8, 128, 256), dtype=torch.complex64)
        w2 = torch.empty((8, 64), dtype=torch.complex64)
        assert tuple(torch.ops.turbofno_b200.spectral_conv2d(x2, w2).shape) == (2, 64, 128, 256)
        with pytest.raises(Exception):
            torch.ops.turbofno_b200.spectral_conv1d(x, w2)      # K mismatch
        # per-mode weights and the centered X block go through the same operators
        wm = torch.empty((16, 64, 64), dtype=torch.complex64)
        assert tuple(torch.ops.turbofno_b200.spectral_conv1d(x, wm).shape) == (3, 64, 256)
        wm2 = torch.empty((8, 128, 64, 64), dtype=torch.complex64)
        assert tuple(torch.ops.turbofno_b200.spectral_conv2d(x2, wm2, True).shape) == (2, 128, 128, 256)
        with pytest.raises(Exception):
            torch.ops.turbofno_b200.spectral_conv1d(x, torch.empty((16, 64, 32), dtype=torch.complex64))   # 64 modes only


def test_operator_has_no_cpu_kernel():
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    x = torch.zeros((1, 8, 128), dtype=torch.complex64)
    w = torch.zeros((8, 64), dtype=torch.complex64)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.turbofno_b200.spectral_conv1d(x, w)           # the path has no CPU implementation


@pytest.mark.gpu
@pytest.mark.parametrize("B,K,N,DY", [(5, 16, 64, 256), (3, 8, 128, 128), (150, 64, 64, 256),
                                        # batch-first strides through the padded-chunk and the two-launch paths of the fused kernel
                                        (300, 24, 64, 256), (300, 128, 64, 256), (300, 104, 128, 128)])
def test_spectral_conv1d_operator(cuda, B, K, N, DY):
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    x, w = oracle_np.make_inputs_1d(B, K, N, DY, seed=B + K)
    y = torch.ops.turbofno_b200.spectral_conv1d(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda))
    assert_close(y.cpu().numpy(), oracle_np.spectral_conv_1d(x, w), "torch op 1d")
    torch.library.opcheck(torch.ops.turbofno_b200.spectral_conv1d.default,
                          (torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda)),
                          test_utils=("test_schema", "test_faketensor"))


@pytest.mark.gpu
def test_spectral_conv2d_operator(cuda):
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    B, K, N, DX, DY = 2, 16, 64, 128, 256
    x, w = oracle_np.make_inputs_2d(B, K, N, DX, DY, seed=11)
    y = torch.ops.turbofno_b200.spectral_conv2d(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda))
    assert_close(y.cpu().numpy(), oracle_np.spectral_conv_2d(x, w), "torch op 2d")


@pytest.mark.gpu
def test_spectral_conv1d_gradients_match_autograd_through_torch_fft(cuda):
    """grad_x and grad_W of the operator (own kernels) against autograd through a torch.fft
    restatement of the layer, for a real-valued loss; complex64, so the parity tolerance."""
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    B, K, N, DY = 6, 64, 64, 256
    x0, w0 = oracle_np.make_inputs_1d(B, K, N, DY, seed=5)
    rng = np.random.default_rng(9)
    t0 = (rng.standard_normal((B, N, DY)) + 1j * rng.standard_normal((B, N, DY))).astype(np.complex64)
    target = torch.from_numpy(t0).to(cuda)

    def loss_of(y):
        return (y - target).abs().pow(2).sum()

    x = torch.from_numpy(x0).to(cuda).requires_grad_(True)
    w = torch.from_numpy(w0).to(cuda).requires_grad_(True)
    loss_of(torch.ops.turbofno_b200.spectral_conv1d(x, w)).backward()

    xr = torch.from_numpy(x0).to(cuda).requires_grad_(True)
    wr = torch.from_numpy(w0).to(cuda).requires_grad_(True)
    spec = torch.fft.fft(xr, dim=-1)[..., :64]
    yhat = torch.einsum("bkm,kn->bnm", spec, wr)
    padded = torch.zeros((B, N, DY), dtype=torch.complex64, device=cuda)
    padded = torch.cat([yhat, padded[..., 64:]], dim=-1)
    loss_of(torch.fft.ifft(padded, dim=-1)).backward()

    assert_close(x.grad.cpu().numpy(), xr.grad.cpu().numpy(), "grad_x")
    assert_close(w.grad.cpu().numpy(), wr.grad.cpu().numpy(), "grad_W")


@pytest.mark.gpu
def test_spectral_conv2d_gradients_match_autograd_through_torch_fft(cuda):
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    B, K, N, DX, DY = 2, 64, 64, 128, 256
    x0, w0 = oracle_np.make_inputs_2d(B, K, N, DX, DY, seed=6)
    rng = np.random.default_rng(10)
    target = torch.from_numpy((rng.standard_normal((B, N, DX, DY)) + 1j * rng.standard_normal((B, N, DX, DY))).astype(np.complex64)).to(cuda)

    def loss_of(y):
        return (y - target).abs().pow(2).sum()

    x = torch.from_numpy(x0).to(cuda).requires_grad_(True)
    w = torch.from_numpy(w0).to(cuda).requires_grad_(True)
    loss_of(torch.ops.turbofno_b200.spectral_conv2d(x, w)).backward()

    xr = torch.from_numpy(x0).to(cuda).requires_grad_(True)
    wr = torch.from_numpy(w0).to(cuda).requires_grad_(True)
    spec = torch.fft.fft2(xr, dim=(-2, -1))[..., :64, :64]
    yhat = torch.einsum("bkxy,kn->bnxy", spec, wr)
    padded = torch.nn.functional.pad(torch.view_as_real(yhat), (0, 0, 0, DY - 64, 0, DX - 64))
    loss_of(torch.fft.ifft2(torch.view_as_complex(padded.contiguous()), dim=(-2, -1))).backward()

    assert_close(x.grad.cpu().numpy(), xr.grad.cpu().numpy(), "grad_x (2D)")
    assert_close(w.grad.cpu().numpy(), wr.grad.cpu().numpy(), "grad_W (2D)")


@pytest.mark.gpu
def test_operators_with_per_mode_weights(cuda):
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    B, K, N, DY = 7, 16, 64, 256
    x, _ = oracle_np.make_inputs_1d(B, K, N, DY, seed=21)
    w = oracle_np.make_per_mode_weights(K, N, (64,))
    y = torch.ops.turbofno_b200.spectral_conv1d(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda))
    assert_close(y.cpu().numpy(), oracle_np.spectral_conv_1d(x, w), "torch op 1d, per-mode weights")

    B, K, N, DX, DY = 2, 8, 64, 128, 256
    x, _ = oracle_np.make_inputs_2d(B, K, N, DX, DY, seed=22)
    w = oracle_np.make_per_mode_weights(K, N, (64, 64))
    for centered in (False, True):
        y = torch.ops.turbofno_b200.spectral_conv2d(torch.from_numpy(x).to(cuda), torch.from_numpy(w).to(cuda), centered)
        assert_close(y.cpu().numpy(), oracle_np.spectral_conv_2d(x, w, x_modes_centered=centered),
                     "torch op 2d, per-mode weights, centered=%s" % centered)


def _fno_layer_through_torch_fft(x, w):
    """rfft2 -> keep kx = -32..31, ky = 0..63 -> per-mode weights -> irfft2, the way FNO code writes it."""
    import torch

    B, K, DX, DY = x.shape
    N = w.shape[1]
    kx = torch.arange(-32, 32, device=x.device) % DX
    spec = torch.fft.rfft2(x, dim=(-2, -1))[:, :, kx, :64]
    out = torch.einsum("bkxy,knxy->bnxy", spec, w)
    full = torch.zeros((B, N, DX, DY // 2 + 1), dtype=torch.complex64, device=x.device)
    full[:, :, kx, :64] = out
    # irfft2 spelled out: complex inverse along X, real inverse along Y.  Run on the CPU: free weights
    # leave a complex value in the ky = 0 bin, whose imaginary part the real inverse drops there;
    # torch's CUDA backend returns something else for such input (measured: 6 % away).
    return torch.fft.irfft(torch.fft.ifft(full, dim=-2), n=DY, dim=-1)


@pytest.mark.gpu
@pytest.mark.parametrize("DX,DY", [(128, 256), (256, 128)])
def test_rfft_layer_of_a_real_field_matches_torch_fft(cuda, DX, DY):
    """Value and gradients of rfft_spectral_conv2d (complex kernels, ky = 0 column halved, twice the
    real part) against the rfft2 / irfft2 formulation under autograd."""
    import torch

    from turbofno_b200.torch_op import rfft_spectral_conv2d

    B, K, N = 2, 64, 64
    rng = np.random.default_rng(31)
    x0 = torch.from_numpy(rng.uniform(-1, 1, (B, K, DX, DY)).astype(np.float32))
    w0 = torch.from_numpy(oracle_np.make_per_mode_weights(K, N, (64, 64)))
    target = torch.from_numpy(rng.standard_normal((B, N, DX, DY)).astype(np.float32))

    x, w = x0.to(cuda).requires_grad_(True), w0.to(cuda).requires_grad_(True)
    y = rfft_spectral_conv2d(x, w)
    (y - target.to(cuda)).pow(2).sum().backward()
    xr, wr = x0.clone().requires_grad_(True), w0.clone().requires_grad_(True)      # reference on the CPU
    yr = _fno_layer_through_torch_fft(xr, wr)
    (yr - target).pow(2).sum().backward()

    assert y.dtype == torch.float32 and tuple(y.shape) == (B, N, DX, DY)
    assert_close(y.detach().cpu().numpy(), yr.detach().cpu().numpy(), "rfft layer")
    assert_close(x.grad.cpu().numpy(), xr.grad.cpu().numpy(), "rfft layer grad_x")
    assert_close(w.grad.cpu().numpy(), wr.grad.cpu().numpy(), "rfft layer grad_W")


@pytest.mark.gpu
def test_per_mode_gradients_match_autograd_through_torch_fft(cuda):
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    B, K, N, DY = 5, 64, 64, 256
    x0, _ = oracle_np.make_inputs_1d(B, K, N, DY, seed=41)
    w0 = oracle_np.make_per_mode_weights(K, N, (64,))
    rng = np.random.default_rng(42)
    target = torch.from_numpy((rng.standard_normal((B, N, DY)) + 1j * rng.standard_normal((B, N, DY))).astype(np.complex64)).to(cuda)
    x = torch.from_numpy(x0).to(cuda).requires_grad_(True)
    w = torch.from_numpy(w0).to(cuda).requires_grad_(True)
    (torch.ops.turbofno_b200.spectral_conv1d(x, w) - target).abs().pow(2).sum().backward()
    xr = torch.from_numpy(x0).to(cuda).requires_grad_(True)
    wr = torch.from_numpy(w0).to(cuda).requires_grad_(True)
    yhat = torch.einsum("bkm,knm->bnm", torch.fft.fft(xr, dim=-1)[..., :64], wr)
    padded = torch.cat([yhat, torch.zeros((B, N, DY - 64), dtype=torch.complex64, device=cuda)], dim=-1)
    (torch.fft.ifft(padded, dim=-1) - target).abs().pow(2).sum().backward()
    assert_close(x.grad.cpu().numpy(), xr.grad.cpu().numpy(), "per-mode grad_x")
    assert_close(w.grad.cpu().numpy(), wr.grad.cpu().numpy(), "per-mode grad_W")

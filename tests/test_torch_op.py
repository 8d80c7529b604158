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


def test_operator_has_no_cpu_kernel():
    import torch

    import turbofno_b200.torch_op  # noqa: F401

    x = torch.zeros((1, 8, 128), dtype=torch.complex64)
    w = torch.zeros((8, 64), dtype=torch.complex64)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.turbofno_b200.spectral_conv1d(x, w)           # the path has no CPU implementation


@pytest.mark.gpu
@pytest.mark.parametrize("B,K,N,DY", [(5, 16, 64, 256), (3, 8, 128, 128), (150, 64, 64, 256)])
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

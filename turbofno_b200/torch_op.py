"""PyTorch operators `torch.ops.turbofno_b200.spectral_conv1d / spectral_conv2d` over the C ABI.

For callers that hold activations the PyTorch way, batch first:

    spectral_conv1d(x[B, K, DY], w[K, N]) -> y[B, N, DY]
    spectral_conv2d(x[B, K, DX, DY], w[K, N]) -> y[B, N, DX, DY]

complex64, CUDA, contiguous; 64 kept modes per transformed axis (the corner block in 2D), weights
shared by all modes, unnormalised forward and 1/DY (1/(DX*DY)) inverse transform -- the layer the
reference's fully fused variant D computes (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/,
fusion_variants/2D_D_exp_fused_fft_cgemm_ifft/), which has no framework binding of its own.

The operators are registered with torch.library, so they carry a shape function for tracing and
export; they run on the caller's current stream and allocate only their output and, in 2D, the
plan's workspace through the caching allocator.  Inference only: no autograd formula is
registered.  Plans are cached per (shape, device).
"""
import torch

from . import api

_plans = {}


def _plan(rank, bs, DY, K, N, DX, device):
    key = (rank, bs, DY, K, N, DX, device)
    plan = _plans.get(key)
    if plan is None:
        plan = api.SpectralConv(rank, bs, DY, K, N, DX=DX, variant="D", layout="batch_major", device=device)
        _plans[key] = plan
    return plan


def _check(x, w, rank):
    if x.dtype != torch.complex64 or w.dtype != torch.complex64:
        raise TypeError("spectral_conv%dd: x and w must be complex64" % rank)
    if x.dim() != rank + 2 or w.dim() != 2 or w.shape[0] != x.shape[1]:
        raise ValueError("spectral_conv%dd: expected x[B, K%s, DY] and w[K, N]" % (rank, ", DX" if rank == 2 else ""))


@torch.library.custom_op("turbofno_b200::spectral_conv1d", mutates_args=(), device_types="cuda")
def spectral_conv1d(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    _check(x, w, 1)
    x, w = x.contiguous(), w.contiguous()
    B, K, DY = x.shape
    N = w.shape[1]
    plan = _plan(1, B, DY, K, N, None, x.device.index)
    y = torch.empty((B, N, DY), dtype=torch.complex64, device=x.device)
    plan(x, w, y=y)
    return y


@spectral_conv1d.register_fake
def _(x, w):
    _check(x, w, 1)
    return x.new_empty((x.shape[0], w.shape[1], x.shape[2]))


@torch.library.custom_op("turbofno_b200::spectral_conv2d", mutates_args=(), device_types="cuda")
def spectral_conv2d(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    _check(x, w, 2)
    x, w = x.contiguous(), w.contiguous()
    B, K, DX, DY = x.shape
    N = w.shape[1]
    plan = _plan(2, B, DY, K, N, DX, x.device.index)
    y = torch.empty((B, N, DX, DY), dtype=torch.complex64, device=x.device)
    plan(x, w, y=y)
    return y


@spectral_conv2d.register_fake
def _(x, w):
    _check(x, w, 2)
    return x.new_empty((x.shape[0], w.shape[1], x.shape[2], x.shape[3]))

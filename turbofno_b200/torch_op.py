"""PyTorch operators `torch.ops.turbofno_b200.spectral_conv1d / spectral_conv2d` over the C ABI.

For callers that hold activations the PyTorch way, batch first:

    spectral_conv1d(x[B, K, DY], w[K, N]) -> y[B, N, DY]
    spectral_conv2d(x[B, K, DX, DY], w[K, N], x_modes_centered=False) -> y[B, N, DX, DY]

complex64, CUDA, contiguous; 64 kept modes per transformed axis (the corner block in 2D), weights
shared by all modes, unnormalised forward and 1/DY (1/(DX*DY)) inverse transform -- the layer the
reference's fully fused variant D computes (fusion_variants/1D_D_exp_fused_fft_cgemm_ifft/,
fusion_variants/2D_D_exp_fused_fft_cgemm_ifft/), which has no framework binding of its own.

Beyond the reference, for callers that train an FNO:

  * per-mode weights: w[K, N, 64] (1D) or w[K, N, 64, 64] (2D), one K x N matrix per kept mode;
  * x_modes_centered (2D): X index i of the kept block is frequency i - 32, i.e. both low-frequency
    blocks of the non-last axis (rows 32..63 are what FNO code calls weights1, kx = 0..31; rows
    0..31 are weights2, kx = -32..-1);
  * rfft_spectral_conv2d(x_real, w): the rfft2 -> weights -> irfft2 layer of a real-valued field,
    computed through the complex kernels (see the function).

The operators are registered with torch.library, so they carry a shape function for tracing and
export; they run on the caller's current stream and allocate only their output and, in 2D, the
plan's workspace through the caching allocator.  Plans are cached per (shape, device).

Both operators have an autograd formula built from the same kernels: the layer is
y = A(x) W with A = (1/DY) F^H P F (P keeps 64 modes), A is self-adjoint, so
grad_x = spectral_conv1d(grad_y, W^H) -- which needs the kernel's shape limits for the swapped
channel counts (K a multiple of 64, N a multiple of 8) -- and grad_W = X^H G / DY per mode, summed
over the batch and (for weights shared by all modes) over the modes, with X, G the truncated spectra of x and grad_y from the stand-alone
transform kernels (tfno_fft_stride_DY; in 2D tfno_fft_stride along X first).  The same holds for
spectral_conv2d with 1/(DX*DY).
"""
import torch

from . import api

_plans = {}


def _plan(rank, bs, DY, K, N, DX, device, per_mode=False, centered=False):
    key = (rank, bs, DY, K, N, DX, device, per_mode, centered)
    plan = _plans.get(key)
    if plan is None:
        plan = api.SpectralConv(rank, bs, DY, K, N, DX=DX, variant="D", layout="batch_major", device=device,
                                per_mode_weights=per_mode, x_modes_centered=centered)
        _plans[key] = plan
    return plan


def _check(x, w, rank):
    """Returns True when w carries one matrix per mode."""
    if x.dtype != torch.complex64 or w.dtype != torch.complex64:
        raise TypeError("spectral_conv%dd: x and w must be complex64" % rank)
    per_mode = w.dim() == 2 + rank
    if x.dim() != rank + 2 or not (w.dim() == 2 or per_mode) or w.shape[0] != x.shape[1] or \
            (per_mode and tuple(w.shape[2:]) != (64,) * rank):
        raise ValueError("spectral_conv%dd: expected x[B, K%s, DY] and w[K, N] or w[K, N%s]" %
                         (rank, ", DX" if rank == 2 else "", ", 64" * rank))
    return per_mode


@torch.library.custom_op("turbofno_b200::spectral_conv1d", mutates_args=(), device_types="cuda")
def spectral_conv1d(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    per_mode = _check(x, w, 1)
    x, w = x.contiguous(), w.contiguous()
    B, K, DY = x.shape
    N = w.shape[1]
    plan = _plan(1, B, DY, K, N, None, x.device.index, per_mode)
    y = torch.empty((B, N, DY), dtype=torch.complex64, device=x.device)
    plan(x, w, y=y)
    return y


@spectral_conv1d.register_fake
def _(x, w):
    _check(x, w, 1)
    return x.new_empty((x.shape[0], w.shape[1], x.shape[2]))


@torch.library.custom_op("turbofno_b200::spectral_conv2d", mutates_args=(), device_types="cuda")
def spectral_conv2d(x: torch.Tensor, w: torch.Tensor, x_modes_centered: bool = False) -> torch.Tensor:
    per_mode = _check(x, w, 2)
    x, w = x.contiguous(), w.contiguous()
    B, K, DX, DY = x.shape
    N = w.shape[1]
    plan = _plan(2, B, DY, K, N, DX, x.device.index, per_mode, bool(x_modes_centered))
    y = torch.empty((B, N, DX, DY), dtype=torch.complex64, device=x.device)
    plan(x, w, y=y)
    return y


@spectral_conv2d.register_fake
def _(x, w, x_modes_centered=False):
    _check(x, w, 2)
    return x.new_empty((x.shape[0], w.shape[1], x.shape[2], x.shape[3]))


def _truncated_spectrum(t):
    """[B, C, DY] -> [B, C, 64]: forward transform of every signal, first 64 modes (tfno_fft_stride_DY)."""
    B, C, DY = t.shape
    out = torch.empty((B, C, 64), dtype=torch.complex64, device=t.device)
    api.fft_stride_DY(t.contiguous(), out, B * C, DY)
    return out


def _conv1d_setup_context(ctx, inputs, output):
    x, w = inputs
    ctx.save_for_backward(x, w)


def _conv2d_setup_context(ctx, inputs, output):
    x, w, centered = inputs
    ctx.save_for_backward(x, w)
    ctx.centered = bool(centered)


def _conv1d_backward(ctx, grad_y):
    x, w = ctx.saved_tensors
    grad_x = grad_w = None
    grad_y = grad_y.contiguous()
    if ctx.needs_input_grad[0]:
        grad_x = spectral_conv1d(grad_y, w.conj().transpose(0, 1).contiguous())
    if ctx.needs_input_grad[1]:
        X, G = _truncated_spectrum(x), _truncated_spectrum(grad_y)
        grad_w = torch.einsum("bkm,bnm->knm" if w.dim() == 3 else "bkm,bnm->kn", X.conj(), G) / x.shape[2]
    return grad_x, grad_w


spectral_conv1d.register_autograd(_conv1d_backward, setup_context=_conv1d_setup_context)


def _truncated_spectrum2d(t, centered=False):
    """[B, C, DX, DY] -> [B, C, 64, 64]: X transform keeping 64 modes (tfno_fft_stride), then Y.
    Centered X modes are the first 64 modes of the field multiplied by exp(2 pi i 32 x / DX)."""
    B, C, DX, DY = t.shape
    if centered:
        turns = (torch.arange(DX, device=t.device) * 32 % DX).to(torch.float64) / DX      # reduced before the sine
        phase = torch.polar(torch.ones(DX, dtype=torch.float64, device=t.device), 2 * torch.pi * turns)
        t = t * phase.to(torch.complex64)[:, None]
    tx = torch.empty((B, C, 64, DY), dtype=torch.complex64, device=t.device)
    api.fft_stride(t.contiguous(), tx, DY, B * C * DY, DX)
    out = torch.empty((B, C, 64, 64), dtype=torch.complex64, device=t.device)
    api.fft_stride_DY(tx, out, B * C * 64, DY)
    return out


def _conv2d_backward(ctx, grad_y):
    x, w = ctx.saved_tensors
    grad_x = grad_w = None
    grad_y = grad_y.contiguous()
    if ctx.needs_input_grad[0]:
        grad_x = spectral_conv2d(grad_y, w.conj().transpose(0, 1).contiguous(), ctx.centered)
    if ctx.needs_input_grad[1]:
        X, G = _truncated_spectrum2d(x, ctx.centered), _truncated_spectrum2d(grad_y, ctx.centered)
        grad_w = torch.einsum("bkxy,bnxy->knxy" if w.dim() == 4 else "bkxy,bnxy->kn", X.conj(), G) / (x.shape[2] * x.shape[3])
    return grad_x, grad_w, None


spectral_conv2d.register_autograd(_conv2d_backward, setup_context=_conv2d_setup_context)


def rfft_spectral_conv2d(x, w):
    """The spectral layer of a real-valued field as FNO code writes it,

        irfft2(pad(einsum("bkxy,knxy->bnxy", rfft2(x)[:, :, kx, :64], w)), s=(DX, DY)),  kx = -32..31,

    for real x[B, K, DX, DY] (float32) and per-mode weights w[K, N, 64, 64] (complex64, X index i is
    frequency i - 32), through spectral_conv2d: the complex transform of a real field carries the
    same 64 non-negative Y modes, and the real inverse transform of a half spectrum Z is
    2 Re(ifft2(Z')) with Z' = Z except for the ky = 0 column, which enters once and is halved.
    irfft2 here means the complex inverse along X followed by a real inverse along Y that drops the
    imaginary part of the ky = 0 bin (torch on the CPU); free weights leave a complex value there,
    for which torch's CUDA backend returns something else.
    Differentiable in x and w.  The complex kernels move twice the bytes a real-input kernel would;
    real-input (R2C / C2R) kernels are not built."""
    if x.is_complex() or w.dim() != 4:
        raise ValueError("rfft_spectral_conv2d: expected real x[B, K, DX, DY] and w[K, N, 64, 64]")
    half = torch.ones(64, dtype=torch.float32, device=w.device)
    half[0] = 0.5
    xc = torch.complex(x.to(torch.float32), torch.zeros_like(x, dtype=torch.float32))
    return 2.0 * spectral_conv2d(xc, w * half, True).real
